"""The checkpoint -> Q4 bank loader on the host: safetensors headers, config.json, part checks,
row concatenation, scale/bias interleave and the non-finite refusal. No device, no oracle.

Cases follow tests/qwen35_mlx_q4_layout.rs and the host-checkable parts of
tests/qwen35_mlx_q4.rs:505-657, 1097-1170 of the reference project.
"""
import json
import struct

import numpy as np
import pytest

from tessl_b200 import capi, loader, synth
from tests import mlx_checkpoint as mc

NAME = mc.PREFIX + ".mlp.gate_proj.weight"


def quant(body):
    return '{"model_type": "qwen3_5", %s}' % body


def refused(fn, *a):
    with pytest.raises(capi.TesslError) as e:
        fn(*a)
    assert e.value.status == capi.TESSL_ERR
    return str(e.value)


@pytest.fixture()
def ckpt(tmp_path):
    ents, banks = mc.entries()
    path = mc.write(tmp_path / "model.safetensors", ents, metadata={"format": "mlx"})
    with loader.Checkpoint(path) as c:
        yield c, banks


# ------------------------------------------------------------- config.json ---

def test_the_converters_quantization_block_is_accepted_in_either_spelling():
    q = '{"group_size": 64, "bits": 4, "mode": "affine"}'
    both = quant(f'"quantization": {q}, "quantization_config": {q}')
    assert loader.MlxQuant.from_config_json(both) == loader.MlxQuant(4, 64)
    for body in (f'"quantization": {q}', f'"quantization_config": {q}', '"quantization": {"group_size": 64, "bits": 4}'):
        assert loader.MlxQuant.from_config_json(quant(body)) == loader.MlxQuant(loader.MLX_Q4_BITS, loader.MLX_Q4_GROUP)


@pytest.mark.parametrize("body,needle", [
    ('"quantization": {"group_size": 64, "bits": 8}', "quantization.bits is 8"),
    ('"quantization": {"group_size": 32, "bits": 4}', "quantization.group_size is 32"),
    ('"quantization": {"group_size": 128, "bits": 4, "mode": "affine"}', "quantization.group_size is 128"),
    ('"quantization": {"group_size": 32, "bits": 4, "mode": "mxfp4"}', 'mode is "mxfp4"'),
    ('"hidden_size": 8', "not an MLX-quantized"),
])
def test_other_bits_groups_and_modes_are_refused_by_name(body, needle):
    assert needle in refused(loader.MlxQuant.from_config_json, quant(body))


def test_per_layer_overrides_are_a_mixed_checkpoint_and_refused():
    e = refused(loader.MlxQuant.from_config_json, quant(
        '"quantization": {"group_size": 64, "bits": 4, '
        '"language_model.model.layers.0.mlp.gate": {"group_size": 64, "bits": 8}, '
        '"language_model.model.embed_tokens": false}'))
    assert '"language_model.model.layers.0.mlp.gate", "language_model.model.embed_tokens"' in e
    assert "mixed-precision" in e


@pytest.mark.parametrize("body", [
    '"quantization": 4',
    '"quantization": {"group_size": 64, "bits": "4"}',
    '"quantization": {"group_size": 64}',
    '"quantization": {"group_size": 64, "bits": 4.5}',
    '"quantization": {"group_size": 64, "bits": -4}',
    '"quantization": {"group_size": 64, "bits": 4, "mode": 3}',
    '"quantization": {"group_size": 64, "bits": 4}, "quantization_config": {"group_size": 64, "bits": 8}',
])
def test_malformed_quantization_blocks_are_refused(body):
    assert refused(loader.MlxQuant.from_config_json, quant(body)).startswith("config.json: quantization")


@pytest.mark.parametrize("text", ["[]", "", "{", '{"quantization": {"bits": 4,}}', '{"a": 1} x', '{"a": 1, "a": 2}'])
def test_text_that_is_not_a_json_object_is_refused(text):
    assert "config.json" in refused(loader.MlxQuant.from_config_json, text)


# ------------------------------------------------------ safetensors header ---

def test_header_facts_are_reported_without_reading_data(ckpt):
    c, _ = ckpt
    names = c.names()
    assert len(names) == 3 * len(mc.LAYER) + 1 and NAME in names and "__metadata__" not in names
    assert c.tensor_info(NAME) == loader.TensorInfo("U32", (192, 16), 192 * 16 * 4)
    assert c.tensor_info(mc.PREFIX + ".mlp.gate_proj.scales") == loader.TensorInfo("BF16", (192, 2), 192 * 2 * 2)
    assert "no such tensor" in refused(c.tensor_info, "nope.weight")


def _raw(tmp_path, header_bytes, data=b"", declared=None):
    p = tmp_path / "bad.safetensors"
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(header_bytes) if declared is None else declared))
        f.write(header_bytes)
        f.write(data)
    return p


def test_malformed_files_are_refused_at_open(tmp_path):
    def opened(p):
        loader.Checkpoint(p).close()

    assert "cannot open" in refused(opened, tmp_path / "missing.safetensors")
    (tmp_path / "short").write_bytes(b"abc")
    assert "shorter than" in refused(opened, tmp_path / "short")
    assert "exceeds the file" in refused(opened, _raw(tmp_path, b"{}", declared=1 << 40))
    assert "header:" in refused(opened, _raw(tmp_path, b'{"a": '))
    assert "not a JSON object" in refused(opened, _raw(tmp_path, b"[1]"))
    ent = lambda **kw: json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8], **kw}}).encode()
    opened(_raw(tmp_path, ent(), b"\0" * 8))
    assert "exceed" in refused(opened, _raw(tmp_path, ent(), b"\0" * 4))
    assert "needs 8 bytes" in refused(opened, _raw(tmp_path, ent(data_offsets=[0, 4]), b"\0" * 8))
    assert "unknown dtype" in refused(opened, _raw(tmp_path, ent(dtype="Q4"), b"\0" * 8))
    assert "shape holds" in refused(opened, _raw(tmp_path, ent(shape=[-2]), b"\0" * 8))
    assert "shape holds" in refused(opened, _raw(tmp_path, ent(shape=[2.5]), b"\0" * 8))
    assert "malformed data_offsets" in refused(opened, _raw(tmp_path, ent(data_offsets=[8, 0]), b"\0" * 8))
    assert "overflows" in refused(opened, _raw(tmp_path, ent(shape=[1 << 40, 1 << 40]), b"\0" * 8))
    two = json.dumps({"a": {"dtype": "U8", "shape": [8], "data_offsets": [0, 8]},
                      "b": {"dtype": "U8", "shape": [8], "data_offsets": [4, 12]}}).encode()
    assert "overlap" in refused(opened, _raw(tmp_path, two, b"\0" * 12))
    assert "duplicate key" in refused(opened, _raw(tmp_path, b'{"a": {"dtype": "U8", "shape": [0], "data_offsets": [0, 0]}, '
                                                              b'"a": {"dtype": "U8", "shape": [0], "data_offsets": [0, 0]}}'))


# -------------------------------------------------------- tensor headers ---

def test_sidecars_are_named_after_the_weight():
    assert loader.sidecar_names(NAME) == (mc.PREFIX + ".mlp.gate_proj.scales", mc.PREFIX + ".mlp.gate_proj.biases")
    assert loader.sidecar_names("language_model.model.norm.scales") is None


def test_a_well_formed_part_is_accepted(ckpt):
    c, _ = ckpt
    for suffix, rows, cols in mc.LAYER:
        c.check_part(f"{mc.PREFIX}.{suffix}.weight", rows, cols)


def _variant(tmp_path, edit):
    ents, _ = mc.entries()
    ents = edit(ents)
    return loader.Checkpoint(mc.write(tmp_path / "variant.safetensors", ents))


def _replace(name, dtype, shape, data):
    return lambda ents: [(n, dtype, shape, data) if n == name else (n, d, s, b) for n, d, s, b in ents]


def test_part_refusals_name_the_tensor_and_the_reason(tmp_path, ckpt):
    c, _ = ckpt
    assert "[0, 128] matrix has nothing to load" in refused(c.check_part, NAME, 0, 128)
    assert "120 columns is not a multiple of the group size 64" in refused(c.check_part, NAME, 192, 120)
    # the rows the model expects must be the rows the file has
    e = refused(c.check_part, NAME, 384, 128)
    assert NAME in e and "shape [192, 16], expected [384, 16]" in e
    assert "no such tensor" in refused(c.check_part, mc.PREFIX + ".mlp.nope.weight", 8, 128)

    # a projection the converter left dense
    with _variant(tmp_path, _replace(NAME, "BF16", [192, 128], bytes(192 * 128 * 2))) as v:
        e = refused(v.check_part, NAME, 192, 128)
        assert NAME in e and "BF16" in e and "mixed" in e
    # 8-bit packs four values per word
    with _variant(tmp_path, _replace(NAME, "U32", [192, 32], bytes(192 * 32 * 4))) as v:
        e = refused(v.check_part, NAME, 192, 128)
        assert NAME in e and "other bits" in e
    # a missing sidecar, by which
    for side in ("scales", "biases"):
        gone = mc.PREFIX + ".mlp.gate_proj." + side
        with _variant(tmp_path, lambda ents: [x for x in ents if x[0] != gone]) as v:
            e = refused(v.check_part, NAME, 192, 128)
            assert NAME in e and f"no {side} tensor beside it" in e
    # group-32 scales, float16 biases
    sname, bname = loader.sidecar_names(NAME)
    with _variant(tmp_path, _replace(sname, "BF16", [192, 4], bytes(192 * 4 * 2))) as v:
        e = refused(v.check_part, NAME, 192, 128)
        assert e.startswith(sname) and "shape [192, 4], expected [192, 2]" in e
    with _variant(tmp_path, _replace(bname, "F16", [192, 2], bytes(192 * 2 * 2))) as v:
        e = refused(v.check_part, NAME, 192, 128)
        assert e.startswith(bname) and "dtype F16, expected BF16" in e


# ------------------------------------------------------------------ banks ---

def test_one_part_is_the_words_unchanged_and_the_pairs_interleaved(ckpt):
    c, banks = ckpt
    for suffix, rows, cols in mc.LAYER:
        packed, pairs = c.read_mlx_q4([(f"{mc.PREFIX}.{suffix}.weight", rows)], cols)
        want_p, want_sb = banks[suffix]
        assert packed.shape == (rows, cols // 8) and pairs.shape == (rows, cols // 64, 2)
        np.testing.assert_array_equal(packed, want_p)
        np.testing.assert_array_equal(pairs, want_sb)


@pytest.mark.parametrize("parts", [
    ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"),
    ("mlp.gate_proj", "mlp.up_proj"),
    ("self_attn.k_proj", "self_attn.v_proj"),
])
def test_parts_are_concatenated_by_rows_in_the_order_given(ckpt, parts):
    c, banks = ckpt
    dims = {s: (r, k) for s, r, k in mc.LAYER}
    packed, pairs = c.read_mlx_q4([(f"{mc.PREFIX}.{s}.weight", dims[s][0]) for s in parts], 128)
    np.testing.assert_array_equal(packed, np.concatenate([banks[s][0] for s in parts]))
    np.testing.assert_array_equal(pairs, np.concatenate([banks[s][1] for s in parts]))


def test_a_bad_part_is_refused_before_anything_is_written(ckpt):
    c, _ = ckpt
    lib = capi.load()
    import ctypes as C

    parts = [(mc.PREFIX + ".self_attn.q_proj.weight", 256), (mc.PREFIX + ".self_attn.k_proj.weight", 65)]
    names = (C.c_char_p * 2)(*[p[0].encode() for p in parts])
    rows = (C.c_uint64 * 2)(*[p[1] for p in parts])
    packed = np.full((321, 16), 0xA5A5A5A5, np.uint32)
    pairs = np.full((321, 2, 2), 0x5A5A, np.uint16)
    err = C.create_string_buffer(1024)
    st = lib.tessl_mlx_q4_read_bank(c._h, names, rows, 2, 128, packed.ctypes.data, packed.nbytes, pairs.ctypes.data,
                                    pairs.nbytes, err, 1024)
    assert st == capi.TESSL_ERR and b"k_proj.weight" in err.value and b"expected [65, 16]" in err.value
    assert (packed == 0xA5A5A5A5).all() and (pairs == 0x5A5A).all()
    # a buffer too small for the bank is refused too
    rows[1] = 64
    st = lib.tessl_mlx_q4_read_bank(c._h, names, rows, 2, 128, packed.ctypes.data, 100, pairs.ctypes.data, pairs.nbytes,
                                    err, 1024)
    assert st == capi.TESSL_ERR and b"the bank needs" in err.value
    assert "no parts" in refused(c.read_mlx_q4, [], 128)


@pytest.mark.parametrize("side,value,word", [("scales", np.nan, "NaN"), ("scales", np.inf, "inf"), ("biases", -np.inf, "-inf")])
def test_non_finite_scales_and_biases_are_refused_by_tensor_row_and_group(tmp_path, side, value, word):
    target = f"{mc.PREFIX}.mlp.up_proj.{side}"
    element = 2 * 77 + 1  # row 77, group 1

    def poison(ents):
        out = []
        for n, d, s, b in ents:
            if n == target:
                a = np.frombuffer(b, np.uint16).copy()
                a[element] = synth.f32_to_bf16_bits(np.array([value], np.float32))[0]
                b = a.tobytes()
            out.append((n, d, s, b))
        return out

    with _variant(tmp_path, poison) as v:
        e = refused(v.read_mlx_q4, [(mc.PREFIX + ".mlp.gate_proj.weight", 192), (mc.PREFIX + ".mlp.up_proj.weight", 192)], 128)
    assert e == f"{target}: element {element} (row 77, group 1) is {word}, not finite"


def test_a_huge_config_over_a_tiny_file_is_refused_from_the_header(ckpt):
    # the caller's dimensions are as untrusted as the file: nothing is sized from them before the header agrees
    c, _ = ckpt
    e = refused(c.check_part, NAME, 1 << 22, 1 << 20)
    assert "expected [4194304, 131072]" in e


def test_the_largest_bf16_finite_values_load(tmp_path):
    big = synth.f32_to_bf16_bits(np.array([3.3895314e38, -3.3895314e38], np.float32))
    sname = mc.PREFIX + ".self_attn.k_proj.scales"

    def edit(ents):
        out = []
        for n, d, s, b in ents:
            if n == sname:
                a = np.frombuffer(b, np.uint16).copy()
                a[:2] = big
                b = a.tobytes()
            out.append((n, d, s, b))
        return out

    with _variant(tmp_path, edit) as v:
        _, pairs = v.read_mlx_q4([(mc.PREFIX + ".self_attn.k_proj.weight", 64)], 128)
    assert pairs[0, 0, 0] == big[0] and pairs[0, 1, 0] == big[1]


# ------------------------------------------------- names and conventions ---
# tests/qwen35_mlx_q4_layout.rs:212-330 of the reference project

def test_the_key_spelling_is_detected_and_ambiguity_refused():
    mlx = ["language_model.model.embed_tokens.weight", "language_model.lm_head.weight"]
    assert loader.MlxNames.detect(mlx) == loader.MlxNames("language_model.model.", "language_model.lm_head")
    hf = ["model.language_model.embed_tokens.weight", "lm_head.weight"]
    assert loader.MlxNames.detect(hf) == loader.MlxNames("model.language_model.", "lm_head")
    assert "not a Qwen3.5 checkpoint" in refused(loader.MlxNames.detect, ["model.visual.x"])
    assert "not a Qwen3.5 checkpoint" in refused(loader.MlxNames.detect, [])
    e = refused(loader.MlxNames.detect, [mlx[0], hf[0]])
    assert e.startswith("checkpoint conventions:") and "both" in e


def test_the_conv_layout_says_which_norm_convention_the_checkpoint_is_in():
    c, k = 6144, 4
    NC = loader.NormConvention
    assert NC.from_conv_shape("conv", [c, 1, k], c, k) == NC.HF
    assert NC.from_conv_shape("conv", [c, k, 1], c, k) == NC.MLX_SHIFTED
    e = refused(NC.from_conv_shape, "conv", [c, 2, 2], c, k)
    assert e.startswith("conv: shape [6144, 2, 2], expected [6144, 1, 4]")
    assert "shape [6144, 4]" in refused(NC.from_conv_shape, "conv", [c, k], c, k)
    # the kernels add 1 themselves, so the shifted convention is undone, and exactly: a bf16 value near 1 minus 1 is
    # exact in f32, and adding the 1 back gives the stored value again bit for bit
    for stored in (0.0, 0.5, 1.0, 1.0078125, 1.75, 2.5, 33.0, -0.25, 0.00390625):
        w = NC.unshift(NC.MLX_SHIFTED, stored)
        assert (np.float32(1.0) + w).view(np.uint32) == np.float32(stored).view(np.uint32), stored
        assert NC.unshift(NC.HF, stored).view(np.uint32) == np.float32(stored).view(np.uint32)
    assert NC.conv_shape(NC.MLX_SHIFTED, c, k) == (c, k, 1) and NC.conv_shape(NC.HF, c, k) == (c, 1, k)


def test_mtp_and_vision_tensors_are_skipped_by_name_and_counted():
    unread = ["mtp.fc.weight", "mtp.layers.0.mlp.down_proj.weight", "mtp.norm.weight",
              "model.visual.blocks.0.attn.qkv.weight", "model.visual.blocks.1.attn.qkv.weight", "vision_tower.merger.weight"]
    assert loader.classify_outside(unread) == {"mtp": unread[:3], "vision": unread[3:]}
    assert loader.classify_outside([]) == {"mtp": [], "vision": []}


def test_any_other_tensor_outside_the_tower_is_refused():
    e = refused(loader.classify_outside, ["mtp.fc.weight", "lm_head.bias", "audio_tower.x"])
    assert e.startswith("2 tensor(s) outside the tower") and '["lm_head.bias", "audio_tower.x"]' in e
    many = [f"stray.{i}" for i in range(11)]
    e = refused(loader.classify_outside, many)
    assert e.startswith("11 tensor(s)") and '"stray.7"' in e and '"stray.8"' not in e


def test_a_drafter_checkpoint_without_a_tower_prefix_is_not_mistaken_for_a_tower():
    # unprefixed names such as a stand-alone multi-token-prediction drafter carries: fails closed
    names = ["fc.biases", "fc.scales", "fc.weight", "layers.0.mlp.down_proj.weight", "norm.weight", "pre_fc_norm_hidden.weight"]
    assert "not a Qwen3.5 checkpoint" in refused(loader.MlxNames.detect, names)
