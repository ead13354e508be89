"""Checkpoint -> device bank -> projection: the loader's device leg and the operators that read its banks."""
import numpy as np
import pytest

from oracle import api
from tessl_b200 import capi, loader, nn, synth
from tests import mlx_checkpoint as mc
from tests.gpu_util import assert_north_star, rt, seeded_f32  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ckpt(tmp_path):
    ents, banks = mc.entries(seed=23)
    with loader.Checkpoint(mc.write(tmp_path / "model.safetensors", ents)) as c:
        yield c, banks


def test_a_loaded_bank_holds_the_files_words_and_pairs(rt, ckpt):
    c, banks = ckpt
    bank = c.mlx_q4(rt, mc.PREFIX, [("self_attn.q_proj", 256), ("self_attn.k_proj", 64), ("self_attn.v_proj", 64)], 128)
    want_p = np.concatenate([banks[s][0] for s in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")])
    want_sb = np.concatenate([banks[s][1] for s in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")])
    np.testing.assert_array_equal(bank.packed.read(np.uint32, want_p.size).reshape(want_p.shape), want_p)
    np.testing.assert_array_equal(bank.scales_biases.read(np.uint16, want_sb.size).reshape(want_sb.shape), want_sb)


def test_a_gate_up_bank_from_the_file_drives_the_fused_projection(rt, ckpt):
    c, banks = ckpt
    rows, cols = 192, 128
    both = c.mlx_q4(rt, mc.PREFIX, [("mlp.gate_proj", rows), ("mlp.up_proj", rows)], cols)
    x = synth.normal_bf16(5, cols)
    xb = rt.buffer_from(x)
    # one GEMV over [gate; up] equals the file's two matrices applied separately
    y = seeded_f32(rt, 2 * rows)
    nn.gemv_q4_mlx_simd(rt, both, xb, y, nn.QuantShape(2 * rows, cols, 64))
    got = y.read(np.float32, 2 * rows)
    for i, s in enumerate(("mlp.gate_proj", "mlp.up_proj")):
        want = api.q4_dense_gemm(banks[s][0].view(np.uint8).reshape(-1), banks[s][1].reshape(-1), x, 1, rows, cols, 64)[0]
        assert_north_star(got[i * rows:(i + 1) * rows], want, s)
    # and the loaded halves, viewed as two banks, feed gate_up_silu
    gate = nn.Q4MlxBank(both.packed.view(0, rows * cols // 2), both.scales_biases.view(0, rows * (cols // 64) * 4))
    up = nn.Q4MlxBank(both.packed.view(rows * cols // 2, rows * cols // 2),
                      both.scales_biases.view(rows * (cols // 64) * 4, rows * (cols // 64) * 4))
    mid = seeded_f32(rt, rows)
    nn.gemv_q4_mlx_gate_up_silu(rt, gate, up, xb, mid, nn.QuantShape(rows, cols, 64), False)
    g, u = got[:rows].astype(np.float64), got[rows:].astype(np.float64)
    np.testing.assert_allclose(mid.read(np.float32, rows), g / (1 + np.exp(-g)) * u, rtol=1e-4, atol=1e-5)


def test_load_refusals_leave_the_runtime_usable(rt, ckpt):
    c, _ = ckpt
    with pytest.raises(capi.TesslError) as e:
        c.mlx_q4(rt, mc.PREFIX, [("mlp.gate_proj", 192), ("mlp.up_proj", 200)], 128)
    assert "up_proj.weight" in str(e.value) and not rt.is_poisoned()
    # a bank too small for the parts is refused by the library, not overrun
    small = nn.Q4MlxBank(rt.alloc_buffer(64), rt.alloc_buffer(64))
    import ctypes as C

    names = (C.c_char_p * 1)((mc.PREFIX + ".mlp.gate_proj.weight").encode())
    rows = (C.c_uint64 * 1)(192)
    with pytest.raises(capi.TesslError) as e:
        capi.call("tessl_mlx_q4_load_bank", rt.handle, c._h, names, rows, 1, 128, small.c())
    assert "packed" in str(e.value) and not rt.is_poisoned()
    c.mlx_q4(rt, mc.PREFIX, [("mlp.down_proj", 128)], 192)
