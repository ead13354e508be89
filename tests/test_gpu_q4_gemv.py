"""GPU parity of the MLX Q4 GEMV family against the CPU oracle, through the C ABI.

Mirrors the reference's own numeric tests for these entries
(tests/nn_wiring.rs:449-600, tests/promoted_numeric.rs:49-260,
tests/q4_kernels_template.rs, tests/qwen35_decode_fusion.rs:357-420 in the
reference project): every epilogue, odd row counts, K tails that leave lanes
idle, fused == unfused bit for bit, sentinel tails, refusals before any launch.
"""
import numpy as np
import pytest

import ref_cases as rc
from gpu_util import SENTINEL_F32, assert_gamma_bound, assert_north_star, bf16_round, rt, seeded_f32, upload_bank  # noqa: F401
from oracle import api
from tessl_b200 import nn, synth

pytestmark = pytest.mark.gpu

REF_SHAPES = [(r, k, g) for _, r, k, g in rc.SHAPES]
MODEL_SHAPES = [(4096, 4096, 64), (6144, 4096, 64), (4096, 12288, 64), (1000, 2048, 128), (257, 4096, 32),
                (12288, 4096, 64), (96, 1024, 512), (64, 512, 256),
                # eight or more stages per SM: the producer fetches four rows per copy; ragged last block
                (19001, 4096, 64), (19030, 1024, 128)]


def make_case(rows, cols, group, seed):
    packed, sb = synth.q4_bank(seed, rows, cols, group)
    x = synth.normal_bf16(seed + 7, cols)
    return packed.view(np.uint8).reshape(-1), sb.reshape(-1), x


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES + MODEL_SHAPES)
def test_nibbles_and_dequantized_weights_are_bit_exact(rt, rows, cols, group):
    packed, sb, _ = make_case(rows, cols, group, 0x7E550000 + rows)
    bank = upload_bank(rt, packed, sb)
    shape = nn.QuantShape(rows, cols, group)
    out_u8 = rt.alloc_buffer(rows * cols)
    nn.q4_mlx_unpack(rt, bank, shape, out_u8)
    assert np.array_equal(out_u8.read(np.uint8, rows * cols), api.q4_unpack(packed, rows * cols))
    out_f32 = rt.alloc_buffer(rows * cols * 4)
    nn.q4_mlx_dequant(rt, bank, shape, out_f32)
    got = out_f32.read(np.uint32, rows * cols)
    want = api.q4_dequant(packed, sb, rows, cols, group).view(np.uint32).reshape(-1)
    assert np.array_equal(got, want)
    for b in (out_u8, out_f32, bank.packed, bank.scales_biases):
        b.free()


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES + MODEL_SHAPES)
def test_gemv_matches_the_dequant_matvec(rt, rows, cols, group):
    packed, sb, x = make_case(rows, cols, group, 0x7E550010 + rows + cols)
    bank = upload_bank(rt, packed, sb)
    xb = rt.buffer_from(x)
    pad = 8
    y = seeded_f32(rt, rows, pad)
    shape = nn.QuantShape(rows, cols, group)
    nn.gemv_q4_mlx_simd(rt, bank, xb, y, shape)
    got = y.read(np.float32, rows + pad)
    assert np.all(got[rows:] == SENTINEL_F32), "wrote past y"
    got = got[:rows]
    want = api.q4_dense_gemm(packed, sb, x, 1, rows, cols, group)[0]
    assert_north_star(got, want, "gemv f32")
    assert_gamma_bound(got, packed, sb, x, 1, rows, cols, group, what="gemv")
    # the reference kernel's own summation order, emulated: same sum, other order
    emu = api.q4_simd_gemv(packed, sb, x, rows, cols, group).view(np.float32)
    np.testing.assert_allclose(got, emu, rtol=2e-4, atol=2e-4)
    # bf16-output twin == round-to-nearest-even of the f32 result, bit for bit
    yb = rt.buffer_from(np.full(rows + pad, 0xA5A5, np.uint16))
    nn.gemv_q4_mlx_simd(rt, bank, xb, yb, shape, y_as_bf16=True)
    gb = yb.read(np.uint16, rows + pad)
    assert np.all(gb[rows:] == 0xA5A5)
    assert np.array_equal(gb[:rows], synth.f32_to_bf16_bits(got))


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES + [(4096, 4096, 64)])
def test_add_resid_and_the_y_is_resid_alias(rt, rows, cols, group):
    packed, sb, x = make_case(rows, cols, group, 0x7E550020 + rows)
    bank = upload_bank(rt, packed, sb)
    xb = rt.buffer_from(x)
    shape = nn.QuantShape(rows, cols, group)
    resid = rc.rand_f32(rows, 0x4200 + rows)
    y0 = seeded_f32(rt, rows)
    nn.gemv_q4_mlx_simd(rt, bank, xb, y0, shape)
    plain = y0.read(np.float32, rows)
    r = rt.buffer_from(resid)
    y1 = seeded_f32(rt, rows)
    nn.gemv_q4_mlx_simd(rt, bank, xb, y1, shape, resid=r)
    assert np.array_equal(y1.read(np.float32, rows), plain + resid)  # one f32 add
    nn.gemv_q4_mlx_simd(rt, bank, xb, r, shape, resid=r)  # tests/nn_aliasing.rs:290: the allowed alias
    assert np.array_equal(r.read(np.float32, rows), plain + resid)


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES + [(12288, 4096, 64)])
@pytest.mark.parametrize("mid_bf16", [False, True])
def test_gate_up_silu_is_two_gemvs_and_swiglu_bit_for_bit(rt, rows, cols, group, mid_bf16):
    gp, gs, x = make_case(rows, cols, group, 0x7E550030 + rows)
    up, us, _ = make_case(rows, cols, group, 0x7E550040 + rows)
    gate, upb = upload_bank(rt, gp, gs), upload_bank(rt, up, us)
    xb = rt.buffer_from(x)
    shape = nn.QuantShape(rows, cols, group)
    esz = 2 if mid_bf16 else 4
    mid = rt.buffer_from(np.full((rows + 8) * esz, 0xA5, np.uint8))
    nn.gemv_q4_mlx_gate_up_silu(rt, gate, upb, xb, mid, shape, mid_bf16)
    fused = mid.read(np.uint8, (rows + 8) * esz)
    assert np.all(fused[rows * esz:] == 0xA5), "wrote past mid"
    g, u = seeded_f32(rt, rows), seeded_f32(rt, rows)
    nn.gemv_q4_mlx_simd(rt, gate, xb, g, shape)
    nn.gemv_q4_mlx_simd(rt, upb, xb, u, shape)
    out = rt.buffer_from(np.full(rows * esz, 0xA5, np.uint8))
    nn.swiglu(rt, g, u, out, rows, mid_bf16)
    assert np.array_equal(fused[: rows * esz], out.read(np.uint8, rows * esz))
    # and against the f64 oracle
    gv, uv = g.read(np.float32, rows).astype(np.float64), u.read(np.float32, rows).astype(np.float64)
    want = np.array([api.silu_f64(a) for a in gv]) * uv
    got = (synth.bf16_bits_to_f32(fused[: rows * 2].view(np.uint16)) if mid_bf16
           else fused[: rows * 4].view(np.float32))
    np.testing.assert_allclose(got, want, rtol=2.0 ** -7 if mid_bf16 else 2e-6, atol=1e-6)


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES + [(1024, 4096, 64)])
def test_kv_and_qkv_equal_separate_launches_bit_for_bit(rt, rows, cols, group):
    rows_kv = rows // 3 + 1
    x = synth.normal_bf16(0x7E550050 + rows, cols)
    xb = rt.buffer_from(x)
    banks, outs = [], []
    for i, r in enumerate((rows, rows_kv, rows_kv)):
        p, s = synth.q4_bank(0x7E550060 + 16 * i + rows, r, cols, group)
        bank = upload_bank(rt, p, s)
        banks.append(bank)
        y = seeded_f32(rt, r)
        nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(r, cols, group))
        outs.append(y.read(np.float32, r))
    qo, ko, vo = (seeded_f32(rt, r, 8) for r in (rows, rows_kv, rows_kv))
    nn.gemv_q4_mlx_qkv(rt, banks[0], banks[1], banks[2], xb, nn.QkvOutputs(qo, ko, vo), rows, rows_kv, cols, group)
    for buf, r, want in zip((qo, ko, vo), (rows, rows_kv, rows_kv), outs):
        got = buf.read(np.float32, r + 8)
        assert np.array_equal(got[:r].view(np.uint32), want.view(np.uint32))
        assert np.all(got[r:] == SENTINEL_F32)
    ko2, vo2 = seeded_f32(rt, rows_kv), seeded_f32(rt, rows_kv)
    nn.gemv_q4_mlx_kv(rt, banks[1], banks[2], xb, ko2, vo2, nn.QuantShape(rows_kv, cols, group))
    assert np.array_equal(ko2.read(np.uint32, rows_kv), outs[1].view(np.uint32))
    assert np.array_equal(vo2.read(np.uint32, rows_kv), outs[2].view(np.uint32))
    # a bank with no rows takes no part (src/nn.rs:4458-4496 of the reference project)
    nn.gemv_q4_mlx_qkv(rt, banks[0], banks[1], banks[2], xb, nn.QkvOutputs(qo, ko, vo), rows, 0, cols, group)
    nn.gemv_q4_mlx_qkv(rt, banks[0], banks[1], banks[2], xb, nn.QkvOutputs(qo, ko, vo), 0, 0, cols, group)


@pytest.mark.parametrize("rows,cols,group", REF_SHAPES[:4] + [(4096, 4096, 64), (151936 // 8, 4096, 64)])
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_small_m_gemm_matches_the_oracle(rt, rows, cols, group, m):
    packed, sb = synth.q4_bank(0x7E550070 + rows, rows, cols, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    x = synth.normal_bf16(0x7E550077 + m, m * cols)
    bank = upload_bank(rt, packed, sb)
    xb = rt.buffer_from(x)
    shape = nn.QuantShape(rows, cols, group)
    y = seeded_f32(rt, m * rows, 8)
    nn.gemm_q4_mlx(rt, bank, xb, y, shape, m)
    got = y.read(np.float32, m * rows + 8)
    assert np.all(got[m * rows:] == SENTINEL_F32)
    got = got[: m * rows].reshape(m, rows)
    want = api.q4_dense_gemm(packed, sb, x, m, rows, cols, group)
    assert_north_star(got, want, f"gemm m={m}")
    assert_gamma_bound(got, packed, sb, x, m, rows, cols, group, what=f"gemm m={m}")
    resid = rc.rand_f32(m * rows, 0x5200 + rows * m)
    r = rt.buffer_from(resid)
    nn.gemm_q4_mlx(rt, bank, xb, r, shape, m, resid=r)
    assert np.array_equal(r.read(np.float32, m * rows), got.reshape(-1) + resid)


TENSOR_GEMV_SHAPES = [(40, 1024, 32), (257, 1024, 64), (40, 2048, 32), (257, 2048, 64), (72, 2048, 128),
                      (40, 4096, 32), (129, 4096, 64), (257, 4096, 128),
                      # longer rows: M = 1 on the FMA-pipe kernels, batches as windows of 4096 columns on
                      # the MMA kernel, each launch adding to the ones before it; same contract
                      (40, 8192, 64), (257, 12288, 64), (72, 8192, 128), (33, 16384, 32),
                      (40, 6144, 64)]  # not a multiple of 4096: FMA-pipe kernels for every M


@pytest.mark.parametrize("rows,cols,group", TENSOR_GEMV_SHAPES)
def test_tensor_core_gemv_shapes(rt, rows, cols, group):
    """Rows of 1024, 2048 or 4096 columns run on the MMA kernel: every (K, G) it is built
    for, ragged row counts, batches of 1, 3 and 8, and the fused gate/up launch against
    two plain launches."""
    packed, sb, _ = make_case(rows, cols, group, 0x7E550090 + rows + cols)
    bank = upload_bank(rt, packed, sb)
    shape = nn.QuantShape(rows, cols, group)
    for m in (1, 3, 8):
        x = synth.normal_bf16(0x7E550097 + m + cols, m * cols)
        xb = rt.buffer_from(x)
        y = seeded_f32(rt, m * rows, 8)
        if m == 1:
            nn.gemv_q4_mlx_simd(rt, bank, xb, y, shape)
        else:
            nn.gemm_q4_mlx(rt, bank, xb, y, shape, m)
        got = y.read(np.float32, m * rows + 8)
        assert np.all(got[m * rows:] == SENTINEL_F32), f"wrote past y (m={m})"
        got = got[: m * rows].reshape(m, rows)
        want = api.q4_dense_gemm(packed, sb, x, m, rows, cols, group)
        assert_north_star(got, want, f"tensor-core gemv m={m} {rows}x{cols} g{group}")
        assert_gamma_bound(got, packed, sb, x, m, rows, cols, group, what=f"tensor-core gemv m={m}")
        if m > 1 and cols <= 4096:  # a batch row equals the same vector run alone, bit for bit
            x0 = rt.buffer_from(x[:cols].copy())
            y0 = seeded_f32(rt, rows)
            nn.gemv_q4_mlx_simd(rt, bank, x0, y0, shape)
            assert np.array_equal(y0.read(np.float32, rows), got[0])
    up, us, x = make_case(rows, cols, group, 0x7E5500A0 + rows + cols)
    upb, xb = upload_bank(rt, up, us), rt.buffer_from(x)
    mid = rt.buffer_from(np.full((rows + 8) * 4, 0xA5, np.uint8))
    nn.gemv_q4_mlx_gate_up_silu(rt, bank, upb, xb, mid, shape, False)
    fused = mid.read(np.uint8, (rows + 8) * 4)
    assert np.all(fused[rows * 4:] == 0xA5), "wrote past mid"
    g, u = seeded_f32(rt, rows), seeded_f32(rt, rows)
    nn.gemv_q4_mlx_simd(rt, bank, xb, g, shape)
    nn.gemv_q4_mlx_simd(rt, upb, xb, u, shape)
    out = seeded_f32(rt, rows)
    nn.swiglu(rt, g, u, out, rows, False)
    assert np.array_equal(fused[: rows * 4], out.read(np.uint8, rows * 4))


def test_refusals_happen_before_any_launch(rt):
    rows, cols, group = 40, 256, 64
    packed, sb, x = make_case(rows, cols, group, 1)
    bank = upload_bank(rt, packed, sb)
    xb, y = rt.buffer_from(x), seeded_f32(rt, rows)
    shape = nn.QuantShape(rows, cols, group)
    rt.take_dispatch_count()
    cases = [
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(rows, cols, 0)), "group_size must be non-zero"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(rows, 250, 64)), "multiple of group_size"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(rows, cols, 16)), "outside the MLX kernel domain"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(rows, 1024, 1024)), "outside the MLX kernel domain"),
        (lambda: nn.gemv_q4_mlx_simd(rt, nn.Q4MlxBank(bank.packed.view(0, 64), bank.scales_biases), xb, y, shape),
         "packed: buffer holds 64 elements"),
        (lambda: nn.gemv_q4_mlx_simd(rt, nn.Q4MlxBank(bank.packed, bank.scales_biases.view(0, 64)), xb, y, shape),
         "scales_biases"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb.view(0, 64), y, shape), "x_bf16"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y.view(0, 64), shape), " y"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, shape, resid=y.view(0, 64)), "resid"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, xb, nn.QuantShape(8, cols, group)),
         "writable buffer y overlaps read-only buffer x_bf16"),
        (lambda: nn.gemv_q4_mlx_simd(rt, bank, xb, y, shape, layout=nn.INTERLEAVED4), "Interleaved4"),
        (lambda: nn.gemm_q4_mlx(rt, bank, xb, y, shape, 9), "exceeds GEMM_MAX_M = 8"),
        (lambda: nn.gemv_q4_mlx_gate_up_silu(rt, bank, bank, xb, bank.packed, shape, False),
         "writable buffer mid overlaps read-only buffer gate_packed"),
        (lambda: nn.gemv_q4_mlx_kv(rt, bank, bank, xb, y, y, shape), "writable buffers k_out and v_out overlap"),
    ]
    for fn, want in cases:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), (want, str(e.value))
        assert e.value.status == 1
    # validated no-ops: rows == 0, m == 0
    nn.gemv_q4_mlx_simd(rt, bank, xb, y, nn.QuantShape(0, cols, group))
    nn.gemm_q4_mlx(rt, bank, xb, y, shape, 0)
    assert rt.take_dispatch_count() == 0, "a refused or empty call launched a kernel"
    assert np.all(y.read(np.float32, rows) == SENTINEL_F32)
    assert not rt.is_poisoned()


def test_q4_weight_policy_routes_by_m(rt):
    rows, cols = 256, 512
    packed, sb = synth.q4_bank(5, rows, cols, 64)
    w = nn.Q4Weight(upload_bank(rt, packed, sb), rows, cols)
    for m, launches in ((0, 0), (1, 1), (4, 1), (8, 1)):
        x = synth.normal_bf16(9 + m, max(m, 1) * cols)
        xb, y = rt.buffer_from(x), seeded_f32(rt, max(m, 1) * rows)
        rt.take_dispatch_count()
        w.matmul(rt, xb, m, y)
        assert rt.take_dispatch_count() == launches
        if m:
            want = api.q4_dense_gemm(packed.view(np.uint8), sb, x, m, rows, cols, 64)
            assert_north_star(y.read(np.float32, m * rows).reshape(m, rows), want, f"Q4Weight m={m}")
    x = synth.normal_bf16(3, 9 * cols)
    xb, y = rt.buffer_from(x), seeded_f32(rt, 9 * rows)
    with pytest.raises(nn.TesslError, match="no fused residual add"):
        w.matmul(rt, xb, 9, y, resid=y)


def test_poisoned_runtime_refuses_work():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tessl_b200 import capi

    r = nn.Runtime()
    capi.load().tessl_runtime_poison_for_test(r.handle)
    assert r.is_poisoned()
    with pytest.raises(nn.TesslError, match="poisoned"):
        r.synchronize()
    r.close()
