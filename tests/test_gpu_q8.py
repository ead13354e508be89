"""GPU parity of the 8-bit GEMVs through the C ABI.

`gemv_q8` follows the reference's own test (tests/quantized_gemv.rs:126-163 in
the reference project): signed codes, f32 scale/zero, both load paths, tolerance
2e-4 * max(|want|, 1). `gemm_q8_mlx` (MLX bank convention at eight bits, M <= 8)
is checked against the dequant-matvec oracle and, for bias = -128 * scale,
against `gemv_q8` on the same weights.
"""
import numpy as np
import pytest

from gpu_util import SENTINEL_F32, assert_north_star, rt, seeded_f32  # noqa: F401
from oracle import api
from tessl_b200 import nn, synth

pytestmark = pytest.mark.gpu


def close_rel(got, want, rel):
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - want) <= rel * np.maximum(np.abs(want), 1.0)), np.abs(got - want).max()


@pytest.mark.parametrize("rows,cols,group", [(16, 256, 64), (13, 768, 32), (300, 512, 128), (16, 96, 6), (9, 90, 10),
                                             (64, 4096, 64), (14336, 4096, 64), (5000, 1024, 16)])
def test_gemv_q8_matches_the_f64_reference(rt, rows, cols, group):
    i = np.arange(rows * cols, dtype=np.int64)
    q = ((i * 53 + 7) % 251).astype(np.int32).astype(np.int8)  # wraps past 127 as the reference's cast does
    groups = rows * (cols // group)
    gi = np.arange(groups)
    scales = (0.004 + (gi % 9) * 0.001).astype(np.float32)
    zeros = (-3.0 + (gi % 4)).astype(np.float32)
    x = synth.unit_from_draws(synth.splitmix_draws(0xB8 + cols, cols))
    want = api.q8_gemv_f64(q, scales, zeros, x, rows, cols, group)
    y = seeded_f32(rt, rows, 8)
    nn.gemv_q8(rt, rt.buffer_from(q), rt.buffer_from(scales), rt.buffer_from(zeros), rt.buffer_from(x), y, rows, cols,
               group)
    got = y.read(np.float32, rows + 8)
    assert np.all(got[rows:] == SENTINEL_F32)
    close_rel(got[:rows], want, 2e-4)
    close_rel(got[:rows], api.q8_simd_gemv(q, scales, zeros, x, rows, cols, group, sum_mode=3), 2e-4)


@pytest.mark.parametrize("m", [1, 4, 8])
@pytest.mark.parametrize("rows,cols,group", [(37, 544, 32), (64, 1024, 64), (14336, 4096, 64), (100, 512, 512),
                                             (37, 512, 32), (100, 2048, 32), (257, 2048, 64), (40, 4096, 32)])
def test_gemm_q8_mlx_matches_the_dequant_matvec(rt, rows, cols, group, m):
    codes, sb = synth.q8_bank(0x7E550200 + rows, rows, cols, group)
    x = synth.normal_bf16(0x7E550207 + m, m * cols)
    cb, sbb, xb = rt.buffer_from(codes), rt.buffer_from(sb), rt.buffer_from(x)
    shape = nn.QuantShape(rows, cols, group)
    y = seeded_f32(rt, m * rows, 8)
    nn.gemm_q8_mlx(rt, cb, sbb, xb, y, shape, m)
    got = y.read(np.float32, m * rows + 8)
    assert np.all(got[m * rows:] == SENTINEL_F32)
    got = got[: m * rows].reshape(m, rows)
    want = api.q8_mlx_dense_gemm(codes.view(np.uint8), sb, x, m, rows, cols, group)
    assert_north_star(got, want, f"q8 mlx m={m}")
    # tighter than the stated tolerance: the products are exact and the accumulation is f32
    # (measured: 1.3e-5 absolute at |y| ~ 15)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=5e-4)
    if m > 1 and cols in (512, 1024, 2048, 4096) and group in (32, 64):
        # on the tensor-core kernel a batch row equals the same vector run alone, bit for bit
        y1 = seeded_f32(rt, rows)
        nn.gemm_q8_mlx(rt, cb, sbb, rt.buffer_from(x[:cols].copy()), y1, shape, 1)
        assert np.array_equal(y1.read(np.uint32, rows), got[0].view(np.uint32))
    yb = rt.buffer_from(np.full(m * rows, 0xA5A5, np.uint16))
    nn.gemm_q8_mlx(rt, cb, sbb, xb, yb, shape, m, y_as_bf16=True)
    assert np.array_equal(yb.read(np.uint16, m * rows), synth.f32_to_bf16_bits(got.reshape(-1)))
    if m == 1:
        # bias = -128 * scale maps onto the reference convention exactly:
        # int8 code = code ^ 0x80, scale widened, zero = 0, x widened.
        q = (codes.view(np.uint8) ^ np.uint8(0x80)).view(np.int8)
        scales = synth.bf16_bits_to_f32(sb[..., 0]).reshape(-1)
        y2 = seeded_f32(rt, rows)
        nn.gemv_q8(rt, rt.buffer_from(q), rt.buffer_from(scales), rt.buffer_from(np.zeros_like(scales)),
                   rt.buffer_from(synth.bf16_bits_to_f32(x)), y2, rows, cols, group)
        np.testing.assert_allclose(y2.read(np.float32, rows), got[0], rtol=1e-4, atol=5e-4)


def test_q8_refusals(rt):
    rows, cols, group = 16, 256, 64
    q = rt.buffer_from(np.zeros(rows * cols, np.int8))
    s = rt.buffer_from(np.ones(rows * 4, np.float32))
    x = rt.buffer_from(np.ones(cols, np.float32))
    y = seeded_f32(rt, rows)
    rt.take_dispatch_count()
    for fn, want in [
        (lambda: nn.gemv_q8(rt, q, s, s, x, y, rows, cols, 0), "group_size must be non-zero"),
        (lambda: nn.gemv_q8(rt, q, s, s, x, y, rows, 250, 64), "silently drop the ragged tail group"),
        (lambda: nn.gemv_q8(rt, q.view(0, 64), s, s, x, y, rows, cols, group), "gemv_q8 packed"),
        (lambda: nn.gemv_q8(rt, q, s.view(0, 8), s, x, y, rows, cols, group), "gemv_q8 scales"),
        (lambda: nn.gemv_q8(rt, q, s, s, x, x, rows, cols, group), "writable buffer y overlaps read-only buffer x"),
    ]:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), str(e.value)
    nn.gemv_q8(rt, q, s, s, x, y, 0, cols, group)
    assert rt.take_dispatch_count() == 0
