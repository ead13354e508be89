"""Pins the restated CPU oracle (`oracle/tessl_oracle.c`) to the reference's own kernel text.

`oracle/_ref/libtessl_ref_kernels.so` is the reference project's simdgroup kernel sources
(kernels/gemv_q8.metal, gemv_q4_mlx_simd.h, gemm_q4_mlx_simd.h, q4_mlx_dot.h, act.h and the entry
points of gemv_q4_mlx.metal / gemm_q4_mlx.metal) compiled as C++ against a stand-in `metal_stdlib`
(`oracle/ref_shim/`, the method of the reference's tools/msl_emu). The same seeded inputs go through
both; with the two free choices set the way that build makes them (`simd_sum` an xor butterfly,
no fused multiply-add: the restatement's order (3, 0, 0)) every output word must be identical.

This is what ties the Q8 oracle to the reference: the reference recorded no known answers for
`gemv_q8` (its own test, tests/quantized_gemv.rs:126-163, compares against an f64 reference within
2e-4), so the restated kernel order is checked here against the compiled kernel itself, on that
test's shapes, and the f64 reference against both.
"""
import numpy as np
import pytest

import ref_cases as rc
from oracle import api, ref_api

pytestmark = pytest.mark.skipif(not ref_api.available(), reason="no reference checkout and no built oracle/_ref library")

ORDER = (3, 0, 0)  # simd_sum: xor butterfly; affine and chain as the source writes them, unfused


def _q8_case(rows, cols, group, seed):
    """tests/quantized_gemv.rs:126-163 of the reference project: int8 codes, scales 0.01 .. 0.03, zeros -2 .. 2."""
    from tessl_b200 import synth

    d = synth.splitmix_draws(seed, rows * cols + 2 * rows * (cols // group) + cols)
    q = ((d[: rows * cols] >> np.uint64(33)) & np.uint64(0xFF)).astype(np.uint8).view(np.int8)
    u = synth.unit_from_draws(d[rows * cols:])
    ng = rows * (cols // group)
    scales = (np.float32(0.02) + np.float32(0.01) * u[:ng]).astype(np.float32)
    zeros = (np.float32(2.0) * u[ng: 2 * ng]).astype(np.float32)
    x = u[2 * ng: 2 * ng + cols].astype(np.float32)
    return q, scales, zeros, x


@pytest.mark.parametrize("rows,cols,group", [(8, 64, 32), (13, 128, 32), (64, 256, 64), (37, 544, 32), (5, 96, 8),
                                            (9, 60, 6), (33, 1024, 128)])
def test_q8_restatement_is_the_reference_kernel_bit_for_bit(rows, cols, group):
    q, scales, zeros, x = _q8_case(rows, cols, group, 0x8800 + rows + cols)
    ref = ref_api.gemv_q8(q, scales, zeros, x, rows, cols, group)
    orc = api.q8_simd_gemv(q, scales, zeros, x, rows, cols, group, sum_mode=3)
    assert np.array_equal(ref.view(np.uint32), orc.view(np.uint32))
    # and both agree with the f64 reference of the reference's own test, within its tolerance
    f64 = api.q8_gemv_f64(q, scales, zeros, x, rows, cols, group)
    assert np.all(np.abs(ref.astype(np.float64) - f64) <= 2e-4 * np.maximum(np.abs(f64), 1.0))


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
def test_q4_gemv_entries_match_the_reference_kernels(case):
    _, rows, cols, group = next(s for s in rc.SHAPES if s[0] == case)
    x = rc.rand_x(cols, 0x4100 + cols)
    resid = rc.rand_f32(rows, 0x4200 + rows)
    p, s = rc.rand_bank(rows, cols, group, 0x4300 + rows)
    assert np.array_equal(ref_api.gemv_q4_mlx_simd(p, s, x, rows, cols, group).view(np.uint32),
                          api.q4_simd_gemv(p, s, x, rows, cols, group, order=ORDER))
    assert np.array_equal(ref_api.gemv_q4_mlx_simd(p, s, x, rows, cols, group, resid=resid).view(np.uint32),
                          api.q4_simd_gemv(p, s, x, rows, cols, group, epi=api.EPI_ADD_RESID, resid=resid, order=ORDER))
    # y == resid: the one alias the reference allows (src/nn.rs:4001)
    y = resid.copy()
    ref_api.gemv_q4_mlx_simd(p, s, x, rows, cols, group, resid=y, out=y)
    assert np.array_equal(y.view(np.uint32),
                          api.q4_simd_gemv(p, s, x, rows, cols, group, epi=api.EPI_ADD_RESID, resid=resid, order=ORDER))


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
def test_q4_bank_routed_entries_match_the_reference_kernels(case):
    _, rows, cols, group = next(s for s in rc.SHAPES if s[0] == case)
    x = rc.rand_x(cols, 0x4100 + cols)
    kp, ks = rc.rand_bank(rows, cols, group, 0x4400 + rows)
    vp, vs = rc.rand_bank(rows, cols, group, 0x4500 + rows)
    ko, vo = ref_api.gemv_q4_mlx_kv(kp, ks, vp, vs, x, rows, cols, group)
    assert np.array_equal(ko.view(np.uint32), api.q4_simd_gemv(kp, ks, x, rows, cols, group, order=ORDER))
    assert np.array_equal(vo.view(np.uint32), api.q4_simd_gemv(vp, vs, x, rows, cols, group, order=ORDER))
    rows_kv = rows // 3 + 1
    banks = [rc.rand_bank(r, cols, group, seed + rows) for seed, r in ((0x4600, rows), (0x4700, rows_kv), (0x4800, rows_kv))]
    outs = ref_api.gemv_q4_mlx_qkv(banks[0][0], banks[0][1], banks[1][0], banks[1][1], banks[2][0], banks[2][1], x, rows,
                                   rows_kv, cols, group)
    for (p, s), r, got in zip(banks, (rows, rows_kv, rows_kv), outs):
        assert np.array_equal(got.view(np.uint32), api.q4_simd_gemv(p, s, x, r, cols, group, order=ORDER))


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
@pytest.mark.parametrize("silu", [True, False])
@pytest.mark.parametrize("mid_bf16", [False, True])
def test_q4_gate_up_entries_match_the_reference_kernels(case, silu, mid_bf16):
    _, rows, cols, group = next(s for s in rc.SHAPES if s[0] == case)
    x = rc.rand_x(cols, 0x4100 + cols)
    gp, gs = rc.rand_bank(rows, cols, group, 0x4400 + rows)
    up, us = rc.rand_bank(rows, cols, group, 0x4500 + rows)
    ref = ref_api.gemv_q4_mlx_gate_up(gp, gs, up, us, x, rows, cols, group, mid_bf16, silu)
    orc = api.q4_simd_gemv(gp, gs, x, rows, cols, group, epi=api.EPI_GATE_UP_SILU if silu else api.EPI_GATE_UP_GELU,
                           packed1=up, sb1=us, mid_as_bf16=mid_bf16, order=ORDER)
    if mid_bf16:
        a = api.bf16_to_f32(ref.view(np.uint16)[:rows]).astype(np.float64)
        b = api.bf16_to_f32(orc.view(np.uint16)[:rows]).astype(np.float64)
    else:
        a, b = ref[:rows].view(np.float32).astype(np.float64), orc[:rows].view(np.float32).astype(np.float64)
    # the sums are identical (previous tests); exp / tanh come from the same libm here, so the epilogue is too
    assert np.array_equal(a, b)


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES[:4]])
@pytest.mark.parametrize("m", [1, 5, 8])
def test_q4_small_batch_entries_match_the_reference_kernels(case, m):
    _, rows, cols, group = next(s for s in rc.SHAPES if s[0] == case)
    x = rc.rand_x(m * cols, 0x5100 + cols * m)
    resid = rc.rand_f32(m * rows, 0x5200 + rows * m)
    p, s = rc.rand_bank(rows, cols, group, 0x5300 + rows)
    for r in (None, resid):
        ref = ref_api.gemm_q4_mlx_simd(p, s, x, rows, cols, group, m, resid=r)
        orc = api.q4_simd_gemm(p, s, x, rows, cols, group, m, resid=r, order=ORDER)
        assert np.array_equal(ref.view(np.uint32), orc.view(np.uint32))
