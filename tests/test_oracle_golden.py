"""Pins the CPU oracle against the reference's own recorded known answers.

`tests/golden/q4_kernels_golden.json` holds the rows of the reference's
`GOLDEN` table (tests/q4_kernels_template.rs:436-1494 in the reference
project; extracted by `tests/golden/extract_reference_golden.py`): for each
kernel entry and shape, an FNV-1a hash of every output word, sentinel tail
included, and the first eight words, recorded from the Metal kernels on an
Apple GPU. The order-faithful oracle regenerates the inputs from the same
seeds and must reproduce those bits.
"""
import json
import os

import numpy as np
import pytest

import ref_cases as rc
from oracle import api

HERE = os.path.dirname(os.path.abspath(__file__))
ROWS = json.load(open(os.path.join(HERE, "golden", "q4_kernels_golden.json")))["rows"]
GOLDEN = {(r["kernel"], r["case"]): r for r in ROWS}
SHAPE = {c: (r, k, g) for c, r, k, g in rc.SHAPES}


def check(kernel, case, words, exact=True, ulps=0):
    g = GOLDEN[(kernel, case)]
    want = np.array([int(w, 16) for w in g["first_words"]], np.uint32)
    got = np.zeros(8, np.uint32)
    got[: min(8, words.size)] = words[:8]
    if exact:
        assert [f"{w:#010x}" for w in got] == g["first_words"], (kernel, case)
        assert f"{api.fnv1a_words(words):#018x}" == g["hash"], (kernel, case, "hash of every word")
    else:
        a, b = got.view(np.float32).astype(np.float64), want.view(np.float32).astype(np.float64)
        assert np.all(np.abs(a - b) <= ulps * np.spacing(np.abs(b).astype(np.float32)).astype(np.float64) + 1e-30), (
            kernel, case, got, want)


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
def test_gemv_store_and_add_resid_bits(case):
    rows, cols, group = SHAPE[case]
    x = rc.rand_x(cols, 0x4100 + cols)
    resid = rc.rand_f32(rows, 0x4200 + rows)
    p, s = rc.rand_bank(rows, cols, group, 0x4300 + rows)
    out = api.q4_simd_gemv(p, s, x, rows, cols, group, out=rc.sentinel(rows + rc.PAD_WORDS))
    check("gemv_q4_mlx_simd", case, out)
    out = api.q4_simd_gemv(p, s, x, rows, cols, group, epi=api.EPI_ADD_RESID, resid=resid,
                           out=rc.sentinel(rows + rc.PAD_WORDS))
    check("gemv_q4_mlx_simd_add", case, out)


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
def test_kv_and_qkv_bits(case):
    rows, cols, group = SHAPE[case]
    x = rc.rand_x(cols, 0x4100 + cols)
    gp, gs = rc.rand_bank(rows, cols, group, 0x4400 + rows)
    up, us = rc.rand_bank(rows, cols, group, 0x4500 + rows)
    ko = api.q4_simd_gemv(gp, gs, x, rows, cols, group, out=rc.sentinel(rows + rc.PAD_WORDS))
    vo = api.q4_simd_gemv(up, us, x, rows, cols, group, out=rc.sentinel(rows + rc.PAD_WORDS))
    check("gemv_q4_mlx_simd_kv", case, np.concatenate([ko, vo]))
    rows_kv = rows // 3 + 1
    outs = []
    for seed, r in ((0x4600, rows), (0x4700, rows_kv), (0x4800, rows_kv)):
        p, s = rc.rand_bank(r, cols, group, seed + rows)
        outs.append(api.q4_simd_gemv(p, s, x, r, cols, group, out=rc.sentinel(r + rc.PAD_WORDS)))
    check("gemv_q4_mlx_simd_qkv", case, np.concatenate(outs))


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES])
@pytest.mark.parametrize("mid_bf16", [False, True])
def test_gate_up_gelu_known_answers(case, mid_bf16):
    # The epilogue calls the device's tanh, whose last bits a host libm need not
    # share, and 1 + tanh cancels for very negative gates: the sums are pinned
    # exactly by the other tests, this one to 1e-5 absolute plus 4e-6 relative
    # (f32 output) or one bf16 step (bf16 output).
    rows, cols, group = SHAPE[case]
    x = rc.rand_x(cols, 0x4100 + cols)
    gp, gs = rc.rand_bank(rows, cols, group, 0x4400 + rows)
    up, us = rc.rand_bank(rows, cols, group, 0x4500 + rows)
    out = api.q4_simd_gemv(gp, gs, x, rows, cols, group, epi=api.EPI_GATE_UP_GELU, packed1=up, sb1=us,
                           mid_as_bf16=mid_bf16, out=rc.sentinel(rows + rc.PAD_WORDS))
    name = f"{case}-{'mid-bf16' if mid_bf16 else 'mid-f32'}"
    g = GOLDEN[("gemv_q4_mlx_simd_gate_up_gelu", name)]
    want = np.array([int(w, 16) for w in g["first_words"]], np.uint32)
    if mid_bf16:
        n = min(16, rows)
        a = api.bf16_to_f32(out[:8].view(np.uint16)[:n]).astype(np.float64)
        b = api.bf16_to_f32(want.view(np.uint16)[:n]).astype(np.float64)
        assert np.all(np.abs(a - b) <= np.abs(b) * 2.0 ** -7 + 1e-5), (name, a, b)
    else:
        n = min(8, rows)
        a, b = out[:n].view(np.float32).astype(np.float64), want[:n].view(np.float32).astype(np.float64)
        assert np.all(np.abs(a - b) <= 4e-6 * np.abs(b) + 1e-5), (name, a, b)
    # words past `rows` keep the sentinel, as on the device
    tail_from = (rows + 1) // 2 if mid_bf16 else rows
    assert np.all(out[tail_from + 1:] == rc.SENTINEL)


@pytest.mark.parametrize("case", [s[0] for s in rc.SHAPES[:4]])
@pytest.mark.parametrize("m", [1, 5, 8])
def test_small_m_gemm_bits(case, m):
    rows, cols, group = SHAPE[case]
    x = rc.rand_x(m * cols, 0x5100 + cols * m)
    resid = rc.rand_f32(m * rows, 0x5200 + rows * m)
    p, s = rc.rand_bank(rows, cols, group, 0x5300 + rows)
    for with_resid in (False, True):
        out = rc.sentinel(m * rows + rc.PAD_WORDS)
        api.q4_simd_gemm(p, s, x, rows, cols, group, m, resid=resid if with_resid else None,
                         out=out.view(np.float32))
        check("gemm_q4_mlx_simd_add" if with_resid else "gemm_q4_mlx_simd", f"{case}-m{m}", out)


@pytest.mark.parametrize("n", [4099, 1, 33])
def test_device_bf16_cast_rule_bits(n):
    """f32 -> bf16 as a device store rounds it (NaN -> 0x7fc0, f32 subnormals
    flushed, ties to even), against the recorded `cast_f32_to_bf16` words; and
    the widening cast back."""
    from tessl_b200 import synth

    doc = json.load(open(os.path.join(HERE, "golden", "q4_kernels_golden.json")))
    specials = [int(w, 16) for w in doc["f32_specials"]]
    draws = (synth.splitmix_draws(0x6100 + n, n) >> np.uint64(32)).astype(np.uint32)
    # the stream only advances for elements past the special list
    src = np.array([specials[i] if i < len(specials) else 0 for i in range(n)], np.uint32)
    k = max(0, n - len(specials))
    src[len(specials):] = draws[:k]
    halves = api.f32_to_bf16_gpu(src.view(np.float32))
    out = np.full(2 * ((n * 2 + 3) // 4), 0xA5A5, np.uint16)
    out[:n] = halves
    check("cast_f32_to_bf16", f"n{n}", out.view(np.uint32))


@pytest.mark.parametrize("n", [65537, 1, 33])
def test_bf16_widening_bits(n):
    i = np.arange(n, dtype=np.uint64)
    pat = (((i * np.uint64(0x9E37)) & np.uint64(0xFFFF)) ^ (i >> np.uint64(16))).astype(np.uint16)
    check("cast_bf16_to_f32", f"n{n}", api.bf16_to_f32(pat).view(np.uint32))
