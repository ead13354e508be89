"""Helpers shared by the GPU parity tests: a runtime fixture, bank upload, tolerances."""
import numpy as np
import pytest

from oracle import api
from tessl_b200 import nn, synth

SENTINEL_F32 = np.float32(-7.7e28)  # tests/gemm_q4_mlx_tensorops.rs:30 of the reference project


@pytest.fixture(scope="module")
def rt():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = nn.Runtime()
    yield r
    r.close()


def upload_bank(rt, packed, sb):
    return nn.Q4MlxBank(rt.buffer_from(np.ascontiguousarray(packed)), rt.buffer_from(np.ascontiguousarray(sb)))


def seeded_f32(rt, n, pad=0, value=SENTINEL_F32):
    return rt.buffer_from(np.full(max(n + pad, 1), value, np.float32))


def bf16_round(a):
    """f32 -> bf16 -> f32 (round to nearest even)."""
    return synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(a, np.float32)))


def assert_north_star(got_f32, want_f32, what=""):
    """The stated output tolerance: after bf16 rounding of both, within
    1e-2 relative + 2e-3 absolute."""
    g = bf16_round(got_f32).astype(np.float64)
    w = bf16_round(want_f32).astype(np.float64)
    err = np.abs(g - w)
    tol = 2e-3 + 1e-2 * np.abs(w)
    bad = np.flatnonzero(err > tol)
    assert bad.size == 0, f"{what}: {bad.size} outputs outside 1e-2 rel / 2e-3 abs, first {bad[:4]}: got {g.flat[bad[:4]]} want {w.flat[bad[:4]]}"


def assert_gamma_bound(got_f32, packed, sb, x_bf16, m, rows, cols, group, extra_terms=0, what=""):
    """The reference's derived bound: |got - exact| <= gamma_t * S with
    t = K + 2K/G (+ extra), S the sum of term magnitudes
    (tests/gemm_q4_mlx_tensorops.rs:11-21 of the reference project)."""
    want, mag = api.q4_affine_f64(packed, sb, x_bf16, m, rows, cols, group)
    g = api.gamma(cols + 2 * (cols // group) + extra_terms)
    err = np.abs(np.asarray(got_f32, np.float64).reshape(m, rows) - want)
    frac = err / np.maximum(g * mag, 1e-300)
    assert np.all(np.isfinite(got_f32)), what
    assert frac.max() <= 1.0, f"{what}: error is {frac.max():.3f} of gamma_t * S"
    return frac.max()
