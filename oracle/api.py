"""ctypes + numpy front end of the CPU oracle (test infrastructure only).

Only `tests/`, the smoke check and the CPU-baseline legs of `bench.py` import
this module; the product package never does. Arrays are numpy, bf16 values
travel as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")

EPI_STORE, EPI_ADD_RESID, EPI_GATE_UP_GELU, EPI_GATE_UP_SILU = 0, 1, 2, 3

# The accumulation order the reference's recorded kernel outputs were found to
# follow (see tests/test_oracle_golden.py): simd_sum mode, affine mode, chain mode.
DEFAULT_ORDER = (3, 3, 0)

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(str(_build.build_oracle()))
        sz, vp = C.c_size_t, C.c_void_p
        L.orc_splitmix_new.restype = C.c_uint64
        L.orc_splitmix_new.argtypes = [C.c_uint64]
        L.orc_splitmix_next.restype = C.c_uint64
        L.orc_splitmix_next.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_splitmix_unit.restype = C.c_float
        L.orc_splitmix_unit.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_f32_to_bf16_bits.restype = C.c_uint16
        L.orc_f32_to_bf16_bits.argtypes = [C.c_float]
        L.orc_f32_to_bf16_bits_gpu.restype = C.c_uint16
        L.orc_f32_to_bf16_bits_gpu.argtypes = [C.c_float]
        L.orc_bf16_bits_to_f32.restype = C.c_float
        L.orc_bf16_bits_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16_array.argtypes = [_f32p, _u16p, sz]
        L.orc_q4_pack.argtypes = [_u8p, sz, _u8p]
        L.orc_q4_unpack.argtypes = [_u8p, sz, _u8p]
        L.orc_interleave_scales_biases.argtypes = [_u16p, _u16p, sz, _u16p]
        L.orc_q4_dequant.argtypes = [_u8p, _u16p, sz, sz, sz, _f32p]
        L.orc_q4_dense_gemm.argtypes = [_u8p, _u16p, _u16p, sz, sz, sz, sz, _f32p, C.c_int]
        L.orc_q4_affine_gemm_f64.argtypes = [_u8p, _u16p, _u16p, sz, sz, sz, sz, _f64p, vp, C.c_int]
        L.orc_gamma.restype = C.c_double
        L.orc_gamma.argtypes = [sz]
        L.orc_reduction_tolerance.restype = C.c_double
        L.orc_reduction_tolerance.argtypes = [sz, C.c_double]
        for name in ("orc_silu_f64", "orc_gelu_f64"):
            getattr(L, name).restype = C.c_double
            getattr(L, name).argtypes = [C.c_double]
        for name in ("orc_silu_f32", "orc_gelu_f32"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.orc_q4_simd_gemv.argtypes = [vp, vp, vp, vp, _u16p, vp, vp, C.c_int, C.c_int, C.c_uint32, C.c_uint32,
                                       C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_q4_simd_gemm.argtypes = [_u8p, _u16p, _u16p, _f32p, vp, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_q8_gemv_f64.argtypes = [_i8p, _f32p, _f32p, _f32p, sz, sz, sz, _f32p, C.c_int]
        L.orc_q8_simd_gemv.argtypes = [_i8p, _f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p,
                                       C.c_int, C.c_int]
        L.orc_q8_mlx_dense_gemm.argtypes = [_u8p, _u16p, _u16p, sz, sz, sz, sz, _f32p, C.c_int]
        L.orc_q8_mlx_dequant.argtypes = [_u8p, _u16p, sz, sz, sz, _f32p]
        L.orc_fnv1a_words.restype = C.c_uint64
        L.orc_fnv1a_words.argtypes = [_u32p, sz]
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class SplitMix:
    """The reference tests' splitmix64 stream, one draw at a time (small cases)."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(lib().orc_splitmix_new(seed & 0xFFFFFFFFFFFFFFFF))

    def next(self) -> int:
        return lib().orc_splitmix_next(C.byref(self._s))

    def word(self) -> int:
        return self.next() >> 32

    def unit(self) -> np.float32:
        return np.float32(lib().orc_splitmix_unit(C.byref(self._s)))


def max_threads() -> int:
    return lib().orc_max_threads()


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().orc_f32_to_bf16_array(a.reshape(-1), out.reshape(-1), a.size)
    return out


def f32_to_bf16_gpu(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    return np.array([lib().orc_f32_to_bf16_bits_gpu(float(v)) for v in a], np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def q4_pack(nibbles: np.ndarray) -> np.ndarray:
    n = np.ascontiguousarray(nibbles, np.uint8).reshape(-1)
    out = np.empty((n.size + 1) // 2, np.uint8)
    lib().orc_q4_pack(n, n.size, out)
    return out


def q4_unpack(packed: np.ndarray, n: int) -> np.ndarray:
    p = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    out = np.empty(n, np.uint8)
    lib().orc_q4_unpack(p, n, out)
    return out


def interleave_sb(scales_bf16: np.ndarray, biases_bf16: np.ndarray) -> np.ndarray:
    s = np.ascontiguousarray(scales_bf16, np.uint16).reshape(-1)
    b = np.ascontiguousarray(biases_bf16, np.uint16).reshape(-1)
    out = np.empty(2 * s.size, np.uint16)
    lib().orc_interleave_scales_biases(s, b, s.size, out)
    return out


def q4_dequant(packed, sb, rows, cols, group) -> np.ndarray:
    out = np.empty((rows, cols), np.float32)
    lib().orc_q4_dequant(_c(packed, np.uint8), _c(sb, np.uint16), rows, cols, group, out.reshape(-1))
    return out


def _c(a, dt):
    return np.ascontiguousarray(a, dt).reshape(-1)


def q4_dense_gemm(packed, sb, x_bf16, m, rows, cols, group, threads=0) -> np.ndarray:
    """f64-accumulated dequant-matvec, [m, rows] f32: the parity reference."""
    y = np.empty((m, rows), np.float32)
    lib().orc_q4_dense_gemm(_c(packed, np.uint8), _c(sb, np.uint16), _c(x_bf16, np.uint16), m, rows, cols, group,
                            y.reshape(-1), threads)
    return y


def q4_affine_f64(packed, sb, x_bf16, m, rows, cols, group, threads=0):
    """Exact affine product in f64 and its magnitude S, each [m, rows]."""
    want = np.empty((m, rows), np.float64)
    mag = np.empty((m, rows), np.float64)
    lib().orc_q4_affine_gemm_f64(_c(packed, np.uint8), _c(sb, np.uint16), _c(x_bf16, np.uint16), m, rows, cols,
                                 group, want.reshape(-1), _ptr(mag), threads)
    return want, mag


def gamma(terms: int) -> float:
    return lib().orc_gamma(terms)


def q4_simd_gemv(packed0, sb0, x_bf16, rows, cols, group, *, epi=EPI_STORE, packed1=None, sb1=None, resid=None,
                 mid_as_bf16=False, out=None, order=DEFAULT_ORDER, threads=0) -> np.ndarray:
    """Order-faithful emulation of the reference's simdgroup GEMV. Returns the
    output buffer as uint32 words (f32 bits, or bf16 halves when mid_as_bf16);
    pass `out` (uint32, pre-filled) to see which words the kernel leaves alone."""
    if out is None:
        out = np.zeros(rows, np.uint32)
    p0, s0 = _c(packed0, np.uint8), _c(sb0, np.uint16)
    p1 = None if packed1 is None else _c(packed1, np.uint8)
    s1 = None if sb1 is None else _c(sb1, np.uint16)
    r = None if resid is None else _c(resid, np.float32)
    lib().orc_q4_simd_gemv(_ptr(p0), _ptr(s0), _ptr(p1), _ptr(s1), _c(x_bf16, np.uint16), _ptr(out), _ptr(r), epi,
                           int(mid_as_bf16), rows, cols, group, order[0], order[1], order[2], threads)
    return out


def q4_simd_gemm(packed, sb, x_bf16, rows, cols, group, m, *, resid=None, out=None, order=DEFAULT_ORDER,
                 threads=0) -> np.ndarray:
    if out is None:
        out = np.zeros(m * rows, np.float32)
    r = None if resid is None else _c(resid, np.float32)
    lib().orc_q4_simd_gemm(_c(packed, np.uint8), _c(sb, np.uint16), _c(x_bf16, np.uint16), out, _ptr(r), rows, cols,
                           group, m, order[0], order[1], order[2], threads)
    return out


def q8_gemv_f64(q, scales, zeros, x, rows, cols, group, threads=0) -> np.ndarray:
    y = np.empty(rows, np.float32)
    lib().orc_q8_gemv_f64(_c(q, np.int8), _c(scales, np.float32), _c(zeros, np.float32), _c(x, np.float32), rows,
                          cols, group, y, threads)
    return y


def q8_simd_gemv(q, scales, zeros, x, rows, cols, group, sum_mode=0, threads=0) -> np.ndarray:
    y = np.empty(rows, np.float32)
    lib().orc_q8_simd_gemv(_c(q, np.int8), _c(scales, np.float32), _c(zeros, np.float32), _c(x, np.float32), rows,
                           cols, group, y, sum_mode, threads)
    return y


def q8_mlx_dense_gemm(codes, sb, x_bf16, m, rows, cols, group, threads=0) -> np.ndarray:
    y = np.empty((m, rows), np.float32)
    lib().orc_q8_mlx_dense_gemm(_c(codes, np.uint8), _c(sb, np.uint16), _c(x_bf16, np.uint16), m, rows, cols, group,
                                y.reshape(-1), threads)
    return y


def q8_mlx_dequant(codes, sb, rows, cols, group) -> np.ndarray:
    out = np.empty((rows, cols), np.float32)
    lib().orc_q8_mlx_dequant(_c(codes, np.uint8), _c(sb, np.uint16), rows, cols, group, out.reshape(-1))
    return out


def silu_f64(x: float) -> float:
    return lib().orc_silu_f64(x)


def gelu_f64(x: float) -> float:
    return lib().orc_gelu_f64(x)


def silu_f32(x) -> np.float32:
    return np.float32(lib().orc_silu_f32(float(x)))


def fnv1a_words(words: np.ndarray) -> int:
    w = np.ascontiguousarray(words, np.uint32).reshape(-1)
    return lib().orc_fnv1a_words(w, w.size)


def embed_lookup_q4_mlx(packed, sb, token_ids, vocab, hidden, group) -> np.ndarray:
    """kernels/embed_lookup.metal:7-38 of the reference project: out[m, :] = the dequantized row
    token_ids[m] (scale * q + bias in f32; the product is exact, so a fused multiply-add gives the
    same bits), a row of zeros for an id outside the table. f32 [n_tokens, hidden]."""
    ids = np.ascontiguousarray(token_ids, np.uint32).reshape(-1)
    out = np.zeros((ids.size, hidden), np.float32)
    p = _c(packed, np.uint8).reshape(vocab, hidden // 2)
    s = _c(sb, np.uint16).reshape(vocab, (hidden // group) * 2)
    for m, tid in enumerate(ids):
        if tid < vocab:
            out[m] = q4_dequant(p[tid], s[tid], 1, hidden, group)[0]
    return out


def qwen35_rms_norm_f64(x, w, rows, dim, eps, resid_add=None) -> np.ndarray:
    """kernels/qwen35_mlp.metal:76-171 of the reference project in f64: out = v * rsqrt(mean(v^2) + eps)
    * (1 + w) with v = x (+ y for the fused add), `1 + w` formed in f32 as the kernel forms it."""
    v = np.asarray(x, np.float32).reshape(rows, dim)
    if resid_add is not None:
        v = v + np.asarray(resid_add, np.float32).reshape(rows, dim)  # the f32 add of the kernel
    v64 = v.astype(np.float64)
    inv = 1.0 / np.sqrt((v64 * v64).mean(axis=1, keepdims=True) + np.float64(np.float32(eps)))
    wp = (np.float32(1.0) + np.asarray(w, np.float32).reshape(dim)).astype(np.float64)
    return v64 * inv * wp


def q4_repack_b200_staged(packed, sb, rows, cols, group) -> np.ndarray:
    """The B200 staged image of a bank, as bytes: units of 8 rows, each four pairs of adjacent packed rows (row 2i,
    row 2i + 1, 32 zero bytes) followed by the eight rows' (scale, bias) pairs; rows past the end are zeros. The
    library's own repack (no counterpart in the reference, whose Interleaved4 plays this role on Apple GPUs,
    tests/q4_interleaved.rs:54-83 of the reference project, holds its repack oracle the same way)."""
    row_bytes, sb_row = cols // 2, (cols // group) * 4
    pair_pitch = 2 * row_bytes + 32
    unit = 4 * pair_pitch + 8 * sb_row
    units = (rows + 7) // 8
    p = np.zeros((units * 8, row_bytes), np.uint8)
    p[:rows] = np.ascontiguousarray(packed).view(np.uint8).reshape(rows, row_bytes)
    s = np.zeros((units * 8, sb_row), np.uint8)
    s[:rows] = np.ascontiguousarray(sb).view(np.uint8).reshape(rows, sb_row)
    out = np.zeros((units, unit), np.uint8)
    pairs = p.reshape(units, 4, 2 * row_bytes)
    for i in range(4):
        out[:, i * pair_pitch: i * pair_pitch + 2 * row_bytes] = pairs[:, i]
    out[:, 4 * pair_pitch:] = s.reshape(units, 8 * sb_row)
    return out.reshape(-1)
