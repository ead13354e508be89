"""ctypes front end of `_ref/libtessl_ref_kernels.so`: the reference project's own MLX-Q4 / Q8
simdgroup kernel sources compiled for the CPU (see `build.build_ref` and `ref_shim/`).

Test infrastructure only, like the rest of this folder: it pins the restated oracle
(`tessl_oracle.c`) to the reference's kernel text. `available()` is False where neither the built
library nor a reference checkout exists.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

_lib = None


def available() -> bool:
    return _build.REF_SO.exists() or _build.reference_root() is not None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        so = _build.build_ref()
        if so is None:
            raise RuntimeError("no reference checkout and no built oracle/_ref library")
        _lib = C.CDLL(str(so))
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dt).reshape(-1)


def gemv_q8(q, scales, zeros, x, rows, cols, group) -> np.ndarray:
    """kernels/gemv_q8.metal:33-122 over ceil(rows / 8) threadgroups."""
    y = np.zeros(rows, np.float32)
    lib().ref_gemv_q8(_p(_c(q, np.int8)), _p(_c(scales, np.float32)), _p(_c(zeros, np.float32)), _p(_c(x, np.float32)),
                      _p(y), C.c_uint(rows), C.c_uint(cols), C.c_uint(group))
    return y


def gemv_q4_mlx_simd(packed, sb, x_bf16, rows, cols, group, resid=None, out=None) -> np.ndarray:
    """`gemv_q4_mlx_simd` / `_add` (kernels/gemv_q4_mlx.metal:381-418)."""
    y = np.zeros(rows, np.float32) if out is None else out
    r = None if resid is None else _c(resid, np.float32)
    lib().ref_gemv_q4_mlx_simd(_p(_c(packed, np.uint8)), _p(_c(sb, np.uint16)), _p(_c(x_bf16, np.uint16)), _p(y),
                               C.c_uint(rows), C.c_uint(cols), C.c_uint(group), _p(r))
    return y


def gemv_q4_mlx_gate_up(gate, gate_sb, up, up_sb, x_bf16, rows, cols, group, mid_as_bf16, silu) -> np.ndarray:
    """`gemv_q4_mlx_simd_gate_up_gelu` / `_silu` (kernels/gemv_q4_mlx.metal:420-467). The output buffer as
    uint32 words (f32 bits, or bf16 halves packed two per word when `mid_as_bf16`)."""
    mid = np.zeros(rows, np.uint32)
    lib().ref_gemv_q4_mlx_simd_gate_up(_p(_c(gate, np.uint8)), _p(_c(gate_sb, np.uint16)), _p(_c(up, np.uint8)),
                                       _p(_c(up_sb, np.uint16)), _p(_c(x_bf16, np.uint16)), _p(mid), C.c_uint(rows),
                                       C.c_uint(cols), C.c_uint(group), C.c_uint(int(mid_as_bf16)), C.c_int(int(silu)))
    return mid


def gemv_q4_mlx_kv(k, k_sb, v, v_sb, x_bf16, rows, cols, group):
    ko, vo = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
    lib().ref_gemv_q4_mlx_simd_kv(_p(_c(k, np.uint8)), _p(_c(k_sb, np.uint16)), _p(_c(v, np.uint8)), _p(_c(v_sb, np.uint16)),
                                  _p(_c(x_bf16, np.uint16)), _p(ko), _p(vo), C.c_uint(rows), C.c_uint(cols), C.c_uint(group))
    return ko, vo


def gemv_q4_mlx_qkv(q, q_sb, k, k_sb, v, v_sb, x_bf16, rows_q, rows_kv, cols, group):
    qo, ko, vo = np.zeros(rows_q, np.float32), np.zeros(rows_kv, np.float32), np.zeros(rows_kv, np.float32)
    lib().ref_gemv_q4_mlx_simd_qkv(_p(_c(q, np.uint8)), _p(_c(q_sb, np.uint16)), _p(_c(k, np.uint8)), _p(_c(k_sb, np.uint16)),
                                   _p(_c(v, np.uint8)), _p(_c(v_sb, np.uint16)), _p(_c(x_bf16, np.uint16)), _p(qo), _p(ko),
                                   _p(vo), C.c_uint(rows_q), C.c_uint(rows_kv), C.c_uint(cols), C.c_uint(group))
    return qo, ko, vo


def gemm_q4_mlx_simd(packed, sb, x_bf16, rows, cols, group, m, resid=None) -> np.ndarray:
    """`gemm_q4_mlx_simd` / `_add` (kernels/gemm_q4_mlx.metal:8-44): [m, rows] f32."""
    y = np.zeros(m * rows, np.float32)
    r = None if resid is None else _c(resid, np.float32)
    lib().ref_gemm_q4_mlx_simd(_p(_c(packed, np.uint8)), _p(_c(sb, np.uint16)), _p(_c(x_bf16, np.uint16)), _p(y),
                               C.c_uint(rows), C.c_uint(cols), C.c_uint(group), C.c_uint(m), _p(r))
    return y
