"""ctypes binding of `libtessl_b200.so` (the declarations of `include/tessl_b200.h`).

The binding style follows the reference's own `python/tessl_torch` package: a
plain `ctypes.CDLL`, an ABI-version check at load, and one error buffer per
call turned into a Python exception. There is no fallback: if the shared
library is missing or its ABI differs, importing fails loudly.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

ABI_VERSION = 1
TESSL_OK, TESSL_ERR, TESSL_PANIC = 0, 1, 2
ROW_MAJOR, INTERLEAVED4, B200_STAGED = 0, 1, 2
GEMM_Q4_MLX_MAX_M = 8

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libtessl_b200.so"


class TesslError(RuntimeError):
    """A TESSL_ERR / TESSL_PANIC status; `.status` holds the code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class Buf(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("nbytes", C.c_uint64)]


class QuantShape(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("group_size", C.c_uint32)]


class Q4MlxBank(C.Structure):
    _fields_ = [("packed", Buf), ("scales_biases", Buf)]


class QkvOutputs(C.Structure):
    _fields_ = [("q_out", Buf), ("k_out", Buf), ("v_out", Buf)]


class TensorInfo(C.Structure):
    _fields_ = [("dtype", C.c_char * 8), ("ndim", C.c_uint32), ("shape", C.c_uint64 * 8), ("nbytes", C.c_uint64)]


class PeerGather(C.Structure):
    _fields_ = [("buffers", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("rank", C.c_uint32), ("world", C.c_uint32),
                ("bytes_per_rank", C.c_uint64)]


_ERR = [C.c_char_p, C.c_size_t]
_RT = C.c_void_p
_u32 = C.c_uint32

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "tessl_abi_version": (_u32, []),
    "tessl_runtime_new": (_RT, _ERR),
    "tessl_runtime_new_on_device": (_RT, [C.c_int32] + _ERR),
    "tessl_runtime_free": (C.c_int32, [_RT]),
    "tessl_synchronize": (C.c_int32, [_RT] + _ERR),
    "tessl_runtime_set_async_encode": (C.c_int32, [_RT, _u32] + _ERR),
    "tessl_runtime_set_encode_only": (C.c_int32, [_RT, _u32] + _ERR),
    "tessl_runtime_poisoned": (C.c_int32, [_RT, C.POINTER(C.c_int32)] + _ERR),
    "tessl_runtime_take_dispatch_count": (C.c_int32, [_RT, C.POINTER(C.c_uint64)] + _ERR),
    "tessl_runtime_stream": (C.c_void_p, [_RT]),
    "tessl_runtime_device": (C.c_int32, [_RT]),
    "tessl_runtime_poison_for_test": (C.c_int32, [_RT]),
    "tessl_runtime_set_prefill_tile": (C.c_int32, [_RT, _u32, C.c_int32] + _ERR),
    "tessl_runtime_last_prefill_tile": (C.c_int32, [_RT, C.POINTER(_u32), C.POINTER(_u32)] + _ERR),
    "tessl_runtime_set_peer_wait_limit": (C.c_int32, [_RT, C.c_uint64] + _ERR),
    "tessl_buffer_alloc": (C.c_int32, [_RT, C.c_uint64, C.POINTER(Buf)] + _ERR),
    "tessl_buffer_free": (C.c_int32, [_RT, Buf] + _ERR),
    "tessl_buffer_write": (C.c_int32, [_RT, Buf, C.c_uint64, C.c_void_p, C.c_uint64] + _ERR),
    "tessl_buffer_read": (C.c_int32, [_RT, Buf, C.c_uint64, C.c_void_p, C.c_uint64] + _ERR),
    "tessl_simd_gemv_threadgroups": (C.c_uint64, [_u32]),
    "tessl_gemv_q4_mlx_simd": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32, C.POINTER(Buf)] + _ERR),
    "tessl_gemv_q4_mlx_simd_bf16": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32, C.POINTER(Buf)] + _ERR),
    "tessl_gemv_q4_mlx_gate_up_silu": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, Buf, QuantShape, _u32] + _ERR),
    "tessl_gemv_q4_mlx_gate_up_gelu": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, Buf, QuantShape, _u32, _u32] + _ERR),
    "tessl_gemv_q4_mlx_kv": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, Buf, Buf, QuantShape, _u32] + _ERR),
    "tessl_gemv_q4_mlx_qkv": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Q4MlxBank, Buf, QkvOutputs, _u32, _u32, _u32,
                                           _u32, _u32] + _ERR),
    "tessl_swiglu": (C.c_int32, [_RT, Buf, Buf, Buf, _u32, _u32] + _ERR),
    "tessl_gemm_q4_mlx": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32, _u32, C.POINTER(Buf)] + _ERR),
    "tessl_gemm_q4_mlx_bf16": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32, _u32, C.POINTER(Buf)] + _ERR),
    "tessl_gemm_q4_mlx_tensorops_max_k": (_u32, [_u32, _u32, _u32]),
    "tessl_gemm_q4_mlx_tensorops": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32] + _ERR),
    "tessl_gemm_q4_mlx_tensorops_bf16": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32] + _ERR),
    "tessl_gemm_q4_mlx_tensorops_noalloc": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, QuantShape, _u32] + _ERR),
    "tessl_peer_gather": (C.c_int32, [_RT, C.POINTER(PeerGather)] + _ERR),
    "tessl_gemv_q4_mlx_simd_sharded_deferred": (C.c_int32, [_RT, Q4MlxBank, Buf, C.POINTER(PeerGather), QuantShape, _u32] + _ERR),
    "tessl_gemv_q4_mlx_gate_up_silu_sharded_deferred": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, C.POINTER(PeerGather),
                                                                    QuantShape, _u32] + _ERR),
    "tessl_gemv_q4_mlx_simd_gathered": (C.c_int32, [_RT, Q4MlxBank, C.POINTER(PeerGather), Buf, QuantShape, C.POINTER(Buf),
                                                    _u32] + _ERR),
    "tessl_peer_wait": (C.c_int32, [_RT, C.POINTER(PeerGather)] + _ERR),
    "tessl_gemv_q4_mlx_simd_sharded": (C.c_int32, [_RT, Q4MlxBank, Buf, C.POINTER(PeerGather), QuantShape, _u32] + _ERR),
    "tessl_gemv_q4_mlx_gate_up_silu_sharded": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, C.POINTER(PeerGather), QuantShape,
                                                           _u32] + _ERR),
    "tessl_q4_weight_matmul": (C.c_int32, [_RT, Q4MlxBank, _u32, _u32, Buf, _u32, Buf, C.POINTER(Buf)] + _ERR),
    "tessl_q4_weight_gate_up_silu": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, _u32, _u32, Buf, Buf, _u32] + _ERR),
    "tessl_gemv_q8": (C.c_int32, [_RT, Buf, Buf, Buf, Buf, Buf, _u32, _u32, _u32] + _ERR),
    "tessl_gemm_q8_mlx": (C.c_int32, [_RT, Buf, Buf, Buf, Buf, QuantShape, _u32, _u32] + _ERR),
    "tessl_embed_lookup_q4_mlx": (C.c_int32, [_RT, Q4MlxBank, Buf, Buf, _u32, _u32, _u32, _u32] + _ERR),
    "tessl_qwen35_rms_norm": (C.c_int32, [_RT, Buf, Buf, Buf, _u32, _u32, _u32, C.c_float] + _ERR),
    "tessl_qwen35_residual_add": (C.c_int32, [_RT, Buf, Buf, _u32, _u32] + _ERR),
    "tessl_qwen35_add_rms_norm": (C.c_int32, [_RT, Buf, Buf, Buf, Buf, _u32, _u32, _u32, C.c_float] + _ERR),
    "tessl_checkpoint_open": (C.c_void_p, [C.c_char_p] + _ERR),
    "tessl_checkpoint_close": (None, [C.c_void_p]),
    "tessl_checkpoint_tensor_count": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64)] + _ERR),
    "tessl_checkpoint_tensor_name": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_char_p, C.c_size_t] + _ERR),
    "tessl_checkpoint_tensor_info": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(TensorInfo)] + _ERR),
    "tessl_mlx_quant_from_config_json": (C.c_int32, [C.c_char_p, C.POINTER(_u32), C.POINTER(_u32)] + _ERR),
    "tessl_mlx_names_detect": (C.c_int32, [C.POINTER(C.c_char_p), C.c_uint64, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p)] + _ERR),
    "tessl_mlx_norm_convention_from_conv_shape": (C.c_int32, [C.c_char_p, C.POINTER(C.c_uint64), _u32, C.c_uint64, C.c_uint64,
                                                              C.POINTER(_u32)] + _ERR),
    "tessl_mlx_classify_outside": (C.c_int32, [C.POINTER(C.c_char_p), C.c_uint64, C.POINTER(C.c_uint8)] + _ERR),
    "tessl_mlx_q4_check_part": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_uint64, C.c_uint64] + _ERR),
    "tessl_mlx_q4_read_bank": (C.c_int32, [C.c_void_p, C.POINTER(C.c_char_p), C.POINTER(C.c_uint64), _u32, C.c_uint64,
                                           C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64] + _ERR),
    "tessl_mlx_q4_load_bank": (C.c_int32, [_RT, C.c_void_p, C.POINTER(C.c_char_p), C.POINTER(C.c_uint64), _u32, C.c_uint64,
                                           Q4MlxBank] + _ERR),
    "tessl_q4_mlx_staged_bytes": (C.c_uint64, [_u32, _u32, _u32]),
    "tessl_q4_mlx_repack_staged": (C.c_int32, [_RT, Q4MlxBank, QuantShape, Buf] + _ERR),
    "tessl_gemv_q4_mlx_gate_up_silu_layout": (C.c_int32, [_RT, Q4MlxBank, Q4MlxBank, Buf, Buf, QuantShape, _u32, _u32] + _ERR),
    "tessl_q4_mlx_unpack": (C.c_int32, [_RT, Q4MlxBank, QuantShape, Buf] + _ERR),
    "tessl_q4_mlx_dequant": (C.c_int32, [_RT, Q4MlxBank, QuantShape, Buf] + _ERR),
}

_lib = None


def load() -> C.CDLL:
    """The shared library, loaded once. Raises if it is absent or of another ABI."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tessl_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    got = lib.tessl_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI {got}, this binding expects {ABI_VERSION}")
    _lib = lib
    return lib


ERR_LEN = 1024


_fn_cache: dict = {}
_err_local = threading.local()


def call(name: str, *args) -> None:
    """Call a status-returning entry; raise TesslError with the library's message.

    The error buffer is per thread and reused (a decode loop makes several calls per
    token; allocating 1 KiB each time showed up in the end-to-end timing)."""
    fn = _fn_cache.get(name)
    if fn is None:
        fn = _fn_cache[name] = getattr(load(), name)
    err = getattr(_err_local, "buf", None)
    if err is None:
        err = _err_local.buf = C.create_string_buffer(ERR_LEN)
    st = fn(*args, err, ERR_LEN)
    if st != TESSL_OK:
        raise TesslError(st, err.value.decode("utf-8", "replace"))
