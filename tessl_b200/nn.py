"""Host-side mirror of the reference's typed kernel API for the MLX quantized path.

Names, argument order and refusals follow `src/nn.rs` and `src/qwen35_q4.rs`
of the reference project (`nn::gemv_q4_mlx_simd`, `nn::gemm_q4_mlx`,
`nn::gemm_q4_mlx_tensorops`, `nn::gemv_q8`, `Q4Weight::matmul`, ...); every
function forwards to the C ABI of `libtessl_b200.so`, where validation and the
CUDA launches live. A refusal surfaces as `TesslError` carrying the library's
message. Nothing here computes: without the CUDA library the import fails.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import capi
from .capi import Buf, Q4MlxBank as _CBank, QkvOutputs as _CQkv, QuantShape as _CShape, TesslError  # noqa: F401

ROW_MAJOR = capi.ROW_MAJOR
B200_STAGED = capi.B200_STAGED
INTERLEAVED4 = capi.INTERLEAVED4
GEMM_Q4_MLX_MAX_M = capi.GEMM_Q4_MLX_MAX_M
GEMM_Q4_MLX_TENSOROPS_GROUP_SIZES = (32, 64, 128)


@dataclass(frozen=True)
class QuantShape:
    """`nn::QuantShape` (src/nn.rs:3238-3245)."""
    rows: int
    cols: int
    group_size: int

    def c(self) -> _CShape:
        cached = self.__dict__.get("_c")  # the ctypes struct is built once (frozen dataclass: fields never change)
        if cached is None:
            cached = _CShape(self.rows, self.cols, self.group_size)
            object.__setattr__(self, "_c", cached)
        return cached


class GpuBuffer:
    """Device memory with a capacity, the analogue of the reference's `GpuBuffer`.

    Either owned (allocated through the runtime) or a view of memory someone
    else owns, e.g. a torch tensor (`GpuBuffer.from_torch`)."""

    def __init__(self, ptr: int, nbytes: int, owner=None, rt: "Runtime | None" = None):
        self.ptr, self.nbytes, self._owner, self._rt = int(ptr or 0), int(nbytes), owner, rt
        self._c = None  # ctypes view, built on first use

    @staticmethod
    def from_torch(t) -> "GpuBuffer":
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("GpuBuffer.from_torch needs a contiguous CUDA tensor")
        return GpuBuffer(t.data_ptr(), t.numel() * t.element_size(), owner=t)

    def view(self, byte_offset: int, nbytes: int) -> "GpuBuffer":
        if byte_offset < 0 or nbytes < 0 or byte_offset + nbytes > self.nbytes:
            raise ValueError("view out of range")
        return GpuBuffer(self.ptr + byte_offset, nbytes, owner=self)

    def c(self) -> Buf:
        b = self._c
        if b is None or b.ptr != (self.ptr or None) or b.nbytes != self.nbytes:
            b = self._c = Buf(self.ptr, self.nbytes)
        return b

    def write(self, data: np.ndarray, byte_offset: int = 0) -> None:
        a = np.ascontiguousarray(data)
        capi.call("tessl_buffer_write", self._runtime().handle, self.c(), byte_offset,
                  a.ctypes.data_as(C.c_void_p), a.nbytes)

    def read(self, dtype, count: int, byte_offset: int = 0, out: "np.ndarray | None" = None) -> np.ndarray:
        """Reads `count` elements; into `out` if given (e.g. a view of pinned host memory, which makes the
        copy a plain DMA instead of a staged one)."""
        if out is None:
            out = np.empty(count, dtype)
        elif out.dtype != np.dtype(dtype) or out.size != count or not out.flags.c_contiguous:
            raise ValueError("out must be a contiguous array of `count` elements of `dtype`")
        capi.call("tessl_buffer_read", self._runtime().handle, self.c(), byte_offset,
                  out.ctypes.data_as(C.c_void_p), out.nbytes)
        return out

    def _runtime(self) -> "Runtime":
        b = self
        while b._rt is None and isinstance(b._owner, GpuBuffer):
            b = b._owner
        if b._rt is None:
            raise ValueError("this buffer was not allocated by a Runtime; copy through its owner instead")
        return b._rt

    def free(self) -> None:
        if self._rt is not None and self.ptr:
            capi.call("tessl_buffer_free", self._rt.handle, self.c())
            self.ptr, self.nbytes = 0, 0


@dataclass
class Q4MlxBank:
    """`nn::Q4MlxBank` (src/nn.rs:3332-3338): packed nibbles + bf16 (scale, bias) pairs."""
    packed: GpuBuffer
    scales_biases: GpuBuffer

    def c(self) -> _CBank:
        key = (self.packed.ptr, self.packed.nbytes, self.scales_biases.ptr, self.scales_biases.nbytes)
        cached = self.__dict__.get("_c")
        if cached is None or cached[0] != key:
            cached = (key, _CBank(self.packed.c(), self.scales_biases.c()))
            self.__dict__["_c"] = cached
        return cached[1]


@dataclass
class QkvOutputs:
    """`nn::QkvOutputs` (src/nn.rs:4408-4415)."""
    q_out: GpuBuffer
    k_out: GpuBuffer
    v_out: GpuBuffer

    def c(self) -> _CQkv:
        return _CQkv(self.q_out.c(), self.k_out.c(), self.v_out.c())


class Runtime:
    """A runtime handle (`tessl_runtime_new`): one device, one stream, thread-affine."""

    def __init__(self, device: Optional[int] = None):
        lib = capi.load()
        err = C.create_string_buffer(capi.ERR_LEN)
        h = (lib.tessl_runtime_new(err, capi.ERR_LEN) if device is None
             else lib.tessl_runtime_new_on_device(device, err, capi.ERR_LEN))
        if not h:
            raise TesslError(capi.TESSL_ERR, err.value.decode("utf-8", "replace"))
        self.handle = C.c_void_p(h)

    def close(self) -> None:
        if self.handle:
            capi.load().tessl_runtime_free(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def stream(self) -> int:
        return capi.load().tessl_runtime_stream(self.handle) or 0

    @property
    def device(self) -> int:
        return capi.load().tessl_runtime_device(self.handle)

    def synchronize(self) -> None:
        capi.call("tessl_synchronize", self.handle)

    def set_async_encode(self, on: bool) -> None:
        capi.call("tessl_runtime_set_async_encode", self.handle, int(on))

    def set_encode_only(self, on: bool) -> None:
        capi.call("tessl_runtime_set_encode_only", self.handle, int(on))

    def is_poisoned(self) -> bool:
        out = C.c_int32(0)
        capi.call("tessl_runtime_poisoned", self.handle, C.byref(out))
        return bool(out.value)

    def take_dispatch_count(self) -> int:
        out = C.c_uint64(0)
        capi.call("tessl_runtime_take_dispatch_count", self.handle, C.byref(out))
        return out.value

    def set_prefill_tile(self, tile_n: int = 0, pair: int = -1) -> None:
        """Force the prefill GEMM's tile width (128 / 192 / 256, 0 = automatic) and kernel
        (1 = CTA pair, 0 = single CTA, -1 = automatic) for later calls on this runtime."""
        capi.call("tessl_runtime_set_prefill_tile", self.handle, tile_n, pair)

    def last_prefill_tile(self) -> tuple:
        """(tile width, pair) the most recent prefill GEMM call launched; (0, 0) if it ran no tile kernel."""
        bn, pair = C.c_uint32(0), C.c_uint32(0)
        capi.call("tessl_runtime_last_prefill_tile", self.handle, C.byref(bn), C.byref(pair))
        return bn.value, pair.value

    def set_peer_wait_limit(self, clocks: int) -> None:
        """Clock budget of bounded waits on another GPU's flags (0 = the default, about 0.5 s)."""
        capi.call("tessl_runtime_set_peer_wait_limit", self.handle, clocks)

    def alloc_buffer(self, nbytes: int) -> GpuBuffer:
        b = Buf()
        capi.call("tessl_buffer_alloc", self.handle, nbytes, C.byref(b))
        return GpuBuffer(b.ptr, b.nbytes, rt=self)

    def buffer_from(self, data: np.ndarray) -> GpuBuffer:
        a = np.ascontiguousarray(data)
        buf = self.alloc_buffer(a.nbytes)
        if a.nbytes:
            buf.write(a)
        return buf

    def bank_from(self, packed: np.ndarray, scales_biases: np.ndarray) -> Q4MlxBank:
        return Q4MlxBank(self.buffer_from(packed), self.buffer_from(scales_biases))


def _opt(buf: Optional[GpuBuffer]):
    return None if buf is None else C.byref(buf.c())


def simd_gemv_threadgroups(rows: int) -> int:
    """`nn::simd_gemv_threadgroups` (src/nn.rs:3699-3701)."""
    return capi.load().tessl_simd_gemv_threadgroups(rows)


def gemv_q4_mlx_simd(rt: Runtime, bank: Q4MlxBank, x_bf16: GpuBuffer, y: GpuBuffer, shape: QuantShape,
                     layout: int = ROW_MAJOR, resid: Optional[GpuBuffer] = None, *, y_as_bf16: bool = False) -> None:
    """`nn::gemv_q4_mlx_simd` (src/nn.rs:3982-4074). `y_as_bf16` selects the bf16-output twin."""
    name = "tessl_gemv_q4_mlx_simd_bf16" if y_as_bf16 else "tessl_gemv_q4_mlx_simd"
    capi.call(name, rt.handle, bank.c(), x_bf16.c(), y.c(), shape.c(), layout, _opt(resid))


def gemv_q4_mlx_gate_up_silu(rt: Runtime, gate: Q4MlxBank, up: Q4MlxBank, x: GpuBuffer, mid: GpuBuffer,
                             shape: QuantShape, mid_as_bf16: bool, layout: int = ROW_MAJOR) -> None:
    """`nn::gemv_q4_mlx_gate_up_silu` (src/nn.rs:4165-4194); `layout` other than row-major goes through the
    library's own entry with a layout argument."""
    if layout == ROW_MAJOR:
        capi.call("tessl_gemv_q4_mlx_gate_up_silu", rt.handle, gate.c(), up.c(), x.c(), mid.c(), shape.c(),
                  int(mid_as_bf16))
    else:
        capi.call("tessl_gemv_q4_mlx_gate_up_silu_layout", rt.handle, gate.c(), up.c(), x.c(), mid.c(), shape.c(), layout,
                  int(mid_as_bf16))


def q4_mlx_staged_bytes(rows: int, cols: int, group_size: int) -> int:
    """Size of the B200 staged image of a bank; 0 for a shape the layout does not exist for."""
    return int(capi.load().tessl_q4_mlx_staged_bytes(rows, cols, group_size))


def q4_mlx_repack_staged(rt: Runtime, bank: Q4MlxBank, shape: QuantShape) -> Q4MlxBank:
    """The bank repacked offline into the B200 staged layout (`tessl_q4_mlx_repack_staged`): pass the result with
    `layout=B200_STAGED` to the one-row GEMV and gate/up operators. Results are those of the row-major bank."""
    nbytes = q4_mlx_staged_bytes(shape.rows, shape.cols, shape.group_size)
    if nbytes == 0 and shape.rows:
        raise ValueError("the B200 staged layout exists for rows of 1024, 2048 or 4096 columns and groups of 32, 64 or 128")
    out = rt.alloc_buffer(nbytes)
    capi.call("tessl_q4_mlx_repack_staged", rt.handle, bank.c(), shape.c(), out.c())
    return Q4MlxBank(out, GpuBuffer(0, 0))


def gemv_q4_mlx_gate_up_gelu(rt: Runtime, gate: Q4MlxBank, up: Q4MlxBank, x: GpuBuffer, mid: GpuBuffer,
                             shape: QuantShape, layout: int, mid_as_bf16: bool) -> None:
    """`nn::gemv_q4_mlx_gate_up_gelu` with `GateUpDispatch::Simd(layout)` (src/nn.rs:4098-4155)."""
    capi.call("tessl_gemv_q4_mlx_gate_up_gelu", rt.handle, gate.c(), up.c(), x.c(), mid.c(), shape.c(), layout,
              int(mid_as_bf16))


def gemv_q4_mlx_kv(rt: Runtime, k: Q4MlxBank, v: Q4MlxBank, x_bf16: GpuBuffer, k_out: GpuBuffer, v_out: GpuBuffer,
                   shape: QuantShape, layout: int = ROW_MAJOR) -> None:
    """`nn::gemv_q4_mlx_kv` (src/nn.rs:4279-4351)."""
    capi.call("tessl_gemv_q4_mlx_kv", rt.handle, k.c(), v.c(), x_bf16.c(), k_out.c(), v_out.c(), shape.c(), layout)


def gemv_q4_mlx_qkv(rt: Runtime, q: Q4MlxBank, k: Q4MlxBank, v: Q4MlxBank, x_bf16: GpuBuffer, out: QkvOutputs,
                    rows_q: int, rows_kv: int, cols: int, group_size: int, layout: int = ROW_MAJOR) -> None:
    """`nn::gemv_q4_mlx_qkv` (src/nn.rs:4366-4515)."""
    capi.call("tessl_gemv_q4_mlx_qkv", rt.handle, q.c(), k.c(), v.c(), x_bf16.c(), out.c(), rows_q, rows_kv, cols,
              group_size, layout)


def swiglu(rt: Runtime, gate: GpuBuffer, up: GpuBuffer, out: GpuBuffer, n: int, out_as_bf16: bool) -> None:
    """`qwen35::swiglu` as the unfused gate/up path uses it (src/qwen35_model.rs:1938-1957)."""
    capi.call("tessl_swiglu", rt.handle, gate.c(), up.c(), out.c(), n, int(out_as_bf16))


def gemm_q4_mlx(rt: Runtime, bank: Q4MlxBank, x_bf16: GpuBuffer, y: GpuBuffer, shape: QuantShape, m: int,
                layout: int = ROW_MAJOR, resid: Optional[GpuBuffer] = None, *, y_as_bf16: bool = False) -> None:
    """`nn::gemm_q4_mlx` (src/nn.rs:4535-4619): m <= 8."""
    name = "tessl_gemm_q4_mlx_bf16" if y_as_bf16 else "tessl_gemm_q4_mlx"
    capi.call(name, rt.handle, bank.c(), x_bf16.c(), y.c(), shape.c(), m, layout, _opt(resid))


def gemm_q4_mlx_tensorops_max_k(m: int, n: int, group_size: int) -> int:
    """`nn::gemm_q4_mlx_tensorops_max_k` (src/nn.rs:4650-4655)."""
    return capi.load().tessl_gemm_q4_mlx_tensorops_max_k(m, n, group_size)


def gemm_q4_mlx_tensorops(rt: Runtime, bank: Q4MlxBank, x_bf16: GpuBuffer, y: GpuBuffer, shape: QuantShape, m: int,
                          *, y_as_bf16: bool = False) -> None:
    """`nn::gemm_q4_mlx_tensorops` (src/nn.rs:4683-4757): the prefill GEMM."""
    name = "tessl_gemm_q4_mlx_tensorops_bf16" if y_as_bf16 else "tessl_gemm_q4_mlx_tensorops"
    capi.call(name, rt.handle, bank.c(), x_bf16.c(), y.c(), shape.c(), m)


def gemm_q4_mlx_tensorops_noalloc(rt: Runtime, bank: Q4MlxBank, x_bf16: GpuBuffer, y: GpuBuffer, shape: QuantShape,
                                  m: int) -> None:
    """The prefill GEMM for callers that cannot allocate device memory (no counterpart in the
    reference): intermediate data goes to a fixed 8 MiB array inside the library, larger
    shapes are refused. See `tessl_gemm_q4_mlx_tensorops_noalloc` in include/tessl_b200.h."""
    capi.call("tessl_gemm_q4_mlx_tensorops_noalloc", rt.handle, bank.c(), x_bf16.c(), y.c(), shape.c(), m)


def gemv_q8(rt: Runtime, packed: GpuBuffer, scales: GpuBuffer, zeros: GpuBuffer, x: GpuBuffer, y: GpuBuffer,
            rows: int, cols: int, group_size: int) -> None:
    """`nn::gemv_q8` (src/nn.rs:716-795)."""
    capi.call("tessl_gemv_q8", rt.handle, packed.c(), scales.c(), zeros.c(), x.c(), y.c(), rows, cols, group_size)


def gemm_q8_mlx(rt: Runtime, codes: GpuBuffer, scales_biases: GpuBuffer, x_bf16: GpuBuffer, y: GpuBuffer,
                shape: QuantShape, m: int, y_as_bf16: bool = False) -> None:
    """MLX-layout 8-bit GEMV/GEMM for m <= 8 (no counterpart in the reference)."""
    capi.call("tessl_gemm_q8_mlx", rt.handle, codes.c(), scales_biases.c(), x_bf16.c(), y.c(), shape.c(), m,
              int(y_as_bf16))


def embed_lookup_q4_mlx(rt: Runtime, bank: Q4MlxBank, token_ids: GpuBuffer, out: GpuBuffer, vocab: int, hidden: int,
                        group_size: int, n_tokens: int) -> None:
    """`nn::embed_lookup_q4_mlx` (src/nn.rs:3592-3658): gather dequantized rows; ids >= vocab give zeros."""
    capi.call("tessl_embed_lookup_q4_mlx", rt.handle, bank.c(), token_ids.c(), out.c(), vocab, hidden, group_size,
              n_tokens)


def qwen35_rms_norm(rt: Runtime, x: GpuBuffer, w: GpuBuffer, out: GpuBuffer, out_as_bf16: bool, rows: int, dim: int,
                    eps: float) -> None:
    """`qwen35::rms_norm` (src/qwen35.rs:2654-2695): out = x * rsqrt(mean(x^2) + eps) * (1 + w)."""
    capi.call("tessl_qwen35_rms_norm", rt.handle, x.c(), w.c(), out.c(), int(out_as_bf16), rows, dim, eps)


def qwen35_residual_add(rt: Runtime, y: GpuBuffer, resid: GpuBuffer, rows: int, width: int) -> None:
    """`qwen35::residual_add` for dense operands (src/qwen35.rs:2586-2623): resid += y."""
    capi.call("tessl_qwen35_residual_add", rt.handle, y.c(), resid.c(), rows, width)


def qwen35_add_rms_norm(rt: Runtime, y: GpuBuffer, resid: GpuBuffer, w: GpuBuffer, out: GpuBuffer, out_as_bf16: bool,
                        rows: int, dim: int, eps: float) -> None:
    """`qwen35::add_rms_norm` (src/qwen35.rs:2697-2747): the add and the norm in one launch."""
    capi.call("tessl_qwen35_add_rms_norm", rt.handle, y.c(), resid.c(), w.c(), out.c(), int(out_as_bf16), rows, dim, eps)


def q4_mlx_unpack(rt: Runtime, bank: Q4MlxBank, shape: QuantShape, out_u8: GpuBuffer) -> None:
    capi.call("tessl_q4_mlx_unpack", rt.handle, bank.c(), shape.c(), out_u8.c())


def q4_mlx_dequant(rt: Runtime, bank: Q4MlxBank, shape: QuantShape, out_f32: GpuBuffer) -> None:
    capi.call("tessl_q4_mlx_dequant", rt.handle, bank.c(), shape.c(), out_f32.c())


class Q4Weight:
    """`Q4Weight` (src/qwen35_q4.rs:455-616): one group-64 bank and the M-dispatch policy."""

    def __init__(self, bank: Q4MlxBank, rows: int, cols: int):
        self.bank, self.rows, self.cols = bank, rows, cols

    def matmul(self, rt: Runtime, x_bf16: GpuBuffer, m: int, y: GpuBuffer, resid: Optional[GpuBuffer] = None) -> None:
        capi.call("tessl_q4_weight_matmul", rt.handle, self.bank.c(), self.rows, self.cols, x_bf16.c(), m, y.c(),
                  _opt(resid))

    def gate_up_silu(self, up: "Q4Weight", rt: Runtime, x_bf16: GpuBuffer, mid: GpuBuffer, mid_as_bf16: bool) -> None:
        if (self.rows, self.cols) != (up.rows, up.cols):
            raise TesslError(capi.TESSL_ERR, f"Q4Weight::gate_up_silu: gate is [{self.rows}, {self.cols}] but up is "
                                             f"[{up.rows}, {up.cols}]")
        capi.call("tessl_q4_weight_gate_up_silu", rt.handle, self.bank.c(), up.bank.c(), self.rows, self.cols,
                  x_bf16.c(), mid.c(), int(mid_as_bf16))
