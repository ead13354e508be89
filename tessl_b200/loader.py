"""MLX 4-bit checkpoints -> Q4 banks (host mirror of the reference's `Loader::mlx_q4` path).

`Checkpoint` wraps the library's safetensors reader; `MlxQuant.from_config_json`, `check_part`,
`Checkpoint.mlx_q4` and `Checkpoint.mlx_q4_named` carry the names, argument meaning and refusals
of `src/qwen35_q4.rs:204-255, 384-449` and `src/loader.rs:236-318` of the reference. All parsing
and checking happens inside the shared library; this file only marshals arguments.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from . import capi
from .capi import TensorInfo as _CInfo
from .nn import Q4MlxBank, Runtime

MLX_Q4_BITS = 4
MLX_Q4_GROUP = 64
NIBBLES_PER_WORD = 8


def sidecar_names(weight_name: str):
    """`X.weight` -> (`X.scales`, `X.biases`); None for a name that does not end in `.weight`."""
    if not weight_name.endswith(".weight"):
        return None
    base = weight_name[: -len(".weight")]
    return base + ".scales", base + ".biases"


@dataclass(frozen=True)
class MlxQuant:
    """A checkpoint's quantization as its config.json declares it."""

    bits: int
    group_size: int

    @staticmethod
    def from_config_json(text: str) -> "MlxQuant":
        bits, group = C.c_uint32(0), C.c_uint32(0)
        capi.call("tessl_mlx_quant_from_config_json", text.encode("utf-8"), C.byref(bits), C.byref(group))
        return MlxQuant(bits.value, group.value)


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: tuple
    nbytes: int


def _parts(parts: Sequence):
    names = (C.c_char_p * len(parts))(*[p[0].encode("utf-8") for p in parts])
    rows = (C.c_uint64 * len(parts))(*[int(p[1]) for p in parts])
    return names, rows


class Checkpoint:
    """One safetensors file, header parsed and verified, bytes memory-mapped."""

    def __init__(self, path):
        lib = capi.load()
        err = C.create_string_buffer(capi.ERR_LEN)
        self._h = lib.tessl_checkpoint_open(os.fsencode(path), err, capi.ERR_LEN)
        if not self._h:
            raise capi.TesslError(capi.TESSL_ERR, err.value.decode("utf-8", "replace"))

    def close(self) -> None:
        if self._h:
            capi.load().tessl_checkpoint_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def names(self) -> list:
        n = C.c_uint64(0)
        capi.call("tessl_checkpoint_tensor_count", self._h, C.byref(n))
        buf = C.create_string_buffer(4096)
        out = []
        for i in range(n.value):
            capi.call("tessl_checkpoint_tensor_name", self._h, i, buf, 4096)
            out.append(buf.value.decode("utf-8"))
        return out

    def tensor_info(self, name: str) -> TensorInfo:
        info = _CInfo()
        capi.call("tessl_checkpoint_tensor_info", self._h, name.encode("utf-8"), C.byref(info))
        return TensorInfo(info.dtype.decode("ascii"), tuple(info.shape[: info.ndim]), info.nbytes)

    def check_part(self, weight_name: str, rows: int, cols: int) -> None:
        capi.call("tessl_mlx_q4_check_part", self._h, weight_name.encode("utf-8"), rows, cols)

    def read_mlx_q4(self, parts: Sequence, cols: int):
        """The bank of `parts` = [(X.weight, rows), ...] as host arrays: (packed u32 [N, cols/8], pairs u16 [N, cols/64, 2])."""
        total = sum(int(p[1]) for p in parts)
        cols8, groups = max(cols // NIBBLES_PER_WORD, 0), max(cols // MLX_Q4_GROUP, 0)
        packed = np.zeros((total, cols8), dtype=np.uint32)
        pairs = np.zeros((total, groups, 2), dtype=np.uint16)
        names, rows = _parts(parts)
        capi.call("tessl_mlx_q4_read_bank", self._h, names, rows, len(parts), cols, packed.ctypes.data, packed.nbytes,
                  pairs.ctypes.data, pairs.nbytes)
        return packed, pairs

    def mlx_q4_named(self, rt: Runtime, parts: Sequence, cols: int) -> Q4MlxBank:
        """`Loader::mlx_q4_named`: the parts' rows concatenated into one device bank."""
        # the headers are verified before the device buffers are sized from the caller's numbers
        for name, rows in parts:
            self.check_part(name, int(rows), cols)
        total = sum(int(p[1]) for p in parts)
        packed = rt.alloc_buffer(total * cols // 2)
        pairs = rt.alloc_buffer(total * (cols // MLX_Q4_GROUP) * 4)
        bank = Q4MlxBank(packed, pairs)
        names, rows = _parts(parts)
        capi.call("tessl_mlx_q4_load_bank", rt.handle, self._h, names, rows, len(parts), cols, bank.c())
        return bank

    def mlx_q4(self, rt: Runtime, prefix: str, parts: Sequence, cols: int) -> Q4MlxBank:
        """`Loader::mlx_q4`: parts named by suffix under a layer prefix, e.g. ("self_attn.q_proj", rows)."""
        return self.mlx_q4_named(rt, [(f"{prefix}.{s}.weight", r) for s, r in parts], cols)


@dataclass(frozen=True)
class MlxNames:
    """How a checkpoint spells its tower (`MlxNames`, src/qwen35_q4.rs:258-293 of the reference)."""

    prefix: str
    head: str

    @staticmethod
    def detect(names: Sequence) -> "MlxNames":
        arr = (C.c_char_p * len(names))(*[n.encode("utf-8") for n in names])
        prefix, head = C.c_char_p(), C.c_char_p()
        capi.call("tessl_mlx_names_detect", arr, len(names), C.byref(prefix), C.byref(head))
        return MlxNames(prefix.value.decode("ascii"), head.value.decode("ascii"))


class NormConvention:
    """Whether the norm weights hold w (`HF`) or 1 + w (`MLX_SHIFTED`), read off a GDN layer's conv1d.weight
    (`NormConvention`, src/qwen35_q4.rs:296-336 of the reference)."""

    HF, MLX_SHIFTED = 0, 1

    @staticmethod
    def from_conv_shape(tensor: str, shape: Sequence, conv_dim: int, kernel: int) -> int:
        arr = (C.c_uint64 * len(shape))(*[int(d) for d in shape])
        out = C.c_uint32(0)
        capi.call("tessl_mlx_norm_convention_from_conv_shape", tensor.encode("utf-8"), arr, len(shape), conv_dim, kernel,
                  C.byref(out))
        return out.value

    @staticmethod
    def conv_shape(convention: int, conv_dim: int, kernel: int) -> tuple:
        return (conv_dim, 1, kernel) if convention == NormConvention.HF else (conv_dim, kernel, 1)

    @staticmethod
    def unshift(convention: int, stored) -> np.float32:
        """The value to hand a kernel that adds 1 itself, from a stored norm weight (f32 arithmetic)."""
        s = np.float32(stored)
        return s if convention == NormConvention.HF else np.float32(s - np.float32(1.0))


def classify_outside(unread: Sequence) -> dict:
    """`classify_outside` (src/qwen35_q4.rs:338-373): {"mtp": [...], "vision": [...]}; anything else is refused."""
    arr = (C.c_char_p * len(unread))(*[n.encode("utf-8") for n in unread])
    classes = (C.c_uint8 * max(len(unread), 1))()
    capi.call("tessl_mlx_classify_outside", arr, len(unread), classes)
    return {"mtp": [n for n, c in zip(unread, classes) if c == 0], "vision": [n for n, c in zip(unread, classes) if c == 1]}
