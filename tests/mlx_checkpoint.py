"""A synthetic mlx-lm-layout checkpoint writer for the loader tests (test infrastructure).

mlx-lm stores one quantized [rows, cols] matrix as `X.weight` U32 [rows, cols/8], `X.scales` and
`X.biases` BF16 [rows, cols/64]; q/k/v and gate/up are separate tensors that the loader concatenates
by rows (tests/qwen35_mlx_q4.rs:268-307 of the reference builds the same entries in memory).
"""
import json
import struct

import numpy as np

from tessl_b200 import synth

PREFIX = "language_model.model.layers.0"
# (suffix, rows, cols) of one small layer: hidden 128, q 256 rows, k/v 64 rows, intermediate 192
LAYER = [
    ("self_attn.q_proj", 256, 128), ("self_attn.k_proj", 64, 128), ("self_attn.v_proj", 64, 128),
    ("self_attn.o_proj", 128, 256), ("mlp.gate_proj", 192, 128), ("mlp.up_proj", 192, 128), ("mlp.down_proj", 128, 192),
]


def entries(seed=7):
    """[(name, dtype, shape, bytes)] in mlx-lm's layout, and {suffix: (packed, pairs)} of what was written."""
    out, banks = [], {}
    for i, (suffix, rows, cols) in enumerate(LAYER):
        packed, sb = synth.q4_bank(seed + 10 * i, rows, cols, 64)
        banks[suffix] = (packed, sb)
        base = f"{PREFIX}.{suffix}"
        out.append((base + ".weight", "U32", [rows, cols // 8], packed.tobytes()))
        out.append((base + ".scales", "BF16", [rows, cols // 64], np.ascontiguousarray(sb[..., 0]).tobytes()))
        out.append((base + ".biases", "BF16", [rows, cols // 64], np.ascontiguousarray(sb[..., 1]).tobytes()))
    norm = np.zeros(128, np.float32)
    out.append((f"{PREFIX}.input_layernorm.weight", "F32", [128], norm.tobytes()))
    return out, banks


def write(path, ents, metadata=None, pad_header_to=8, raw_header=None):
    """Write `ents` as a safetensors file; `raw_header` replaces the generated JSON (for malformed-file cases)."""
    header, offset, blobs = {}, 0, []
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dtype, shape, data in ents:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
        blobs.append(data)
    text = (json.dumps(header, separators=(",", ":")) if raw_header is None else raw_header).encode("utf-8")
    text += b" " * (-len(text) % pad_header_to)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)
    return path
