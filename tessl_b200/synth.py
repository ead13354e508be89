"""Seeded synthetic inputs for the MLX affine-quantized matmul path.

Real MLX-Q4 checkpoints are not available offline, so benchmarks and tests
draw every tensor from a splitmix64 stream. The generator is the one the
reference's tests use (tests/common/mod.rs:153-180 and
tests/qwen35_mlx_q4.rs:40-64 in the reference project): the state starts at
`seed ^ GAMMA`, every draw adds GAMMA and mixes. Draw i therefore depends only
on `seed` and `i`, which lets numpy produce a whole tensor at once.

bf16 values are carried as uint16 bit patterns; rounding is to nearest even
(src/tensor.rs:804-813 in the reference project).
"""
from __future__ import annotations

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix_draws(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Draws `start .. start+n` of the stream seeded with `seed`, as uint64."""
    with np.errstate(over="ignore"):
        s0 = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) ^ GAMMA
        idx = np.arange(start + 1, start + n + 1, dtype=np.uint64)
        z = s0 + idx * GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def unit_from_draws(d: np.ndarray) -> np.ndarray:
    """Uniform in [-1, 1): top 24 bits over 2^23, minus one, in f32."""
    return (d >> np.uint64(40)).astype(np.float32) / np.float32(8388608.0) - np.float32(1.0)


def uniform01_from_draws(d: np.ndarray) -> np.ndarray:
    """Uniform in (0, 1) as f64: (top 24 bits + 0.5) / 2^24."""
    return ((d >> np.uint64(40)).astype(np.float64) + 0.5) / 16777216.0


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32)
    nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    rounded = ((bits.astype(np.uint64) + 0x7FFF + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint64(16)).astype(np.uint16)
    quiet = ((bits >> np.uint32(16)) | np.uint32(0x0040)).astype(np.uint16)
    return np.where(nan, quiet, rounded)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16(seed: int, n: int) -> np.ndarray:
    """N(0,1) by Box-Muller in f64, rounded f64 -> f32 -> bf16; uint16 bits."""
    pairs = (n + 1) // 2
    d = splitmix_draws(seed, 2 * pairs)
    u1 = uniform01_from_draws(d[0::2])
    u2 = uniform01_from_draws(d[1::2])
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.empty(2 * pairs, np.float64)
    z[0::2] = r * np.cos(2.0 * np.pi * u2)
    z[1::2] = r * np.sin(2.0 * np.pi * u2)
    return f32_to_bf16_bits(z[:n].astype(np.float32))


def q4_bank(seed: int, rows: int, cols: int, group: int = 64, scale_lo: float = 0.002, scale_hi: float = 0.02,
            bias_noise: float = 0.001):
    """One MLX Q4 bank: (packed uint32 [rows, cols/8], scales_biases uint16 [rows, cols/group, 2]).

    Nibbles are uniform 0..15 (the top four bits of a draw), packed eight per
    little-endian uint32 with element i at bits 4i..4i+4. scale ~ U(lo, hi) and
    bias = -8 * scale + N(0, bias_noise), both rounded to bf16 and stored as
    adjacent (scale, bias) pairs.
    """
    n = rows * cols
    nib = (splitmix_draws(seed, n) >> np.uint64(60)).astype(np.uint32).reshape(rows, cols // 8, 8)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    packed = np.bitwise_or.reduce(nib << shifts, axis=2).astype(np.uint32)
    groups = rows * (cols // group)
    d = splitmix_draws(seed + 1, 3 * groups)
    u = uniform01_from_draws(d[:groups])
    scale = (scale_lo + u * (scale_hi - scale_lo)).astype(np.float32)
    scale_b = f32_to_bf16_bits(scale)
    u1 = uniform01_from_draws(d[groups:2 * groups])
    u2 = uniform01_from_draws(d[2 * groups:])
    noise = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * bias_noise
    bias = (-8.0 * bf16_bits_to_f32(scale_b).astype(np.float64) + noise).astype(np.float32)
    sb = np.empty((rows, cols // group, 2), np.uint16)
    sb[..., 0] = scale_b.reshape(rows, -1)
    sb[..., 1] = f32_to_bf16_bits(bias).reshape(rows, -1)
    return packed, sb


def q8_bank(seed: int, rows: int, cols: int, group: int = 64, scale_lo: float = 0.0005, scale_hi: float = 0.005):
    """One MLX-layout Q8 bank: (codes uint32 [rows, cols/4], scales_biases uint16 [rows, cols/group, 2]).

    Codes are uniform 0..255 (the top byte of a draw) packed four per uint32,
    low byte first; scale ~ U(lo, hi) in bf16; bias = -128 * scale (exact in bf16).
    """
    n = rows * cols
    codes = (splitmix_draws(seed, n) >> np.uint64(56)).astype(np.uint8).reshape(rows, cols)
    packed = codes.view(np.uint32) if codes.flags["C_CONTIGUOUS"] else np.ascontiguousarray(codes).view(np.uint32)
    groups = rows * (cols // group)
    u = uniform01_from_draws(splitmix_draws(seed + 1, groups))
    scale_b = f32_to_bf16_bits((scale_lo + u * (scale_hi - scale_lo)).astype(np.float32))
    bias = (-128.0 * bf16_bits_to_f32(scale_b)).astype(np.float32)
    sb = np.empty((rows, cols // group, 2), np.uint16)
    sb[..., 0] = scale_b.reshape(rows, -1)
    sb[..., 1] = f32_to_bf16_bits(bias).reshape(rows, -1)
    return packed.reshape(rows, cols // 4), sb
