"""Inputs of the reference's known-answer test, regenerated from its seeds.

Follows tests/q4_kernels_template.rs:119-167 of the reference project: one
splitmix64 stream per tensor; a bank is `rows*cols/2` random bytes followed by
one (scale, bias) draw pair per group with scale = 0.002 + 0.05*|u| and
bias = 0.5*u in f32, rounded to bf16; x is 2*u rounded to bf16; a residual is u.
"""
import numpy as np

from tessl_b200 import synth

SENTINEL = 0xA5A5A5A5
PAD_WORDS = 8
SHAPES = [("r37c544g32", 37, 544, 32), ("r64c1024g64", 64, 1024, 64), ("r13c96g32", 13, 96, 32),
          ("r6c512g128", 6, 512, 128), ("r9c2112g64", 9, 2112, 64)]


def rand_bank(rows, cols, group, seed):
    nbytes = rows * cols // 2
    groups = rows * (cols // group)
    d = synth.splitmix_draws(seed, nbytes + 2 * groups)
    packed = ((d[:nbytes] >> np.uint64(32)) & np.uint64(0xFF)).astype(np.uint8)
    u = synth.unit_from_draws(d[nbytes:])
    scale = np.float32(0.002) + np.float32(0.05) * np.abs(u[0::2])
    bias = np.float32(0.5) * u[1::2]
    sb = np.empty(2 * groups, np.float32)
    sb[0::2], sb[1::2] = scale, bias
    return packed, synth.f32_to_bf16_bits(sb)


def rand_x(n, seed):
    return synth.f32_to_bf16_bits(synth.unit_from_draws(synth.splitmix_draws(seed, n)) * np.float32(2.0))


def rand_f32(n, seed):
    return synth.unit_from_draws(synth.splitmix_draws(seed, n))


def sentinel(words):
    return np.full(words, SENTINEL, np.uint32)
