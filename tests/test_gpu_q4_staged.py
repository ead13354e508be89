"""The offline repack for the B200 GEMV kernel (`tessl_q4_mlx_repack_staged`, layout TESSL_Q4_B200_STAGED): the role
the reference's Interleaved4 plays on Apple GPUs, tested the way the reference tests that one
(tests/q4_interleaved.rs:54-83 of the reference project): the device repack against a host repack oracle bit for
bit, and every operator that takes the layout against the same operator on the row-major bank, bit for bit."""
import numpy as np
import pytest

from gpu_util import SENTINEL_F32, rt, seeded_f32, upload_bank  # noqa: F401
from oracle import api
from tessl_b200 import capi, nn, synth

pytestmark = pytest.mark.gpu

SHAPES = [(16, 4096, 64), (13, 1024, 32), (5, 2048, 128), (1000, 4096, 128), (264, 2048, 64), (12288, 4096, 64),
          (4100, 4096, 32), (777, 1024, 64)]


@pytest.mark.parametrize("rows,cols,group", SHAPES)
def test_the_device_repack_is_the_oracle_repack(rt, rows, cols, group):
    packed, sb = synth.q4_bank(0x57A6E0 + rows, rows, cols, group)
    bank = upload_bank(rt, packed, sb)
    staged = nn.q4_mlx_repack_staged(rt, bank, nn.QuantShape(rows, cols, group))
    want = api.q4_repack_b200_staged(packed, sb, rows, cols, group)
    assert staged.packed.nbytes >= want.size
    assert np.array_equal(staged.packed.read(np.uint8, want.size), want)


@pytest.mark.parametrize("rows,cols,group", SHAPES)
def test_every_operator_that_takes_the_layout_returns_the_row_major_bits(rt, rows, cols, group):
    shape = nn.QuantShape(rows, cols, group)
    gp, gs = synth.q4_bank(0x57A6E1 + rows, rows, cols, group)
    up, us = synth.q4_bank(0x57A6E2 + rows, rows, cols, group)
    gate, upb = upload_bank(rt, gp, gs), upload_bank(rt, up, us)
    sgate, sup = nn.q4_mlx_repack_staged(rt, gate, shape), nn.q4_mlx_repack_staged(rt, upb, shape)
    x = rt.buffer_from(synth.normal_bf16(0x57A6E3 + cols, cols))
    resid = synth.unit_from_draws(synth.splitmix_draws(0x57A6E4, rows))
    for bf16 in (False, True):
        dt, esz = (np.uint16, 2) if bf16 else (np.uint32, 4)
        a, b = rt.buffer_from(np.full(rows + 8, 0xA5A5A5A5, np.uint32)), rt.buffer_from(np.full(rows + 8, 0xA5A5A5A5, np.uint32))
        rt.take_dispatch_count()
        nn.gemv_q4_mlx_simd(rt, sgate, x, a, shape, layout=nn.B200_STAGED, y_as_bf16=bf16)
        assert rt.take_dispatch_count() == 1
        nn.gemv_q4_mlx_simd(rt, gate, x, b, shape, y_as_bf16=bf16)
        assert np.array_equal(a.read(np.uint8, (rows + 8) * 4), b.read(np.uint8, (rows + 8) * 4)), f"gemv bf16={bf16}"
        nn.gemv_q4_mlx_gate_up_silu(rt, sgate, sup, x, a, shape, bf16, layout=nn.B200_STAGED)
        nn.gemv_q4_mlx_gate_up_silu(rt, gate, upb, x, b, shape, bf16)
        assert np.array_equal(a.read(dt, rows), b.read(dt, rows)), f"gate/up silu bf16={bf16}"
        nn.gemv_q4_mlx_gate_up_gelu(rt, sgate, sup, x, a, shape, nn.B200_STAGED, bf16)
        nn.gemv_q4_mlx_gate_up_gelu(rt, gate, upb, x, b, shape, nn.ROW_MAJOR, bf16)
        assert np.array_equal(a.read(dt, rows), b.read(dt, rows)), f"gate/up gelu bf16={bf16}"
    # add-residual with y == resid
    ra, rb = rt.buffer_from(resid), rt.buffer_from(resid)
    nn.gemv_q4_mlx_simd(rt, sgate, x, ra, shape, layout=nn.B200_STAGED, resid=ra)
    nn.gemv_q4_mlx_simd(rt, gate, x, rb, shape, resid=rb)
    assert np.array_equal(ra.read(np.uint32, rows), rb.read(np.uint32, rows))


def test_refusals_before_any_launch(rt):
    rows, cols, group = 64, 1024, 64
    packed, sb = synth.q4_bank(9, rows, cols, group)
    bank = upload_bank(rt, packed, sb)
    shape = nn.QuantShape(rows, cols, group)
    staged = nn.q4_mlx_repack_staged(rt, bank, shape)
    x = rt.buffer_from(synth.normal_bf16(10, 8 * cols))
    y = seeded_f32(rt, 8 * rows)
    # a bank that lives inside the buffer it would be repacked into
    big = rt.alloc_buffer(nn.q4_mlx_staged_bytes(rows, cols, group) + packed.nbytes)
    big.write(packed.view(np.uint8).reshape(-1))
    inside = nn.Q4MlxBank(big.view(0, packed.nbytes), bank.scales_biases)
    rt.take_dispatch_count()
    only = "taken by the one-row GEMV and gate/up entries only"
    cases = [
        (lambda: nn.gemv_q4_mlx_kv(rt, staged, staged, x, y, y.view(0, rows * 4), shape, nn.B200_STAGED), only),
        (lambda: nn.gemm_q4_mlx(rt, staged, x, y, shape, 4, nn.B200_STAGED), only),
        (lambda: nn.gemv_q4_mlx_simd(rt, staged, x, y, nn.QuantShape(rows, 1536, 64), layout=nn.B200_STAGED), "staged layout exists for"),
        (lambda: nn.gemv_q4_mlx_simd(rt, staged, x, y, nn.QuantShape(rows + 8, cols, group), layout=nn.B200_STAGED), "staged image"),
        (lambda: nn.gemv_q4_mlx_simd(rt, nn.Q4MlxBank(staged.packed.view(8, staged.packed.nbytes - 8), nn.GpuBuffer(0, 0)), x, y,
                                     nn.QuantShape(rows - 8, cols, group), layout=nn.B200_STAGED), "16-byte aligned"),
        (lambda: nn.gemv_q4_mlx_simd(rt, staged, x, y, shape, layout=7), "unknown layout 7"),
        (lambda: capi.call("tessl_q4_mlx_repack_staged", rt.handle, bank.c(), nn.QuantShape(rows, cols, 256).c(), y.c()), "staged layout exists for"),
        (lambda: capi.call("tessl_q4_mlx_repack_staged", rt.handle, bank.c(), shape.c(), y.view(0, 64).c()), " out"),
        (lambda: capi.call("tessl_q4_mlx_repack_staged", rt.handle, inside.c(), shape.c(), big.c()), "overlaps"),
    ]
    for fn, want in cases:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), (want, str(e.value))
    assert rt.take_dispatch_count() == 0
    assert np.all(y.read(np.float32, 8 * rows) == SENTINEL_F32)
