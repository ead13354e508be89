"""GPU parity of the operators either side of a decode projection, through the C ABI:
the Q4 embedding gather (`nn::embed_lookup_q4_mlx`), the zero-centred RMSNorm that produces the
bf16 activations (`qwen35::rms_norm`), the residual add and the two fused (`qwen35::add_rms_norm`).

Mirrors tests/nn_wiring.rs:339-387 (gather incl. an out-of-range id), tests/nn_aliasing.rs:222-229
(aliasing refusals) and the fused == unfused bit-for-bit promise of kernels/qwen35_mlp.metal:124-133 of
the reference project.
"""
import numpy as np
import pytest

from gpu_util import SENTINEL_F32, assert_north_star, rt, seeded_f32, upload_bank  # noqa: F401
from oracle import api
from tessl_b200 import nn, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vocab,hidden,group", [(64, 32, 32), (1000, 4096, 64), (77, 2560, 128), (300, 1024, 512)])
def test_embed_lookup_is_the_dequantized_row_bit_for_bit(rt, vocab, hidden, group):
    packed, sb = synth.q4_bank(0x7E550700 + vocab, vocab, hidden, group)
    packed, sb = packed.view(np.uint8).reshape(-1), sb.reshape(-1)
    bank = upload_bank(rt, packed, sb)
    ids = np.array([3, vocab - 1, 0, vocab + 5, 17 % vocab, 0xFFFFFFFF, vocab, 3], np.uint32)
    tb = rt.buffer_from(ids)
    pad = 64
    out = seeded_f32(rt, ids.size * hidden, pad)
    rt.take_dispatch_count()
    nn.embed_lookup_q4_mlx(rt, bank, tb, out, vocab, hidden, group, ids.size)
    assert rt.take_dispatch_count() == 1
    got = out.read(np.float32, ids.size * hidden + pad)
    assert np.all(got[ids.size * hidden:] == SENTINEL_F32), "wrote past out"
    want = api.embed_lookup_q4_mlx(packed, sb, ids, vocab, hidden, group)
    assert np.array_equal(got[: ids.size * hidden].view(np.uint32), want.reshape(-1).view(np.uint32))
    assert np.all(got[: ids.size * hidden].reshape(ids.size, hidden)[ids >= vocab] == 0.0)
    # the full table through the gather equals the dequantized bank (the bit-exact parity gate)
    all_ids = rt.buffer_from(np.arange(min(vocab, 256), dtype=np.uint32))
    n = min(vocab, 256)
    full = seeded_f32(rt, n * hidden)
    nn.embed_lookup_q4_mlx(rt, bank, all_ids, full, vocab, hidden, group, n)
    dq = api.q4_dequant(packed, sb, vocab, hidden, group)[:n]
    assert np.array_equal(full.read(np.uint32, n * hidden), dq.reshape(-1).view(np.uint32))


def test_embed_lookup_refusals_and_empty_calls(rt):
    vocab, hidden, group = 16, 64, 32
    packed, sb = synth.q4_bank(5, vocab, hidden, group)
    bank = upload_bank(rt, packed, sb)
    ids = rt.buffer_from(np.arange(4, dtype=np.uint32))
    out = seeded_f32(rt, 4 * hidden)
    rt.take_dispatch_count()
    small = rt.alloc_buffer(8)
    cases = [
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, ids, out, vocab, hidden, 0, 4), "group_size must be non-zero"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, ids, out, vocab, hidden, 48, 4), "multiple of group_size"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, ids, out, vocab, hidden, 16, 4), "MLX kernel domain"),
        (lambda: nn.embed_lookup_q4_mlx(rt, nn.Q4MlxBank(small, bank.scales_biases), ids, out, vocab, hidden, group, 4),
         "packed"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, small, out, vocab, hidden, group, 4), "token_ids"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, ids, small, vocab, hidden, group, 4), " out"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, ids, bank.packed, vocab, hidden, group, 1), "overlaps"),
        (lambda: nn.embed_lookup_q4_mlx(rt, bank, out, out, vocab, hidden, group, 4), "overlaps"),
    ]
    for fn, want in cases:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), (want, str(e.value))
    nn.embed_lookup_q4_mlx(rt, bank, ids, out, vocab, hidden, group, 0)  # validated no-op
    assert rt.take_dispatch_count() == 0
    assert np.all(out.read(np.float32, 4 * hidden) == SENTINEL_F32)


def _norm_inputs(rows, dim, seed):
    d = synth.splitmix_draws(seed, rows * dim * 2 + dim)
    x = synth.unit_from_draws(d[: rows * dim]) * np.float32(3.0)
    y = synth.unit_from_draws(d[rows * dim: 2 * rows * dim])
    w = synth.unit_from_draws(d[2 * rows * dim:]) * np.float32(0.5)
    return x, y, w


@pytest.mark.parametrize("rows,dim", [(1, 4096), (5, 4096), (3, 1000), (2, 37), (1, 12288)])
def test_rms_norm_matches_the_f64_reference_in_f32_and_bf16(rt, rows, dim):
    x, _, w = _norm_inputs(rows, dim, 0x7E550800 + dim)
    eps = 1e-6
    xb, wb = rt.buffer_from(x), rt.buffer_from(w)
    want = api.qwen35_rms_norm_f64(x, w, rows, dim, eps)
    of = seeded_f32(rt, rows * dim, 16)
    nn.qwen35_rms_norm(rt, xb, wb, of, False, rows, dim, eps)
    got = of.read(np.float32, rows * dim + 16)
    assert np.all(got[rows * dim:] == SENTINEL_F32)
    np.testing.assert_allclose(got[: rows * dim].reshape(rows, dim), want, rtol=2e-6, atol=1e-6)
    ob = rt.buffer_from(np.full(rows * dim + 16, 0xA5A5, np.uint16))
    nn.qwen35_rms_norm(rt, xb, wb, ob, True, rows, dim, eps)
    gb = ob.read(np.uint16, rows * dim + 16)
    assert np.all(gb[rows * dim:] == 0xA5A5)
    # the bf16 output is the f32 output rounded to nearest even, bit for bit
    assert np.array_equal(gb[: rows * dim], synth.f32_to_bf16_bits(got[: rows * dim]))
    # in place (f32): out may be x itself
    nn.qwen35_rms_norm(rt, xb, wb, xb, False, rows, dim, eps)
    assert np.array_equal(xb.read(np.uint32, rows * dim), got[: rows * dim].view(np.uint32))


@pytest.mark.parametrize("out_bf16", [False, True])
@pytest.mark.parametrize("rows,dim", [(1, 4096), (4, 4096), (3, 1000)])
def test_add_rms_norm_is_the_add_and_the_norm_bit_for_bit(rt, rows, dim, out_bf16):
    x, y, w = _norm_inputs(rows, dim, 0x7E550900 + dim + rows)
    eps = 1e-6
    esz = np.uint16 if out_bf16 else np.uint32
    wb, yb = rt.buffer_from(w), rt.buffer_from(y)
    # the two separate calls
    r1 = rt.buffer_from(x)
    o1 = rt.alloc_buffer(rows * dim * 4)
    nn.qwen35_residual_add(rt, yb, r1, rows, dim)
    nn.qwen35_rms_norm(rt, r1, wb, o1, out_bf16, rows, dim, eps)
    # the fused call
    r2 = rt.buffer_from(x)
    o2 = rt.alloc_buffer(rows * dim * 4)
    rt.take_dispatch_count()
    nn.qwen35_add_rms_norm(rt, yb, r2, wb, o2, out_bf16, rows, dim, eps)
    assert rt.take_dispatch_count() == 1
    assert np.array_equal(r1.read(np.uint32, rows * dim), r2.read(np.uint32, rows * dim))
    assert np.array_equal(r1.read(np.float32, rows * dim), (x + y).astype(np.float32))
    assert np.array_equal(o1.read(esz, rows * dim), o2.read(esz, rows * dim))
    want = api.qwen35_rms_norm_f64(x, w, rows, dim, eps, resid_add=y)
    got = o2.read(esz, rows * dim)
    gotf = synth.bf16_bits_to_f32(got) if out_bf16 else got.view(np.float32)
    np.testing.assert_allclose(gotf.reshape(rows, dim), want, rtol=8e-3 if out_bf16 else 2e-6, atol=1e-6)


def test_norm_refusals(rt):
    rows, dim = 2, 64
    x, y, w = _norm_inputs(rows, dim, 9)
    xb, yb, wb = rt.buffer_from(x), rt.buffer_from(y), rt.buffer_from(w)
    out = rt.alloc_buffer(rows * dim * 4)
    rt.take_dispatch_count()
    cases = [
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, out, False, rows, 0, 1e-6), "dim must be non-zero"),
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, out, False, rows, dim, 0.0), "eps must be finite and positive"),
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, out, False, rows, dim, float("nan")), "eps must be finite and positive"),
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, out, False, rows + 1, dim, 1e-6), "rms_norm x"),
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, xb, True, rows, dim, 1e-6), "overlaps"),
        (lambda: nn.qwen35_rms_norm(rt, xb, wb, wb, False, 1, dim, 1e-6), "overlaps"),
        (lambda: nn.qwen35_add_rms_norm(rt, yb, xb, wb, xb, False, rows, dim, 1e-6), "overlap"),
        (lambda: nn.qwen35_add_rms_norm(rt, xb, xb, wb, out, False, rows, dim, 1e-6), "overlaps"),
        (lambda: nn.qwen35_residual_add(rt, xb, xb, rows, dim), "overlaps"),
    ]
    for fn, want in cases:
        with pytest.raises(nn.TesslError) as e:
            fn()
        assert want in str(e.value), (want, str(e.value))
    nn.qwen35_rms_norm(rt, xb, wb, out, False, 0, dim, 1e-6)
    nn.qwen35_add_rms_norm(rt, yb, xb, wb, out, True, 0, dim, 1e-6)
    assert rt.take_dispatch_count() == 0


def test_an_mlp_block_is_three_launches_and_replays_from_a_graph(rt):
    """The steps either side of the projections in decode (src/qwen35_model.rs:1630-1687, 1938-1957 of the
    reference project): resid += y_prev; x = bf16(rms_norm(resid)); mid = bf16(silu(W_gate x) * (W_up x));
    resid += W_down mid. Three launches; every stage checked against the oracle with the same rounding points;
    then the same three calls captured once and replayed."""
    import torch

    hidden, inter, group, eps = 4096, 12288, 64, 1e-6
    gp, gs = synth.q4_bank(0x7E550A00, inter, hidden, group)
    up, us = synth.q4_bank(0x7E550A10, inter, hidden, group)
    dp, ds = synth.q4_bank(0x7E550A20, hidden, inter, group)
    gate, upb, down = upload_bank(rt, gp, gs), upload_bank(rt, up, us), upload_bank(rt, dp, ds)
    resid0, y_prev, w = _norm_inputs(1, hidden, 0x7E550A30)
    wb, yb = rt.buffer_from(w), rt.buffer_from(y_prev)
    resid = rt.buffer_from(resid0)
    xb = rt.alloc_buffer(hidden * 2)
    mid = rt.alloc_buffer(inter * 2)

    def block():
        nn.qwen35_add_rms_norm(rt, yb, resid, wb, xb, True, 1, hidden, eps)
        nn.gemv_q4_mlx_gate_up_silu(rt, gate, upb, xb, mid, nn.QuantShape(inter, hidden, group), True)
        nn.gemv_q4_mlx_simd(rt, down, mid, resid, nn.QuantShape(hidden, inter, group), resid=resid)

    rt.take_dispatch_count()
    block()
    assert rt.take_dispatch_count() == 3
    # oracle, stage by stage, fed with the device's own rounded intermediates so that each stage is checked alone
    r1 = (resid0 + y_prev).astype(np.float32)
    x_dev = xb.read(np.uint16, hidden)
    want_x = api.qwen35_rms_norm_f64(resid0, w, 1, hidden, eps, resid_add=y_prev)[0]
    np.testing.assert_allclose(synth.bf16_bits_to_f32(x_dev), want_x, rtol=8e-3, atol=1e-6)
    g = api.q4_dense_gemm(gp.view(np.uint8).reshape(-1), gs.reshape(-1), x_dev, 1, inter, hidden, group)[0].astype(np.float64)
    u = api.q4_dense_gemm(up.view(np.uint8).reshape(-1), us.reshape(-1), x_dev, 1, inter, hidden, group)[0].astype(np.float64)
    mid_dev = mid.read(np.uint16, inter)
    assert_north_star(synth.bf16_bits_to_f32(mid_dev), (g / (1.0 + np.exp(-g)) * u).astype(np.float32), "mid")
    d = api.q4_dense_gemm(dp.view(np.uint8).reshape(-1), ds.reshape(-1), mid_dev, 1, hidden, inter, group)[0]
    got = resid.read(np.float32, hidden)
    assert_north_star(got - r1, d, "down")
    # captured once, replayed twice on a fresh residual: the same bits as the eager run
    st = torch.cuda.ExternalStream(rt.stream)
    resid.write(resid0)
    rt.set_encode_only(True)
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            block()
        for _ in range(2):
            resid.write(resid0)
            with torch.cuda.stream(st):
                graph.replay()
            rt.synchronize()
            assert np.array_equal(resid.read(np.uint32, hidden), got.view(np.uint32))
    finally:
        rt.set_encode_only(False)
