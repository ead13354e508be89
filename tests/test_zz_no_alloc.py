"""The allocation-free prefill GEMM entry (`tessl_gemm_q4_mlx_tensorops_noalloc`).

Some callers may not allocate device memory while they run: a serving loop
that rules out cudaMalloc in steady state (it can synchronise the device and
can fail when memory is tight) or code that must live inside another
framework's allocator. For them the library keeps
the GEMM's intermediate data in a fixed 8 MiB array of its own instead of a
buffer it grows on demand. This test calls that entry through the C ABI twice
in a row (the array is shared and keeps the previous call's contents) and
checks both results against the regular entry bit for bit - they run the same
kernels - and the refusal of a shape that does not fit.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import numpy as np
import pytest

from tessl_b200 import nn, synth

pytestmark = pytest.mark.gpu


@pytest.fixture()
def rt():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = nn.Runtime()
    yield r
    r.close()


def _case(rt, seed, m, n, k, group):
    packed, sb = synth.q4_bank(seed, n, k, group)
    bank = nn.Q4MlxBank(rt.buffer_from(packed), rt.buffer_from(sb))
    x = rt.buffer_from(synth.normal_bf16(seed + 5, m * k))
    return bank, x, nn.QuantShape(n, k, group)


def _free_bytes():
    import torch

    return torch.cuda.mem_get_info()[0]


def test_noalloc_entry_matches_the_regular_entry_on_two_calls_in_a_row(rt):
    # Two different shapes back to back, so the second call finds the first one's data in the array. On this
    # fresh runtime the allocation-free entry runs first, with every buffer already in place: the device's free
    # memory must not move across its calls. Only then does the regular entry (which allocates its scratch)
    # produce the bits to compare with.
    cases = [(200, 520, 4096, 64), (70, 300, 1024, 32)]
    held = []
    for seed, (m, n, k, group) in enumerate(cases):
        bank, x, shape = _case(rt, 0x7E550400 + 16 * seed, m, n, k, group)
        held.append((bank, x, shape, [rt.buffer_from(np.full(m * n + 64, -7.7e28, np.float32)) for _ in range(2)]))
    # First round: kernels load on first use (the driver may take device memory for their code).
    # Second round: nothing may move.
    for rnd in range(2):
        rt.synchronize()
        free_before = _free_bytes()
        for (m, n, k, group), (bank, x, shape, outs) in zip(cases, held):
            rt.take_dispatch_count()
            nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, x, outs[rnd], shape, m)
            assert rt.take_dispatch_count() == 2  # the pre-pass and the GEMM, nothing else
        rt.synchronize()
        if rnd == 1:
            assert _free_bytes() == free_before, "the allocation-free entry changed the device's free memory"
    for (m, n, k, group), (bank, x, shape, outs) in zip(cases, held):
        want_buf = rt.buffer_from(np.full(m * n, -7.7e28, np.float32))
        nn.gemm_q4_mlx_tensorops(rt, bank, x, want_buf, shape, m)
        want = want_buf.read(np.uint32, m * n)
        for call, got_buf in enumerate(outs):
            got = got_buf.read(np.uint32, m * n + 64)
            assert np.array_equal(got[: m * n], want), f"shape {(m, n, k, group)} call {call}: bits differ"
            assert np.all(got[m * n:].view(np.float32) == np.float32(-7.7e28)), "wrote past y"
            assert np.all(np.isfinite(got[: m * n].view(np.float32)))


def test_noalloc_entry_on_the_widest_tile(rt):
    # a shape for which the library picks the 256-wide tile (m = 600 rows of 256 columns fit the array)
    m, n, k, group = 600, 12288, 256, 64
    bank, x, shape = _case(rt, 0x7E550480, m, n, k, group)
    got_buf = rt.buffer_from(np.full(m * n, -7.7e28, np.float32))
    nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, x, got_buf, shape, m)
    assert rt.last_prefill_tile() == (256, 1)
    want_buf = rt.buffer_from(np.full(m * n, -7.7e28, np.float32))
    nn.gemm_q4_mlx_tensorops(rt, bank, x, want_buf, shape, m)
    assert np.array_equal(got_buf.read(np.uint32, m * n), want_buf.read(np.uint32, m * n))


def test_noalloc_entry_refuses_what_does_not_fit_and_keeps_the_other_refusals(rt):
    bank, x, shape = _case(rt, 0x7E550440, 8, 64, 4096, 64)
    y = rt.alloc_buffer(8 * 64 * 4)
    rt.take_dispatch_count()
    # real (never touched) buffers of the claimed sizes: capacity claims laid over the small ones could
    # overlap each other, depending on where the allocator put them, and trip the aliasing refusal first
    big = rt.alloc_buffer(2000 * 4096 * 2)
    ybig = rt.alloc_buffer(2000 * 64 * 4)
    with pytest.raises(nn.TesslError, match="built-in scratch holds 8388608"):
        nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, big, ybig, shape, 2000)
    with pytest.raises(nn.TesslError, match="group_size 256"):
        nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, x, y, nn.QuantShape(64, 4096, 256), 8)
    with pytest.raises(nn.TesslError, match="x_bf16"):
        nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, x.view(0, 64), y, shape, 8)
    nn.gemm_q4_mlx_tensorops_noalloc(rt, bank, x, y, shape, 0)  # validated no-op
    assert rt.take_dispatch_count() == 0
