"""`tessl_gemv_q4_mlx_simd_sharded` / `tessl_gemv_q4_mlx_gate_up_silu_sharded`: a column-sharded GEMV whose
kernel also exchanges its outputs over NVLink peer memory (no counterpart in the reference, a single-device
library).

On one GPU: a one-rank descriptor gives the plain operator's bits in one launch, the refusals, and a peer that
never arrives makes the kernel's bounded wait run out without hurting the context. With two or more GPUs two
ranks (child processes; NCCL only for the rendezvous, NVLS off) run both entries several times on changing
activations, eagerly and replayed from a CUDA graph, and every rank compares the gathered vector bit for bit
with the single-GPU operator on the unsharded bank.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from gpu_util import rt, seeded_f32, upload_bank  # noqa: F401
from tessl_b200 import capi, nn, synth

pytestmark = pytest.mark.gpu


def _desc(world, rank, nbytes, bufs, flags):
    d = capi.PeerGather()
    for r in range(8):
        d.buffers[r] = bufs[r] if r < len(bufs) else None
        d.flags[r] = flags[r] if r < len(flags) else None
    d.rank, d.world, d.bytes_per_rank = rank, world, nbytes
    return d


@pytest.mark.parametrize("rows,cols,group", [(1000, 4096, 64), (264, 2048, 32), (520, 1024, 128), (96, 1536, 64)])
def test_one_rank_is_the_plain_operator_in_one_launch(rt, rows, cols, group):
    packed, sb = synth.q4_bank(0x5A4D + rows, rows, cols, group)
    packed2, sb2 = synth.q4_bank(0x5A4E + rows, rows, cols, group)
    x = rt.buffer_from(synth.normal_bf16(rows + cols, cols))
    bank, bank2 = upload_bank(rt, packed, sb), upload_bank(rt, packed2, sb2)
    shape = nn.QuantShape(rows, cols, group)
    nbytes = -(-rows * 4 // 16) * 16
    out = rt.buffer_from(np.full(nbytes // 4 + 4, -7.0, np.float32))
    flags = rt.buffer_from(np.zeros(32, np.uint32))
    d = _desc(1, 0, nbytes, [out.ptr], [flags.ptr])
    want = rt.alloc_buffer(rows * 4)
    for bf16 in (False, True):
        elem, dt = (2, np.uint16) if bf16 else (4, np.uint32)
        rt.take_dispatch_count()
        capi.call("tessl_gemv_q4_mlx_simd_sharded", rt.handle, bank.c(), x.c(), ctypes.byref(d), shape.c(), int(bf16))
        assert rt.take_dispatch_count() == 1
        nn.gemv_q4_mlx_simd(rt, bank, x, want, shape, y_as_bf16=bf16)
        assert np.array_equal(out.read(dt, rows), want.read(dt, rows))
        capi.call("tessl_gemv_q4_mlx_gate_up_silu_sharded", rt.handle, bank.c(), bank2.c(), x.c(), ctypes.byref(d), shape.c(),
                  int(bf16))
        nn.gemv_q4_mlx_gate_up_silu(rt, bank, bank2, x, want, shape, bf16)
        assert np.array_equal(out.read(dt, rows), want.read(dt, rows))
        assert rows * elem <= nbytes
    assert np.all(out.read(np.float32, 4, byte_offset=nbytes) == -7.0), "wrote past the gather slot"
    assert np.all(flags.read(np.uint32, 32) == 0), "a one-rank launch has no exchange"


def test_refusals_before_any_launch(rt):
    rows, cols = 64, 1024
    packed, sb = synth.q4_bank(3, rows, cols, 64)
    bank = upload_bank(rt, packed, sb)
    x = rt.buffer_from(synth.normal_bf16(4, cols))
    out = rt.alloc_buffer(4096)
    flags = rt.buffer_from(np.zeros(32, np.uint32))
    shape = nn.QuantShape(rows, cols, 64)
    rt.take_dispatch_count()
    cases = [
        (_desc(1, 0, 128, [out.ptr], [flags.ptr]), shape, "the slice needs 256 bytes, the gather holds 128"),
        (_desc(0, 0, 256, [out.ptr], [flags.ptr]), shape, "outside 1..8"),
        (_desc(2, 0, 256, [out.ptr, None], [flags.ptr] * 2), shape, "null buffer or flag"),
        (_desc(1, 0, 256, [out.ptr], [flags.ptr]), nn.QuantShape(0, cols, 64), "no rows takes part through tessl_peer_gather"),
        (_desc(1, 0, 256, [out.ptr], [flags.ptr]), nn.QuantShape(rows, cols, 48), "group_size"),
    ]
    for d, shp, text in cases:
        for name, args in (("tessl_gemv_q4_mlx_simd_sharded", (bank.c(), x.c())),
                           ("tessl_gemv_q4_mlx_gate_up_silu_sharded", (bank.c(), bank.c(), x.c()))):
            with pytest.raises(capi.TesslError, match=text):
                capi.call(name, rt.handle, *args, ctypes.byref(d), shp.c(), 0)
    with pytest.raises(capi.TesslError, match="null descriptor"):
        capi.call("tessl_gemv_q4_mlx_simd_sharded", rt.handle, bank.c(), x.c(), None, shape.c(), 0)
    assert rt.take_dispatch_count() == 0


@pytest.mark.parametrize("cols", [4096, 1536])  # the exchange inside the GEMV kernel, and the GEMV + stand-alone gather
def test_a_peer_that_never_arrives_makes_the_bounded_wait_run_out(cols):
    """Rank 0 of a two-rank launch whose "peer" is a pair of local buffers nobody signals: with the wait limit at
    about a millisecond the kernel gives up, leaves a status word and returns; the call reports it, the runtime is
    poisoned, and a fresh runtime on the same GPU works. Nothing faults or hangs."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    rows = 2048
    r = nn.Runtime()
    try:
        packed, sb = synth.q4_bank(11, rows, cols, 64)
        bank = upload_bank(r, packed, sb)
        x = r.buffer_from(synth.normal_bf16(12, cols))
        bufs = [r.alloc_buffer(2 * rows * 4) for _ in range(2)]
        flags = [r.buffer_from(np.zeros(32, np.uint32)) for _ in range(2)]
        r.set_peer_wait_limit(2_000_000)
        d = _desc(2, 0, rows * 4, [b.ptr for b in bufs], [f.ptr for f in flags])
        with pytest.raises(capi.TesslError) as e:
            capi.call("tessl_gemv_q4_mlx_simd_sharded", r.handle, bank.c(), x.c(), ctypes.byref(d), nn.QuantShape(rows, cols, 64).c(), 0)
        assert e.value.status == capi.TESSL_ERR
        assert "gave up a bounded wait" in str(e.value) and "role 80" in str(e.value), str(e.value)
        assert r.is_poisoned()
    finally:
        r.close()
    with nn.Runtime() as fresh:
        b = fresh.buffer_from(np.arange(64, dtype=np.uint32))
        assert np.array_equal(b.read(np.uint32, 64), np.arange(64, dtype=np.uint32))


@pytest.mark.parametrize("cols", [4096, 1536])  # the wait inside the GEMV kernel, and as a launch of its own
def test_a_reader_of_a_gathered_vector_whose_peer_never_finishes_gives_up(cols):
    """The reader's side of a deferred exchange: this rank's call counter says one exchange was launched, the
    "peer" never reports completion. The bounded wait runs out, the call reports it, the runtime is poisoned and
    nothing was computed from the incomplete vector; a fresh runtime works."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    rows = 256
    r = nn.Runtime()
    try:
        packed, sb = synth.q4_bank(21, rows, cols, 64)
        bank = upload_bank(r, packed, sb)
        bufs = [r.buffer_from(np.zeros(cols, np.uint16)) for _ in range(2)]  # world * bytes_per_rank = cols * 2 bytes
        f0 = np.zeros(32, np.uint32)
        f0[16] = 1  # one exchange launched by this rank; flag 8 + 1 (the peer's completion) stays 0
        flags = [r.buffer_from(f0), r.buffer_from(np.zeros(32, np.uint32))]
        y = seeded_f32(r, rows)
        r.set_peer_wait_limit(2_000_000)
        d = _desc(2, 0, cols, [b.ptr for b in bufs], [f.ptr for f in flags])
        with pytest.raises(capi.TesslError) as e:
            capi.call("tessl_gemv_q4_mlx_simd_gathered", r.handle, bank.c(), ctypes.byref(d), y.c(),
                      nn.QuantShape(rows, cols, 64).c(), None, 0)
        assert "gave up a bounded wait" in str(e.value) and "role 80" in str(e.value), str(e.value)
        assert r.is_poisoned()
    finally:
        r.close()
    with nn.Runtime() as fresh:
        b = fresh.buffer_from(np.arange(64, dtype=np.uint32))
        assert np.array_equal(b.read(np.uint32, 64), np.arange(64, dtype=np.uint32))


def test_a_gathered_reader_on_one_rank_is_the_plain_operator(rt):
    rows, cols = 264, 4096
    packed, sb = synth.q4_bank(31, rows, cols, 64)
    bank = upload_bank(rt, packed, sb)
    xv = synth.normal_bf16(32, cols)
    buf = rt.buffer_from(xv)
    flags = rt.buffer_from(np.zeros(32, np.uint32))
    d = _desc(1, 0, cols * 2, [buf.ptr], [flags.ptr])
    a, b = seeded_f32(rt, rows), seeded_f32(rt, rows)
    capi.call("tessl_gemv_q4_mlx_simd_gathered", rt.handle, bank.c(), ctypes.byref(d), a.c(), nn.QuantShape(rows, cols, 64).c(), None, 0)
    nn.gemv_q4_mlx_simd(rt, bank, buf, b, nn.QuantShape(rows, cols, 64))
    assert np.array_equal(a.read(np.uint32, rows), b.read(np.uint32, rows))
    capi.call("tessl_peer_wait", rt.handle, ctypes.byref(d))  # one rank: nothing to wait for, nothing launched
    with pytest.raises(capi.TesslError, match="gathered x"):
        capi.call("tessl_gemv_q4_mlx_simd_gathered", rt.handle, bank.c(), ctypes.byref(_desc(1, 0, 64, [buf.ptr], [flags.ptr])),
                  a.c(), nn.QuantShape(rows, cols, 64).c(), None, 0)


_CHILD = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["TESSL_REPO"])
from tessl_b200 import nn, sharded, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rt = nn.Runtime(rank)
st = torch.cuda.ExternalStream(rt.stream, device=rank)
B = nn.GpuBuffer.from_torch

def dev_bank(seed, rows, cols, group):
    p, sb = synth.q4_bank(seed, rows, cols, group)
    return torch.from_numpy(p.view(np.int32)).cuda(), torch.from_numpy(sb.view(np.int16)).cuda()

def as_bank(p, sb):
    return nn.Q4MlxBank(B(p), B(sb))

def xs(seed, cols):
    return torch.from_numpy(synth.normal_bf16(seed, cols).view(np.int16)).cuda()

# (rows, cols, group, bf16 out): the tensor-core kernel with several stages per block, a ragged slice,
# and a width that kernel does not take (the GEMV + stand-alone exchange path)
# and rows of 8192 / 12288 columns (windowed stages; 14-row blocks whose slots are only 4-byte aligned in bf16)
for rows, cols, group, bf16 in ((12288, 4096, 64, True), (4104, 2048, 32, False), (1000, 1536, 64, False),
                                (1000, 12288, 64, True), (4096, 12288, 64, False), (520, 8192, 128, True)):
    elem, tdt = (2, torch.int16) if bf16 else (4, torch.int32)
    gp, gsb = dev_bank(100 + rows, rows, cols, group)
    up, usb = dev_bank(200 + rows, rows, cols, group)
    sh = sharded.make_shard(rows, world, rank)
    per = sharded.slice_rows_per_rank(rows, world)
    pg = sharded.PeerGather(-(-per * elem // 16) * 16)
    lg, lu = sharded.slice_bank(gp, gsb, sh), sharded.slice_bank(up, usb, sh)
    keep = [gp, gsb, up, usb, lg, lu]
    full_g, full_u, loc_g, loc_u = as_bank(gp, gsb), as_bank(up, usb), as_bank(*lg), as_bank(*lu)
    want = torch.empty(rows, dtype=tdt, device="cuda")
    shape_l, shape_f = nn.QuantShape(sh.local_rows, cols, group), nn.QuantShape(rows, cols, group)
    slot = pg.bytes_per_rank // elem

    def gathered():
        g = pg.full(tdt).view(world, slot)
        return torch.cat([g[r, : sharded.make_shard(rows, world, r).local_rows] for r in range(world)])

    for call in range(6):
        x = xs(7 * call + rows, cols)
        if call % 2 == 0:
            pg.gemv(rt, loc_g, B(x), shape_l, y_as_bf16=bf16)
            nn.gemv_q4_mlx_simd(rt, full_g, B(x), B(want), shape_f, y_as_bf16=bf16)
        else:
            pg.gate_up_silu(rt, loc_g, loc_u, B(x), shape_l, mid_as_bf16=bf16)
            nn.gemv_q4_mlx_gate_up_silu(rt, full_g, full_u, B(x), B(want), shape_f, bf16)
        assert torch.equal(gathered(), want), (rank, rows, call)
        if call == 3:
            with torch.cuda.stream(st):
                pg.local(tdt).zero_()
            pg.run(rt)  # the stand-alone exchange on the same descriptor, between fused calls
            assert int(gathered().abs().max().item()) == 0
        dist.barrier()  # nobody starts the next call before everyone has compared

    # deferred exchange: the producing kernel does not wait for the peers, the kernel that reads the gathered vector
    # does (in the kernel for widths the tensor-core GEMV takes, as a launch of its own otherwise); a down-like
    # projection over the gathered vector against the single-GPU chain, bit for bit
    if bf16 and rows % (8 * world) == 0:
        dp, dsb = dev_bank(300 + rows, 512, rows, 64) if rows in (1024, 2048, 4096, 8192, 12288) else (None, None)
        if dp is not None:
            down = as_bank(dp, dsb)
            keep += [dp, dsb]
            y_got = torch.empty(512, device="cuda")
            y_want = torch.empty(512, device="cuda")
            mid_ref = torch.empty(rows, dtype=torch.int16, device="cuda")
            sdn = nn.QuantShape(512, rows, 64)
            for call in range(6):
                x = xs(900 + call + rows, cols)
                pg.gate_up_silu(rt, loc_g, loc_u, B(x), shape_l, mid_as_bf16=True, defer=True)
                if call % 2 == 0:
                    pg.gemv_from_gathered(rt, down, B(y_got), sdn)
                else:
                    pg.wait(rt)
                    nn.gemv_q4_mlx_simd(rt, down, nn.GpuBuffer(pg.full(torch.int16).data_ptr(), rows * 2), B(y_got), sdn)
                nn.gemv_q4_mlx_gate_up_silu(rt, full_g, full_u, B(x), B(mid_ref), shape_f, True)
                nn.gemv_q4_mlx_simd(rt, down, B(mid_ref), B(y_want), sdn)
                assert torch.equal(gathered(), mid_ref), (rank, rows, "deferred mid", call)
                assert torch.equal(y_got.view(torch.int32), y_want.view(torch.int32)), (rank, rows, "deferred down", call)
                dist.barrier()
            # and replayed from a graph: exchange + reader, three times per replay
            xg2 = xs(7000, cols)
            rt.set_encode_only(True)
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=st):
                for i in range(3):
                    pg.gate_up_silu(rt, loc_g, loc_u, B(xg2), shape_l, mid_as_bf16=True, defer=True)
                    pg.gemv_from_gathered(rt, down, B(y_got), sdn)
            for rep in range(3):
                with torch.cuda.stream(st):
                    xg2.copy_(xs(7100 + rep, cols))
                    g2.replay()
                rt.synchronize()
                rt.set_encode_only(False)
                nn.gemv_q4_mlx_gate_up_silu(rt, full_g, full_u, B(xg2), B(mid_ref), shape_f, True)
                nn.gemv_q4_mlx_simd(rt, down, B(mid_ref), B(y_want), sdn)
                assert torch.equal(y_got.view(torch.int32), y_want.view(torch.int32)), (rank, rows, "deferred graph", rep)
                rt.set_encode_only(True)
                dist.barrier()
            rt.set_encode_only(False)

    # replayed from a CUDA graph: four calls per replay, the activations rewritten between replays
    xg = xs(999, cols)
    rt.set_encode_only(True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=st):
        for i in range(4):
            if i % 2 == 0:
                pg.gemv(rt, loc_g, B(xg), shape_l, y_as_bf16=bf16)
            else:
                pg.gate_up_silu(rt, loc_g, loc_u, B(xg), shape_l, mid_as_bf16=bf16)
    for rep in range(3):
        with torch.cuda.stream(st):
            xg.copy_(xs(5000 + rep, cols))
            graph.replay()
        rt.synchronize()
        rt.set_encode_only(False)
        nn.gemv_q4_mlx_gate_up_silu(rt, full_g, full_u, B(xg), B(want), shape_f, bf16)
        assert torch.equal(gathered(), want), (rank, rows, "graph", rep)
        rt.set_encode_only(True)
        dist.barrier()
    rt.set_encode_only(False)
assert not rt.is_poisoned()
dist.barrier()
dist.destroy_process_group()
print("sharded gemv ok", rank)
"""


def test_two_ranks_compute_and_exchange_in_one_kernel():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TESSL_REPO=repo, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541", WORLD_SIZE="2",
               NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    procs = [subprocess.Popen([sys.executable, "-c", _CHILD], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out))
    for code, out in outs:
        assert code == 0 and "sharded gemv ok" in out, out[-2000:]
