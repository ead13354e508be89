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

from gpu_util import rt, upload_bank  # noqa: F401
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
