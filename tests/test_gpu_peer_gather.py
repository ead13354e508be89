"""`tessl_peer_gather`: the NVLink peer-memory all-gather behind the column-sharded
GEMVs (no counterpart in the reference, a single-device library).

On one GPU only the argument checks, the world == 1 no-op and a wait that runs out can
run; with two or more GPUs two ranks (child processes, NCCL only for the rendezvous, NVLS
off) gather changing patterns several times - a one-block slice, then 512 KiB slices
copied by sixteen blocks, eagerly and replayed from a CUDA graph - and compare every byte.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from gpu_util import rt  # noqa: F401
from tessl_b200 import capi, nn

pytestmark = pytest.mark.gpu


def _desc(world, rank, nbytes, bufs, flags):
    d = capi.PeerGather()
    for r in range(8):
        d.buffers[r] = bufs[r] if r < len(bufs) else None
        d.flags[r] = flags[r] if r < len(flags) else None
    d.rank, d.world, d.bytes_per_rank = rank, world, nbytes
    return d


def test_refusals_and_single_rank_noop(rt):
    buf = rt.alloc_buffer(4096)
    flg = rt.alloc_buffer(128)
    rt.take_dispatch_count()
    bad = [
        (_desc(0, 0, 64, [buf.ptr], [flg.ptr]), "outside 1..8"),
        (_desc(9, 0, 64, [buf.ptr] * 8, [flg.ptr] * 8), "outside 1..8"),
        (_desc(2, 2, 64, [buf.ptr] * 2, [flg.ptr] * 2), "outside world"),
        (_desc(2, 0, 24, [buf.ptr] * 2, [flg.ptr] * 2), "multiple of 16"),
        (_desc(2, 0, 64, [buf.ptr, None], [flg.ptr] * 2), "null buffer or flag"),
        (_desc(2, 0, 64, [buf.ptr, buf.ptr + 4], [flg.ptr] * 2), "16-byte aligned"),
    ]
    for d, text in bad:
        with pytest.raises(capi.TesslError, match=text):
            capi.call("tessl_peer_gather", rt.handle, ctypes.byref(d))
    with pytest.raises(capi.TesslError, match="null descriptor"):
        capi.call("tessl_peer_gather", rt.handle, None)
    # one rank: nothing to exchange, nothing launched
    capi.call("tessl_peer_gather", rt.handle, ctypes.byref(_desc(1, 0, 64, [buf.ptr], [flg.ptr])))
    assert rt.take_dispatch_count() == 0


def test_a_peer_that_never_arrives_poisons_the_runtime_and_nothing_else():
    """A bounded device-side wait runs out: rank 0 of a two-rank exchange whose "peer" is a pair of local
    buffers nobody signals. With the wait limit set to about a millisecond the kernel gives up, writes its
    status word and returns; the call reports it, the runtime is poisoned and refuses further work, and a
    fresh runtime on the same GPU works (the context is intact: nothing faulted or hung). The reference
    reports a shared-event timeout the same way (src/runtime.rs:1498-1531, src/capi.rs:212-247)."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = nn.Runtime()
    try:
        bufs = [r.alloc_buffer(2 * 4096) for _ in range(2)]
        flags = [r.buffer_from(np.zeros(32, np.uint32)) for _ in range(2)]
        r.set_peer_wait_limit(2_000_000)  # clocks: ~1 ms
        d = _desc(2, 0, 4096, [b.ptr for b in bufs], [f.ptr for f in flags])
        with pytest.raises(capi.TesslError) as e:
            capi.call("tessl_peer_gather", r.handle, ctypes.byref(d))
        assert e.value.status == capi.TESSL_ERR
        assert "gave up a bounded wait" in str(e.value) and "role 80" in str(e.value), str(e.value)  # 0x50
        assert r.is_poisoned()
        with pytest.raises(capi.TesslError, match="poisoned"):
            r.alloc_buffer(16)
    finally:
        r.close()
    with nn.Runtime() as fresh:
        b = fresh.buffer_from(np.arange(64, dtype=np.uint32))
        assert np.array_equal(b.read(np.uint32, 64), np.arange(64, dtype=np.uint32))
        assert not fresh.is_poisoned()


_CHILD = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["TESSL_REPO"])
from tessl_b200 import nn, sharded
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rt = nn.Runtime(rank)
n = 6144  # bf16 elements per rank
pg = sharded.PeerGather(n * 2)
st = torch.cuda.ExternalStream(rt.stream, device=rank)
for call in range(5):
    with torch.cuda.stream(st):
        pg.local(torch.int16).copy_(torch.arange(n, device="cuda", dtype=torch.int32).add_(1000 * rank + 7 * call).to(torch.int16))
    pg.run(rt)   # synchronous: returns when this rank's buffer holds every slice
    got = pg.full(torch.int16).cpu().numpy().reshape(world, n)
    for r in range(world):
        want = (np.arange(n, dtype=np.int32) + 1000 * r + 7 * call).astype(np.int16)
        assert np.array_equal(got[r], want), (rank, call, r)
    dist.barrier()   # nobody starts overwriting its slice before everyone has checked
# slices large enough for several thread blocks (the ticket counter, the last block's completion
# handshake, the counters' reset), eagerly and replayed from a CUDA graph
big = 512 * 1024 // 2  # bf16 elements per rank: 512 KiB, 16 blocks
pgb = sharded.PeerGather(big * 2)
def fill(call):
    pgb.local(torch.int16).copy_(torch.arange(big, device="cuda", dtype=torch.int32).mul_(3).add_(1000 * rank + 7 * call).to(torch.int16))
def check(call, what):
    got = pgb.full(torch.int16).cpu().numpy().reshape(world, big)
    for r in range(world):
        want = (np.arange(big, dtype=np.int64) * 3 + 1000 * r + 7 * call).astype(np.int16)
        assert np.array_equal(got[r], want), (rank, what, call, r)
for call in range(4):
    with torch.cuda.stream(st):
        fill(call)
    pgb.run(rt)
    check(call, "eager")
    dist.barrier()
rt.set_encode_only(True)
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph, stream=st):
    for i in range(3):
        pgb.run(rt)
for rep in range(3):
    with torch.cuda.stream(st):
        fill(100 + rep)
        graph.replay()
    rt.synchronize()
    check(100 + rep, "graph")
    dist.barrier()
rt.set_encode_only(False)
assert not rt.is_poisoned()
dist.destroy_process_group()
print("peer gather ok", rank)
"""


def test_two_ranks_gather_changing_patterns():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TESSL_REPO=repo, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE="2",
               NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    procs = [subprocess.Popen([sys.executable, "-c", _CHILD], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out))
    for code, out in outs:
        assert code == 0 and "peer gather ok" in out, out[-2000:]
