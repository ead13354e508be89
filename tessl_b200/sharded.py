"""Column sharding of an MLX Q4 bank over the GPUs of one node.

Output rows are independent (every output row of `W x` reads only its own
packed row and scale/bias pairs), so a bank is cut into contiguous row slices,
one per rank; each GPU streams only its slice from its own HBM, and one
all-gather of the bf16 (or f32) outputs over NVLink rebuilds the full vector.
The activation vector (a few KiB) is replicated. The reference is a
single-device library; this module has no counterpart there.

The partition and the gather are plain `torch.distributed` code and work on any
backend (NCCL on GPUs, gloo on CPU for the tests); the local product is done by
whatever `compute` callable the caller supplies, which on a GPU is the
`tessl_b200.nn` operator on the rank's slice.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def shard_rows(rows: int, world: int, rank: int, align: int = 8) -> Tuple[int, int]:
    """Rows [begin, end) of rank `rank`: contiguous, `align`-row aligned slices
    of ceil(rows / world) rounded up to `align`; trailing ranks may get fewer
    rows or none."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    per = -(-rows // world)
    per = -(-per // align) * align
    begin = min(rows, rank * per)
    return begin, min(rows, begin + per)


def slice_rows_per_rank(rows: int, world: int, align: int = 8) -> int:
    """The padded slice height every rank contributes to the all-gather."""
    per = -(-rows // world)
    return -(-per // align) * align


@dataclass
class RowShard:
    """This rank's slice of a [rows, ...] row-major array."""
    rows: int
    world: int
    rank: int
    begin: int
    end: int

    @property
    def local_rows(self) -> int:
        return self.end - self.begin


def make_shard(rows: int, world: int, rank: int, align: int = 8) -> RowShard:
    b, e = shard_rows(rows, world, rank, align)
    return RowShard(rows, world, rank, b, e)


def slice_bank(packed: torch.Tensor, scales_biases: torch.Tensor, shard: RowShard):
    """The rank's rows of a bank given as [rows, cols/8] words and [rows, groups, 2] pairs."""
    return packed[shard.begin:shard.end].contiguous(), scales_biases[shard.begin:shard.end].contiguous()


def all_gather_rows(local: torch.Tensor, shard: RowShard, m: int = 1, group=None, align: int = 8,
                    out: "torch.Tensor | None" = None) -> torch.Tensor:
    """All-gather of per-rank outputs `local` [m, local_rows] into [m, rows].

    Fast path: with m == 1 and rows == world * local_rows the slices already sit
    in output order, so the collective writes straight into `out` (or a new
    tensor) with no staging copy.

    Every rank contributes a slice padded to the common height, the gather is
    one `all_gather_into_tensor`, and the padding is dropped afterwards. With
    m == 1 and rows divisible by world * align no copy is needed beyond the
    collective itself."""
    per = slice_rows_per_rank(shard.rows, shard.world, align)
    if m == 1 and shard.local_rows == per and per * shard.world == shard.rows:
        full = out if out is not None else local.new_empty(shard.rows)
        dist.all_gather_into_tensor(full.reshape(-1), local.reshape(-1), group=group)
        return full.reshape(1, shard.rows)
    local = local.reshape(m, shard.local_rows)
    if shard.local_rows != per:
        padded = local.new_zeros((m, per))
        padded[:, : shard.local_rows] = local
        local = padded
    gathered = local.new_empty((shard.world * m, per))  # rank-major blocks of [m, per]
    dist.all_gather_into_tensor(gathered, local.contiguous(), group=group)
    # [world, m, per] -> [m, world * per] -> first `rows` columns
    full = gathered.reshape(shard.world, m, per).permute(1, 0, 2).reshape(m, shard.world * per)[:, : shard.rows]
    if out is not None:
        out.reshape(m, shard.rows).copy_(full)
        return out.reshape(m, shard.rows)
    return full.contiguous()


def sharded_matvec(compute: Callable[[RowShard], torch.Tensor], rows: int, m: int = 1, group=None,
                   align: int = 8) -> torch.Tensor:
    """Runs `compute(shard)` (this rank's [m, local_rows] outputs) and gathers [m, rows]."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    shard = make_shard(rows, world, rank, align)
    local = compute(shard)
    if world == 1:
        return local.reshape(m, rows)
    return all_gather_rows(local, shard, m, group, align)


def partition_table(rows: int, world: int, align: int = 8) -> List[Tuple[int, int]]:
    return [shard_rows(rows, world, r, align) for r in range(world)]


class PeerGather:
    """All-gather of this rank's output slice through NVLink peer memory
    (`tessl_peer_gather`): for slices of a few KB to a few hundred KB, where a
    library all-gather is pure latency.

    Holds one gather buffer of `world * bytes_per_rank` bytes per rank in
    symmetric memory (torch's `_symmetric_memory`: peer-mapped allocations, used
    here only as the allocator and for the address exchange). The producer writes
    into `local(dtype)` (this rank's part of its own buffer); `run(rt)` encodes
    the gather on the runtime's stream; afterwards `full(dtype)` holds every
    rank's slice. Every rank must call `run` the same number of times in the
    same order."""

    def __init__(self, bytes_per_rank: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        from . import capi
        if bytes_per_rank % 16:
            raise ValueError("bytes_per_rank must be a multiple of 16")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerGather serves the GPUs of one node (at most 8)")
        self.bytes_per_rank = bytes_per_rank
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(self.world * bytes_per_rank, dtype=torch.uint8, device=dev)
        self.flags = symm_mem.empty(32, dtype=torch.int32, device=dev)
        self.buf.zero_()
        self.flags.zero_()
        torch.cuda.synchronize()
        self._hb = symm_mem.rendezvous(self.buf, group)
        self._hf = symm_mem.rendezvous(self.flags, group)
        dist.barrier(group)  # every rank's flags are zero before anyone can signal
        desc = capi.PeerGather()
        for r in range(self.world):
            desc.buffers[r] = int(self._hb.buffer_ptrs[r])
            desc.flags[r] = int(self._hf.buffer_ptrs[r])
        desc.rank, desc.world, desc.bytes_per_rank = self.rank, self.world, bytes_per_rank
        self._desc = desc

    def local(self, dtype) -> torch.Tensor:
        """This rank's slice of its own gather buffer, as a 1-D tensor of `dtype`."""
        b = self.bytes_per_rank
        return self.buf[self.rank * b:(self.rank + 1) * b].view(dtype)

    def full(self, dtype) -> torch.Tensor:
        return self.buf.view(dtype)

    def run(self, rt) -> None:
        import ctypes

        from . import capi
        capi.call("tessl_peer_gather", rt.handle, ctypes.byref(self._desc))

    def wait(self, rt) -> None:
        """`tessl_peer_wait`: the wait a deferred exchange left to its reader, as a launch of its own."""
        import ctypes

        from . import capi
        capi.call("tessl_peer_wait", rt.handle, ctypes.byref(self._desc))

    def gemv_from_gathered(self, rt, bank, y, shape, resid=None, y_as_bf16: bool = False) -> None:
        """`tessl_gemv_q4_mlx_simd_gathered`: y = W x with x the gathered vector of this descriptor; the kernel waits
        for the peers' slices itself (what a deferred exchange leaves undone)."""
        import ctypes

        from . import capi
        r = ctypes.byref(resid.c()) if resid is not None else None
        capi.call("tessl_gemv_q4_mlx_simd_gathered", rt.handle, bank.c(), ctypes.byref(self._desc), y.c(), shape.c(), r,
                  1 if y_as_bf16 else 0)

    def gemv(self, rt, bank, x_bf16, shape, y_as_bf16: bool = False, defer: bool = False) -> None:
        """`tessl_gemv_q4_mlx_simd_sharded`: this rank's slice of W x computed and exchanged by one kernel;
        afterwards `full(dtype)` holds every rank's slice."""
        import ctypes

        from . import capi
        capi.call("tessl_gemv_q4_mlx_simd_sharded_deferred" if defer else "tessl_gemv_q4_mlx_simd_sharded", rt.handle,
                  bank.c(), x_bf16.c(), ctypes.byref(self._desc), shape.c(), 1 if y_as_bf16 else 0)

    def gate_up_silu(self, rt, gate, up, x_bf16, shape, mid_as_bf16: bool = True, defer: bool = False) -> None:
        """`tessl_gemv_q4_mlx_gate_up_silu_sharded`: the fused gate/up projection on this rank's rows, exchanged
        by the same kernel."""
        import ctypes

        from . import capi
        capi.call("tessl_gemv_q4_mlx_gate_up_silu_sharded_deferred" if defer else "tessl_gemv_q4_mlx_gate_up_silu_sharded",
                  rt.handle, gate.c(), up.c(), x_bf16.c(), ctypes.byref(self._desc), shape.c(), 1 if mid_as_bf16 else 0)
