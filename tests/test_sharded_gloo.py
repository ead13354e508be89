"""The multi-GPU path's host logic on CPU: row partition, slice padding and the
all-gather that rebuilds a column-sharded output, run as two gloo ranks. Each
rank computes its slice of the GEMV with the CPU oracle (standing in for the
GPU operator, which needs a device) and the gathered vector must equal the
unsharded product bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tessl_b200 import sharded, synth


def test_partition_covers_rows_once_and_stays_aligned():
    for rows in (151936, 12288, 4096, 37, 8, 1, 100):
        for world in (1, 2, 4, 8):
            table = sharded.partition_table(rows, world)
            assert table[0][0] == 0 and table[-1][1] == rows
            for (b0, e0), (b1, e1) in zip(table, table[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 8 == 0 for b, e in table if e > b)
            per = sharded.slice_rows_per_rank(rows, world)
            assert all(e - b <= per for b, e in table) and per * world >= rows
    assert sharded.shard_rows(151936, 8, 3) == (3 * 18992, 4 * 18992)
    with pytest.raises(ValueError):
        sharded.shard_rows(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, cols, m, out_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import api
        packed, sb = synth.q4_bank(0x7E550500, rows, cols, 64)
        x = synth.normal_bf16(0x7E550501, m * cols)
        tp, tsb = torch.from_numpy(packed.view(np.int32)), torch.from_numpy(sb.view(np.int16))

        def compute(shard):
            lp, lsb = sharded.slice_bank(tp, tsb, shard)
            if shard.local_rows == 0:
                return torch.empty((m, 0), dtype=torch.float32)
            y = api.q4_dense_gemm(lp.numpy().view(np.uint8), lsb.numpy().view(np.uint16), x, m, shard.local_rows,
                                  cols, 64, threads=1)
            return torch.from_numpy(y)

        full = sharded.sharded_matvec(compute, rows, m)
        if rank == 0:
            want = api.q4_dense_gemm(packed.view(np.uint8), sb, x, m, rows, cols, 64, threads=1)
            np.save(out_path, np.stack([full.numpy(), want]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,m", [(96, 1), (100, 3), (13, 1)])
def test_two_ranks_gather_the_unsharded_result(tmp_path, rows, m):
    out = str(tmp_path / "out.npy")
    mp.spawn(_worker, args=(2, _free_port(), rows, 256, m, out), nprocs=2, join=True)
    got, want = np.load(out)
    assert got.shape == (m, rows)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
