"""Host-side logic of the R-sharded linear, on CPU ranks over gloo (world sizes 2 and 3).

A dense matmul stands in for the BSI dot of a shard (the CUDA kernels have no CPU fallback); what is
under test is the row partition and the all-gather reassembly, including a ragged last shard."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bsipytorch_b200.sharded import gather_columns, shard_rows


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, R, multiple, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        W = torch.randn(R, 64, generator=g)
        b = torch.randn(R, generator=g)
        x = torch.randn(10, 64, generator=g)
        lo, hi = shard_rows(R, world, rank, multiple)
        y_shard = x @ W[lo:hi].T + b[lo:hi]
        y = gather_columns(y_shard, R, world, None, multiple)
        full = x @ W.T + b
        results[rank] = bool(torch.equal(y, full)) and y.shape == (10, R)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,R,multiple", [(2, 512, 256), (2, 96, 32), (3, 100, 32), (2, 70, 1)])
def test_gather_columns_reassembles_the_full_output(world, R, multiple):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), R, multiple, results), nprocs=world, join=True)
    assert all(results[r] for r in range(world)), dict(results)


def test_shard_rows_partitions_exactly():
    for R, world, mult in [(4096, 8, 256), (16384, 8, 256), (768, 2, 32), (100, 3, 32), (50272, 8, 1), (5, 8, 1)]:
        spans = [shard_rows(R, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == R
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a <= b and c <= d
        widths = {hi - lo for lo, hi in spans if hi - lo}
        assert max(widths) == spans[0][1] - spans[0][0]
    assert shard_rows(4096, 8, 3, 256) == (1536, 2048)
