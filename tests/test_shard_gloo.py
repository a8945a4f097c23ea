"""Partitioning and cross-rank reduction logic, run as two CPU ranks over gloo."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from opfoundry_b200 import shard


def test_shard_batch_and_heads():
    for n, w in [(64, 8), (65, 8), (3, 4), (128, 2)]:
        got = [shard.shard_batch(n, w, r) for r in range(w)]
        assert got[0][0] == 0 and got[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        sizes = [b - a for a, b in got]
        assert max(sizes) - min(sizes) <= 1
    assert [shard.shard_heads(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 128)]


def test_equal_work_query_chunks():
    T, topk = 131072, 2048
    valid = np.minimum(np.arange(T) + 1, topk)
    b = shard.shard_queries_equal_work(valid, 8)
    assert b[0] == 0 and b[-1] == T and all(x <= y for x, y in zip(b, b[1:]))
    work = [int(valid[b[i]:b[i + 1]].sum()) for i in range(8)]
    assert max(work) - min(work) <= topk            # equal within one query's worth
    assert b[1] - b[0] > b[2] - b[1]                # the first chunk holds the cheap early queries


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # time aggregation: every rank reports its own duration, all get the maximum
        mx = shard.max_over_ranks([10.0 + rank, 5.0 - rank], "cpu")
        # head-sharded outputs gathered back into [rows, H, D]
        H, D, rows = 8, 4, 3
        full = torch.arange(rows * H * D, dtype=torch.float32).view(rows, H, D)
        h0, h1 = shard.shard_heads(H, world, rank)
        gathered = shard.all_gather_heads(full[:, h0:h1].clone(), world)
        ret[rank] = (mx, bool(torch.equal(gathered, full)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret[0][0] == [11.0, 5.0] and ret[1][0] == [11.0, 5.0]
    assert ret[0][1] and ret[1][1]
