"""Partitioning and cross-rank reduction logic, run as two CPU ranks over gloo: index arithmetic, the
maximum over ranks, the gather layout, and - with the CPU oracle standing in for the kernels - that head,
sequence and query-chunk shards computed on separate ranks reassemble to the single-rank result."""
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
        # the three partitions of the path on a tiny problem: every rank runs the oracle on its shard only,
        # the shards are exchanged, and the reassembled result must equal the oracle's on the whole problem
        from oracle import build as obuild
        obuild.build_oracle()
        from oracle import oracle as O
        from opfoundry_b200 import synth
        scale = 0.07
        case = synth.make_decode_case(4, 8, 64, 16, s_q=2, seed=5)          # 8 query rows, 8 heads, bf16 cache
        run = lambda q, idx, s_q=2: O.sparse_mla(q, case["kv"], idx, scale, s_q=s_q, kv_batch_stride_rows=case["kv_batch_stride_rows"],
                                                 num_threads=1)
        want_out, want_lse = run(case["q"], case["indices"])

        def gather_np(a, dim):
            t = torch.from_numpy(np.ascontiguousarray(a).astype(np.float32))
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            return torch.cat(parts, dim=dim).numpy()

        # heads: rank r computes heads [h0, h1) of every row
        h0, h1 = shard.shard_heads(8, world, rank)
        o, l = run(np.ascontiguousarray(case["q"][:, h0:h1]), case["indices"])
        ok_heads = np.array_equal(gather_np(o, 1), want_out.astype(np.float32)) and np.array_equal(gather_np(l, 1), want_lse)
        # sequences: rank r computes its sequences (both query rows of each)
        b0, b1 = shard.shard_batch(4, world, rank)
        sel = np.zeros((8, 16), np.int32) - 1
        sel[2 * b0:2 * b1] = case["indices"][2 * b0:2 * b1]                 # rows of other ranks: empty lists, ignored below
        o, l = run(case["q"], sel)
        ok_batch = np.array_equal(gather_np(o[2 * b0:2 * b1], 0), want_out.astype(np.float32)) and \
            np.array_equal(gather_np(l[2 * b0:2 * b1], 0), want_lse)
        # query chunks of a causal prefill: contiguous ranges of equal work
        pre = synth.make_prefill_case(24, 8, 8, seed=3)
        p_out, p_lse = O.sparse_mla(pre["q"], pre["kv"], pre["indices"], scale, s_q=24, num_threads=1)
        bounds = shard.shard_queries_equal_work(pre["valid_len"], world)
        sub = np.arange(bounds[rank], bounds[rank + 1], dtype=np.int32)
        c_out, c_lse = O.sparse_mla(pre["q"], pre["kv"], pre["indices"], scale, s_q=24, subset=sub, num_threads=1)
        mine = torch.zeros(24, 8, 512)
        mine[sub] = torch.from_numpy(c_out[sub].astype(np.float32))
        dist.all_reduce(mine)                                               # disjoint rows: the sum is the concatenation
        ok_chunks = np.array_equal(mine.numpy(), p_out.astype(np.float32)) and sum(bounds[i + 1] - bounds[i] for i in range(world)) == 24
        ret[rank] = (mx, bool(torch.equal(gathered, full)), bool(ok_heads), bool(ok_batch), bool(ok_chunks))
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
    for r in range(world):
        assert ret[r][2], "head shards do not reassemble to the oracle's result"
        assert ret[r][3], "sequence shards do not reassemble to the oracle's result"
        assert ret[r][4], "query chunks do not reassemble to the oracle's result"
