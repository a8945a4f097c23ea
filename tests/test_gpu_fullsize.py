"""The benchmark configurations at full size on the GPU: a subset of query rows against the CPU oracle
(the oracle reads the same bytes, copied back from the device), plus properties that do not depend on
size: permuting a query's top-k list leaves its output unchanged, and a different split plan gives the
same result."""
import math

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_FP8, check_lse, check_out
from opfoundry_b200 import api, workloads

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(192.0)


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_lib):
    assert torch.cuda.is_available()


def test_decode_fp8_config2_full_size(oracle):
    """Batch 64, 128 heads, kv_len 32768 paged(64) fp8 cache, top-k 2048 with the last 5 % of slots -1."""
    W = workloads.decode_fp8(n_batches=1, seed=7)
    q, idx = W["steps"][0]
    B, H, topk = W["B"], W["H"], W["topk"]
    plan = api.mla_decode_plan_create(B, H, topk, 1, valid_len_hint=[W["n_valid"]] * B)
    out, lse = api.mla_decode_launch_pipeline(q, W["cache"], idx, plan, SCALE, block_table=W["block_table"], page_block_size=64)
    # without the hint the padded tail is visited and masked: same numbers
    plan2 = api.mla_decode_plan_create(B, H, topk, 1)
    out2, lse2 = api.mla_decode_launch_pipeline(q, W["cache"], idx, plan2, SCALE, block_table=W["block_table"], page_block_size=64)
    torch.cuda.synchronize()
    check_out(bits(out2), bits(out), **TOL_FP8)
    check_lse(lse2.cpu().numpy(), lse.cpu().numpy())
    # every query against the oracle (the reference's CPU function does all 64 in seconds)
    r_out, r_lse = oracle.sparse_mla(bits(q), W["cache"].cpu().numpy(), idx.cpu().numpy(), SCALE, kv_is_fp8=True,
                                     block_table=W["block_table"].cpu().numpy(), page_block_size=64)
    check_out(bits(out), r_out, **TOL_FP8)
    check_lse(lse.cpu().numpy(), r_lse)
    # permuting the valid part of every list changes the order of the sums only
    perm = torch.randperm(W["n_valid"], device="cuda")
    idx_p = idx.clone()
    idx_p[:, :W["n_valid"]] = idx[:, :W["n_valid"]][:, perm]
    out3, lse3 = api.mla_decode_launch_pipeline(q, W["cache"], idx_p, plan, SCALE, block_table=W["block_table"], page_block_size=64)
    torch.cuda.synchronize()
    check_out(bits(out3), bits(out), **TOL_FP8)
    check_lse(lse3.cpu().numpy(), lse.cpu().numpy())


def test_prefill_bf16_config3_full_size(oracle):
    """One sequence of 4096 tokens, 128 heads, causal top-k 2048."""
    W = workloads.prefill_bf16(T=4096, seed=11)
    T, H, topk = W["T"], W["H"], W["topk"]
    plan = api.mla_decode_plan_create(T, H, topk, T, valid_len_hint=W["valid_len"])
    assert plan.info.num_lists > 1
    out, lse = api.sparse_mla_prefill(W["q"], W["kv"], W["indices"], plan, SCALE)
    torch.cuda.synchronize()
    idx = W["indices"].cpu().numpy()
    for t in (0, 5, 2046, 2047, 4095):     # generator invariants at full size
        n = min(t + 1, topk)
        assert np.all(idx[t, :n] >= 0) and np.all(idx[t, :n] <= t) and np.all(idx[t, n:] == -1)
        assert len(set(idx[t, :n].tolist())) == n
    # all short rows, the tile-boundary rows, every 32nd row and the last one
    subset = np.unique(np.concatenate([np.arange(64), [65, 2046, 2047, 2048, 2049], np.arange(0, T, 32), [T - 1]])).astype(np.int32)
    r_out, r_lse = oracle.sparse_mla(bits(W["q"]), bits(W["kv"]), idx, SCALE, s_q=T, subset=subset)
    check_out(bits(out)[subset], r_out[subset], **TOL_BF16)
    check_lse(lse.cpu().numpy()[subset], r_lse[subset])
    g = (bits(out).astype(np.uint32) << 16).view(np.float32)
    assert np.all(np.isfinite(g)) and np.all(np.isfinite(lse.cpu().numpy()))


def _compact_cache(cache, block_table, seqs, page=64):
    """The pages of `seqs` copied into a small cache with a renumbered block table, so the oracle
    reads the same bytes without the whole cache crossing to the host."""
    bt = block_table[seqs].long()                                   # [n, pages_per_seq]
    n, pps = bt.shape
    rows = (bt.reshape(-1, 1) * page + torch.arange(page, device=cache.device)[None, :]).reshape(-1)
    small = cache[rows].contiguous()
    new_bt = torch.arange(n * pps, dtype=torch.int32, device=cache.device).view(n, pps)
    return small, new_bt


def test_decode_fp8_mtp_config4_full_batch(oracle):
    """Config 4 at full size (batch 128, s_q = 2, kv_len 65536, 5.5 GB paged fp8 cache): all 128 heads
    and the 16 heads one GPU of a TP-8 group owns; the two tokens of a sequence share a list for half of
    the sequences.  32 query rows (16 sequences spread over the batch) go through the oracle."""
    B = 128
    W = workloads.decode_fp8(B=B, kv_len=65536, pad_frac=0.0, n_batches=1, seed=13, s_q=2)
    q, idx = W["steps"][0]
    idx = idx.clone()
    idx[1::4] = idx[0::4]                     # sequences 0, 2, 4, ...: token 1 reuses token 0's list
    bt, cache = W["block_table"], W["cache"]
    seqs = torch.arange(0, B, 8, device="cuda")                     # 16 sequences
    qrows = (seqs[:, None] * 2 + torch.arange(2, device="cuda")[None, :]).reshape(-1)
    small, small_bt = _compact_cache(cache, bt, seqs)
    for heads in (128, 16):
        qh = q[:, :heads].contiguous()
        plan = api.mla_decode_plan_create(2 * B, heads, 2048, 2)
        out, lse = api.mla_decode_launch_pipeline(qh, cache, idx, plan, SCALE, block_table=bt, page_block_size=64)
        torch.cuda.synchronize()
        g = (bits(out).astype(np.uint32) << 16).view(np.float32)
        assert np.all(np.isfinite(g)) and np.all(np.isfinite(lse.cpu().numpy()))
        r_out, r_lse = oracle.sparse_mla(bits(qh[qrows]), small.cpu().numpy(), idx[qrows].cpu().numpy(), SCALE, kv_is_fp8=True,
                                         block_table=small_bt.cpu().numpy(), page_block_size=64, s_q=2)
        sel = qrows.cpu().numpy()
        check_out(bits(out)[sel], r_out, **TOL_FP8)
        check_lse(lse.cpu().numpy()[sel], r_lse)


def test_prefill_query_chunks_config5_path(oracle):
    """The long-prefill partition on one GPU: two adjacent query chunks of an 8192-token sequence, each
    generated and run on its own as a rank would (its own plan, the whole latent cache), must reproduce
    the unsharded run (inputs bit for bit, outputs to the last place); rows around the seam also go through the oracle."""
    from opfoundry_b200 import shard
    T, H, topk = 8192, 128, 2048
    full = workloads.prefill_bf16(T=T, seed=5)
    plan = api.mla_decode_plan_create(T, H, topk, T, valid_len_hint=full["valid_len"])
    out, lse = api.sparse_mla_prefill(full["q"], full["kv"], full["indices"], plan, SCALE)
    torch.cuda.synchronize()
    bounds = shard.shard_queries_equal_work(np.minimum(np.arange(T) + 1, topk), 2)
    assert bounds[0] == 0 and bounds[2] == T and bounds[1] > T // 2       # equal work, not equal length
    for r in range(2):
        q0, q1 = bounds[r], bounds[r + 1]
        Wc = workloads.prefill_bf16(T=T, seed=5, q_begin=q0, q_end=q1)
        assert torch.equal(Wc["q"], full["q"][q0:q1]) and torch.equal(Wc["indices"], full["indices"][q0:q1])
        pc = api.mla_decode_plan_create(q1 - q0, H, topk, q1 - q0, valid_len_hint=Wc["valid_len"])
        oc, lc = api.sparse_mla_prefill(Wc["q"], Wc["kv"], Wc["indices"], pc, SCALE)
        torch.cuda.synchronize()
        # same inputs bit for bit; the outputs may differ in the last place only: which softmax team sums
        # which tiles of a query depends on the query's position in its work list
        check_out(bits(oc), bits(out[q0:q1]), atol=2e-3, rtol=2.0 ** -6, what="chunk %d vs unsharded" % r)
        assert float((lc - lse[q0:q1]).abs().max()) <= 1e-5, "chunk %d: lse differs from the unsharded run" % r
    s = bounds[1]
    subset = np.array([s - 2, s - 1, s, s + 1, T - 1], np.int32)
    r_out, r_lse = oracle.sparse_mla(bits(full["q"]), bits(full["kv"]), full["indices"].cpu().numpy(), SCALE, s_q=T, subset=subset)
    check_out(bits(out)[subset], r_out[subset], **TOL_BF16)
    check_lse(lse.cpu().numpy()[subset], r_lse[subset])
