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
    subset = np.array([0, 1, 31, 63], np.int32)
    r_out, r_lse = oracle.sparse_mla(bits(q), W["cache"].cpu().numpy(), idx.cpu().numpy(), SCALE, kv_is_fp8=True,
                                     block_table=W["block_table"].cpu().numpy(), page_block_size=64, subset=subset)
    check_out(bits(out)[subset], r_out[subset], **TOL_FP8)
    check_lse(lse.cpu().numpy()[subset], r_lse[subset])
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
    subset = np.array([0, 1, 30, 31, 32, 33, 63, 64, 65, 1000, 2046, 2047, 2048, 2049, 4095], np.int32)
    r_out, r_lse = oracle.sparse_mla(bits(W["q"]), bits(W["kv"]), idx, SCALE, s_q=T, subset=subset)
    check_out(bits(out)[subset], r_out[subset], **TOL_BF16)
    check_lse(lse.cpu().numpy()[subset], r_lse[subset])
    g = (bits(out).astype(np.uint32) << 16).view(np.float32)
    assert np.all(np.isfinite(g)) and np.all(np.isfinite(lse.cpu().numpy()))


def test_decode_fp8_mtp_config4_shape_reduced_batch(oracle):
    """Config 4's shape per sequence (s_q = 2, kv_len 65536, paged fp8 cache) at batch 16, with all 128
    heads and with the 16 heads one GPU of a TP-8 group owns; the two tokens of a sequence share a list
    for half of the sequences."""
    W = workloads.decode_fp8(B=16, kv_len=65536, pad_frac=0.0, n_batches=1, seed=13, s_q=2)
    q, idx = W["steps"][0]
    idx = idx.clone()
    idx[1::4] = idx[0::4]                     # sequences 0, 2, 4, ...: token 1 reuses token 0's list
    bt, cache = W["block_table"], W["cache"]
    for heads in (128, 16):
        qh = q[:, :heads].contiguous()
        plan = api.mla_decode_plan_create(32, heads, 2048, 2)
        out, lse = api.mla_decode_launch_pipeline(qh, cache, idx, plan, SCALE, block_table=bt, page_block_size=64)
        torch.cuda.synchronize()
        subset = np.array([0, 1, 2, 3, 31], np.int32)
        r_out, r_lse = oracle.sparse_mla(bits(qh), cache.cpu().numpy(), idx.cpu().numpy(), SCALE, kv_is_fp8=True,
                                         block_table=bt.cpu().numpy(), page_block_size=64, s_q=2, subset=subset)
        check_out(bits(out)[subset], r_out[subset], **TOL_FP8)
        check_lse(lse.cpu().numpy()[subset], r_lse[subset])
