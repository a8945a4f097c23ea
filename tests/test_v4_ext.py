"""Attention sink and second KV pool (the two features of the reference's v4 prefill kernels,
opus_attn/dsa_v4/common/mla_v4_host.cc:455-532): the oracle's restatement against the formula of
dsa_v4/README.md "Attention Model" written out in numpy (CPU), and the CUDA path against the oracle (GPU)."""
import math

import numpy as np
import pytest

from opfoundry_b200 import synth

SCALE = 1.0 / math.sqrt(192.0)


def _f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _make(T=40, H=8, topk=24, rows2=16, seed=9):
    """A small causal prefill whose last slots point into a second pool of `rows2` bf16 rows."""
    case = synth.make_prefill_case(T, H, topk, seed=seed)
    rng = np.random.default_rng(seed)
    kv2 = synth.normal_bf16(seed, "kv2", (rows2, 576))
    idx = case["indices"].copy()
    split = np.zeros(T, np.int32)
    for t in range(T):
        n1 = int(min(t + 1, topk - 6))                      # prefix slots: positions of the cache
        n2 = int(rng.integers(0, 7))                        # extend slots: physical rows of the second pool
        row = np.full(topk, -1, np.int32)
        row[:n1] = idx[t, :n1]
        row[n1:n1 + n2] = rng.choice(rows2, size=n2, replace=False)
        idx[t] = row
        split[t] = n1
    sink = rng.normal(size=H).astype(np.float32) * 2.0
    return case, idx, split, kv2, sink


def _numpy_reference(case, idx, split, kv2, sink, scale):
    q, kv = _f32(case["q"]).astype(np.float64), _f32(case["kv"]).astype(np.float64)
    k2 = _f32(kv2).astype(np.float64)
    T, H = q.shape[0], q.shape[1]
    out = np.zeros((T, H, 512)); lse = np.zeros((T, H))
    for t in range(T):
        rows = [kv[i] if j < split[t] else k2[i] for j, i in enumerate(idx[t]) if i >= 0]
        for h in range(H):
            if not rows:
                lse[t, h] = sink[h]
                continue
            K = np.stack(rows)
            s = K @ q[t, h] * scale
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            den = e.sum() + math.exp(sink[h] - m)
            out[t, h] = (e / den) @ K[:, :512]
            lse[t, h] = math.log(den) + m
    return out, lse


def test_oracle_sink_and_second_pool_follow_the_v4_formula(oracle):
    case, idx, split, kv2, sink = _make()
    o, l = oracle.sparse_mla_v4(case["q"], case["kv"], idx, SCALE, attn_sink=sink, kv2=kv2, pool_split=split, s_q=idx.shape[0])
    ro, rl = _numpy_reference(case, idx, split, kv2, sink, SCALE)
    assert np.abs(_f32(o) - ro).max() < 2e-2 and np.abs(l - rl).max() < 1e-4
    # without the extensions the function is the plain oracle, bit for bit
    a = oracle.sparse_mla_v4(case["q"], case["kv"], case["indices"], SCALE, s_q=idx.shape[0])
    b = oracle.sparse_mla(case["q"], case["kv"], case["indices"], SCALE, s_q=idx.shape[0])
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.gpu
@pytest.mark.parametrize("what", ["sink", "pool", "both", "sink_fp8_split"])
def test_gpu_sink_and_second_pool(built_lib, oracle, what):
    import torch
    from helpers import TOL_BF16, TOL_FP8, check_lse, check_out
    from opfoundry_b200 import api
    dev = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a.view(np.int16)).cuda().view(dt)
    if what == "sink_fp8_split":
        # decode on an fp8 cache with split work items: the sink must be counted once per row, in the first piece
        case = synth.make_decode_case(3, 128, 2048, 1024, fp8=True, paged=True, pad_frac=0.1, seed=21)
        sink = (np.random.default_rng(3).normal(size=128) * 3.0).astype(np.float32)
        sink[:4] = [-40.0, 40.0, 0.0, 9.0]
        plan = api.mla_decode_plan_create(3, 128, 1024, 1)
        assert plan.info.num_partials > 0
        out, lse = api.mla_v4_launch_pipeline(dev(case["q"], torch.bfloat16), dev(case["kv"]), dev(case["indices"]), plan, SCALE,
                                              attn_sink=dev(sink), block_table=dev(case["block_table"]), page_block_size=64)
        r_out, r_lse = oracle.sparse_mla_v4(case["q"], case["kv"], case["indices"], SCALE, attn_sink=sink, kv_is_fp8=True,
                                            block_table=case["block_table"], page_block_size=64)
        tol = TOL_FP8
    else:
        case, idx, split, kv2, sink = _make(T=300, H=128, topk=256, rows2=64, seed=5)
        idx[7] = -1                                            # a row without any position
        use_sink, use_pool = what in ("sink", "both"), what in ("pool", "both")
        if not use_pool:
            idx, split = case["indices"].copy(), None
            idx[7] = -1
        T = idx.shape[0]
        plan = api.mla_decode_plan_create(T, 128, 256, T, valid_len_hint=(idx >= 0).sum(1))
        out, lse = api.mla_v4_launch_pipeline(dev(case["q"], torch.bfloat16), dev(case["kv"], torch.bfloat16), dev(idx), plan, SCALE,
                                              attn_sink=dev(sink) if use_sink else None,
                                              kv2=dev(kv2, torch.bfloat16) if use_pool else None,
                                              pool_split=dev(split) if use_pool else None)
        r_out, r_lse = oracle.sparse_mla_v4(case["q"], case["kv"], idx, SCALE, attn_sink=sink if use_sink else None,
                                            kv2=kv2 if use_pool else None, pool_split=split, s_q=T)
        tol = TOL_BF16
    torch.cuda.synchronize()
    check_out(out.view(torch.int16).cpu().numpy().view(np.uint16), r_out, **tol)
    check_lse(lse.cpu().numpy(), r_lse)
