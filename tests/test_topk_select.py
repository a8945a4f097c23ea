"""The index-list producer (dsa_v32_topk_select) against a numpy selection on the same scores: exact sets,
ties at the threshold resolved toward the lower position, -1 padding, NaN never preferred; and its output
driving the attention (select -> gather -> attend) against the oracle."""
import math

import numpy as np
import pytest
import torch

from opfoundry_b200 import api, synth

pytestmark = pytest.mark.gpu


def numpy_select(scores, topk, valid_len):
    total_q, kv_len = scores.shape
    out = np.full((total_q, topk), -1, np.int32)
    for q in range(total_q):
        n = kv_len if valid_len is None else int(valid_len[q])
        s = scores[q, :n].astype(np.float64)
        s[np.isnan(s)] = -np.inf
        order = np.lexsort((np.arange(n), -s))          # by score descending, then position ascending
        k = min(topk, n)
        out[q, :k] = np.sort(order[:k])
    return out


@pytest.mark.parametrize("kv_len,topk", [(4096, 2048), (32768, 2048), (1000, 64), (517, 600), (70000, 512)])
def test_select_matches_numpy(built_lib, kv_len, topk):
    g = torch.Generator(device="cuda")
    g.manual_seed(kv_len + topk)
    total_q = 12
    scores = torch.randn(total_q, kv_len, generator=g, device="cuda")
    scores[1] = torch.round(scores[1] * 2) / 2                       # heavy ties
    scores[2] = 0.0                                                   # all equal
    scores[3, ::7] = float("nan")
    scores[4] = -scores[4].abs()                                      # all negative
    scores[5, :10] = float("inf")
    valid = torch.full((total_q,), kv_len, dtype=torch.int32, device="cuda")
    valid[6], valid[7], valid[8], valid[9] = 0, 1, min(topk, kv_len) - 1 if topk > 1 else 1, min(kv_len, topk + 1)
    got = api.topk_select(scores, topk, valid).cpu().numpy()
    want = numpy_select(scores.cpu().numpy(), topk, valid.cpu().numpy())
    assert np.array_equal(got, want)
    got2 = api.topk_select(scores, topk).cpu().numpy()
    assert np.array_equal(got2, numpy_select(scores.cpu().numpy(), topk, None))


def test_select_then_attend(built_lib, oracle):
    """Lists produced on the device feed the attention kernel directly; the oracle gets the same lists."""
    from gpu_util import to_dev
    from helpers import TOL_FP8, check_lse, check_out
    B, H, kv_len, topk = 4, 128, 2048, 512
    case = synth.make_decode_case(B, H, kv_len, topk, fp8=True, paged=True, seed=31)
    d = to_dev(case)
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    scores = torch.randn(B, kv_len, generator=g, device="cuda")
    valid = torch.tensor([kv_len, 300, kv_len, 1500], dtype=torch.int32, device="cuda")
    idx = api.topk_select(scores, topk, valid)
    plan = api.mla_decode_plan_create(B, H, topk, 1, valid_len_hint=[min(topk, int(v)) for v in valid.cpu()])
    scale = 1.0 / math.sqrt(192.0)
    out, lse = api.mla_decode_launch_pipeline(d["q"], d["kv"], idx, plan, scale, block_table=d["block_table"], page_block_size=64)
    torch.cuda.synchronize()
    r_out, r_lse = oracle.sparse_mla(case["q"], case["kv"], idx.cpu().numpy(), scale, kv_is_fp8=True,
                                     block_table=case["block_table"], page_block_size=64)
    check_out(out.view(torch.int16).cpu().numpy().view(np.uint16), r_out, **TOL_FP8)
    check_lse(lse.cpu().numpy(), r_lse)
