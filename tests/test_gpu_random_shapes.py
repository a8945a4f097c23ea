"""Seeded random shapes through the C ABI against the oracle: batch, heads, rows per sequence, cache type,
page size, top-k (including 1 and sizes around the 32-row tile), padding at the tail or scattered, lengths
given to the planner or not, MTP rows sharing a list or not.  Every case is small enough for the oracle."""
import math
import random

import numpy as np
import pytest

from helpers import TOL_BF16, TOL_FP8, check_lse, check_out
from opfoundry_b200 import synth

pytestmark = pytest.mark.gpu

SCALE = 1.0 / math.sqrt(192.0)


def draw_case(rng):
    fp8 = rng.random() < 0.6
    H = rng.choice([8, 16, 32, 64, 128, 128, 128, 192])
    s_q = rng.choice([1, 1, 2, 4]) if H <= 64 else rng.choice([1, 1, 2])
    B = rng.randint(1, 6)
    page = rng.choice([64, 64, 16, 128])
    paged = fp8 or rng.random() < 0.5
    kv_len = rng.choice([256, 512, 1024, 2048])
    if paged:
        kv_len = max(page, kv_len // page * page)
    topk = min(rng.choice([1, 31, 32, 33, 64, 100, 160, 257, 512, 1000]), kv_len)
    pad = rng.choice([0.0, 0.0, 0.05, 0.3, 0.9])
    share = "coin" if s_q > 1 and rng.random() < 0.6 else None
    case = synth.make_decode_case(B, H, kv_len, topk, s_q=s_q, fp8=fp8, paged=paged, page_block_size=page, pad_frac=pad,
                                  share_mtp=share, seed=rng.randint(1, 10 ** 6), scatter_pad=rng.random() < 0.3)
    hint = None
    if rng.random() < 0.5 and pad > 0:
        valid = (case["indices"] >= 0).sum(axis=1)
        if all((row[:n] >= 0).all() for row, n in zip(case["indices"], valid)):   # only a tail of -1 may be hinted
            hint = valid.tolist()
    mtp = None
    if share == "coin":
        idx = case["indices"].reshape(B, s_q, topk)
        mtp = np.array([all((idx[b, t] == idx[b, 0]).all() for t in range(s_q)) for b in range(B)], dtype=np.uint8)
    what = "fp8=%s B=%d H=%d s_q=%d kv=%d topk=%d page=%d paged=%s pad=%.2f share=%s hint=%s" % (
        fp8, B, H, s_q, kv_len, topk, page, paged, pad, share, hint is not None)
    return case, hint, mtp, fp8, what


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_match_the_oracle(oracle, seed):
    from gpu_util import run_gpu, run_oracle
    rng = random.Random(seed)
    for _ in range(12):
        case, hint, mtp, fp8, what = draw_case(rng)
        g_out, g_lse, _ = run_gpu(case, SCALE, valid_len_hint=hint, mtp_shared=mtp)
        r_out, r_lse = run_oracle(oracle, case, SCALE)
        try:
            check_out(g_out, r_out, **(TOL_FP8 if fp8 else TOL_BF16))
            check_lse(g_lse, r_lse)
        except AssertionError as e:
            raise AssertionError(what + ": " + str(e)[:400])
