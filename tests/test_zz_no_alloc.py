"""The no-allocation entry point (dsa_v32_decode_pipeline_static) against the regular pipeline.

Some hosts of this library may not allocate device memory once they are running - a plugin inside a
process that owns the memory pool, a serving loop that must stay out of the allocator.  For them the
library carries its split workspace inside its own device image.  This test calls that entry point
through the C ABI twice in a row (the array is shared and keeps the previous call's contents, so the
second call is the one that proves nothing stale leaks through) and compares with the regular entry
point on the same inputs, with the tolerances the other parity tests use.  It is collected last.
"""
import math

import numpy as np
import pytest
import torch

from helpers import TOL_FP8, TOL_BF16, check_lse, check_out
from opfoundry_b200 import api, synth

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(192.0)


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("fp8", [True, False])
def test_static_scratch_matches_regular_pipeline_twice(built_lib, fp8):
    assert torch.cuda.is_available()
    from gpu_util import to_dev
    tol = TOL_FP8 if fp8 else TOL_BF16
    # two different problems of the same shape, run back to back through the shared array
    cases = [synth.make_decode_case(6, 128, 2048, 700, fp8=fp8, paged=True, pad_frac=0.1, seed=900 + i) for i in range(2)]
    for n_call, case in enumerate(cases):
        d = to_dev(case)
        plan = api.mla_decode_plan_create(6, 128, 700, 1)
        assert plan.info.num_partials > 0          # the shape really uses split scratch
        ref_out, ref_lse = api.mla_decode_launch_pipeline(d["q"], d["kv"], d["indices"], plan, SCALE,
                                                          block_table=d["block_table"], page_block_size=64)
        out = torch.full((6, 128, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((6, 128), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        api.mla_decode_launch_pipeline_static(d["q"], d["kv"], d["indices"], SCALE, block_table=d["block_table"],
                                              page_block_size=64, out=out, lse=lse)
        torch.cuda.synchronize()
        if n_call > 0:
            # the property in the entry point's name: with the outputs handed in, a call leaves the device's free
            # memory where it was (the first call on a device may still load the library's image with its array)
            assert torch.cuda.mem_get_info()[0] == free_before
        check_out(_bits(out), _bits(ref_out), **tol)
        check_lse(lse.cpu().numpy(), ref_lse.cpu().numpy())


def test_static_scratch_rejects_shapes_beyond_its_size(built_lib):
    assert torch.cuda.is_available()
    # The split partials are bounded by the number of work lists (at most two per list boundary), so only
    # the per-unit tables of a very long query list outgrow the array: probe with one head and top-k 1.
    H, topk = 1, 1
    total_q = None
    for cand in (1_700_000, 2_400_000, 4_800_000):
        sh, _ = api._shape(cand, H, topk, 1, 0, None)
        info = api.PlanInfo()
        api._check(api.lib().dsa_v32_plan_info_get(sh, info), "dsa_v32_plan_info_get")
        if info.workspace_bytes > api.STATIC_SCRATCH_BYTES:
            total_q = cand
            break
    assert total_q is not None, "no probe shape exceeds the static scratch on this device"
    q = torch.zeros(total_q, H, 576, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(4096, 576, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(total_q, topk, dtype=torch.int32, device="cuda")
    with pytest.raises(api.DsaError) as e:
        api.mla_decode_launch_pipeline_static(q, kv, idx, SCALE, kv_batch_stride_rows=0)
    assert e.value.status == api.ERR_SCRATCH_TOO_SMALL
