"""Runs a synthetic case through the C ABI on the GPU and through the CPU oracle on the same bytes."""
import numpy as np
import torch

from opfoundry_b200 import api


def to_dev(case):
    d = {}
    d["q"] = torch.from_numpy(case["q"].view(np.int16)).cuda().view(torch.bfloat16)
    if case["fp8"]:
        d["kv"] = torch.from_numpy(case["kv"]).cuda()
    else:
        d["kv"] = torch.from_numpy(case["kv"].view(np.int16)).cuda().view(torch.bfloat16)
    d["indices"] = torch.from_numpy(case["indices"]).cuda()
    d["block_table"] = None if case["block_table"] is None else torch.from_numpy(case["block_table"]).cuda()
    return d


def run_gpu(case, sm_scale, *, valid_len_hint=None, poison_out=True, mtp_shared=None):
    d = to_dev(case)
    total_q, H = d["q"].shape[0], d["q"].shape[1]
    plan = api.mla_decode_plan_create(total_q, H, case["topk"], case["s_q"], valid_len_hint=valid_len_hint, mtp_shared=mtp_shared)
    out = torch.empty(total_q, H, 512, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(total_q, H, dtype=torch.float32, device="cuda")
    if poison_out:  # anything the kernels fail to write stays NaN
        out.fill_(float("nan"))
        lse.fill_(float("nan"))
    api.mla_decode_launch_pipeline(d["q"], d["kv"], d["indices"], plan, sm_scale, block_table=d["block_table"],
                                   page_block_size=case["page_block_size"],
                                   kv_batch_stride_rows=case["kv_batch_stride_rows"], out=out, lse=lse)
    torch.cuda.synchronize()
    return out.view(torch.int16).cpu().numpy().view(np.uint16), lse.cpu().numpy(), plan


def run_oracle(O, case, sm_scale, subset=None):
    return O.sparse_mla(case["q"], case["kv"], case["indices"], sm_scale, kv_is_fp8=case["fp8"],
                        block_table=case["block_table"], page_block_size=case["page_block_size"], s_q=case["s_q"],
                        kv_batch_stride_rows=case["kv_batch_stride_rows"], subset=subset)


def poison_unselected(case):
    """NaN-poisons every cache row no query selects, so one wrong gather shows up in the output
    (the idea of opus_attn/dsa_v4/common/mla_v4_host.cc:295-323)."""
    from oracle import oracle as O
    _, _, rows = O.sparse_mla(case["q"], case["kv"], case["indices"], 1.0, kv_is_fp8=case["fp8"],
                              block_table=case["block_table"], page_block_size=case["page_block_size"], s_q=case["s_q"],
                              kv_batch_stride_rows=case["kv_batch_stride_rows"], want_rows=True, num_threads=8)
    used = np.zeros(case["kv"].shape[0], bool)
    used[rows[rows >= 0]] = True
    kv = case["kv"].copy()
    if case["fp8"]:
        kv[~used, :512] = 0x7F                      # e4m3 NaN
        kv[~used, 512:528] = 0xFF                   # NaN scales
        kv[~used, 528:] = 0xFF
    else:
        kv[~used] = 0x7FC0                          # bf16 NaN
    out = dict(case)
    out["kv"] = kv
    return out, int((~used).sum())
