#!/usr/bin/env python
"""Verify-then-bench harness with the command line of the reference's own test program
(opus_attn/dsa_v32/common/host.cc:818-895):

    python tests/mla_decode_harness.py -dtype fp8 -h_q 128 -b 64 -s 32768 -s_q 1 [--varlen] [--verify]
                                       [-mode decode|prefill] [-topk 2048] [-page 64] [-pad_frac 0.05]
                                       [-seed 2026] [-warmup 100] [-iters 50]

Flags take `-flag value` or `-flag=value`, as there.  One run generates seeded inputs, (with --verify)
checks the GPU result against the CPU oracle on the same bytes and prints the reference's report lines
(host.cc:365-374, 399-403), then times the pipeline as the reference does (host.cc:263-320: plan outside
the loop, 100 warm-up + 50 timed launches between two events, mean) and prints its performance line, plus
one JSON line.  --varlen draws every sequence's length uniformly in [min(5, s), s] like init_kv_page_table
(host.cc:239-261) and hands the lengths to the planner.  Under torchrun every rank runs its own sequences.

This is test infrastructure (it imports the oracle); the library's own entry points are the C ABI.
"""
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

D_QK, D_V = 576, 512
DEFAULTS = dict(dtype="fp8", h_q=128, b=128, s=1024, s_q=1, varlen=False, verify=False, mode="decode", topk=2048,
                page=64, pad_frac=0.0, seed=2026, warmup=100, iters=50, ngpu=1)
INT_FLAGS = ("h_q", "b", "s", "s_q", "topk", "page", "seed", "warmup", "iters", "ngpu")


def parse_args(argv):
    """Returns the option dict or raises ValueError with the reference's wording for a bad argument."""
    o = dict(DEFAULTS)
    i = 0
    while i < len(argv):
        arg = argv[i]
        if arg == "--verify":
            o["verify"] = True
        elif arg == "--varlen":
            o["varlen"] = True
        elif arg.startswith("-") and not arg.startswith("--"):
            name, eq, val = arg[1:].partition("=")
            if name not in o or name in ("verify", "varlen"):
                raise ValueError("unknown argument '%s'" % arg)
            if not eq:
                if i + 1 >= len(argv):
                    raise ValueError("missing value for '%s'" % arg)
                i += 1
                val = argv[i]
            o[name] = int(val) if name in INT_FLAGS else (float(val) if name == "pad_frac" else val)
        else:
            raise ValueError("unknown argument '%s'" % arg)
        i += 1
    if min(o["h_q"], o["b"], o["s"], o["s_q"]) <= 0:
        raise ValueError("Invalid parameters. H_Q,B,S,S_Q must be positive.")
    if o["dtype"] not in ("fp8", "bf16"):
        raise ValueError("unknown -dtype '%s'; available: fp8, bf16" % o["dtype"])
    if o["mode"] not in ("decode", "prefill"):
        raise ValueError("unknown -mode '%s'; available: decode, prefill" % o["mode"])
    if o["mode"] == "prefill" and o["dtype"] != "bf16":
        raise ValueError("prefill runs on the bf16 cache")
    return o


def sequence_lengths(o):
    """Per-sequence kv lengths: all s, or uniform in [min(5, s), s] with the reference's seed."""
    import numpy as np
    if not o["varlen"]:
        return np.full(o["b"], o["s"], np.int64)
    return np.random.RandomState(1234).randint(min(5, o["s"]), o["s"] + 1, size=o["b"]).astype(np.int64)


def build_case(o, device="cuda"):
    """Device tensors of one run: q, cache, block table (fp8: paged), per-query lists, valid lengths."""
    import numpy as np
    import torch
    from opfoundry_b200 import workloads
    B, H, s, s_q, topk = o["b"], o["h_q"], o["s"], o["s_q"], o["topk"]
    if o["mode"] == "prefill":
        W = workloads.prefill_bf16(T=s, H=H, topk=topk, seed=o["seed"], device=device)
        return dict(q=W["q"], kv=W["kv"], indices=W["indices"], block_table=None, page=1, kv_batch_stride_rows=0, s_q=s,
                    valid_len=np.asarray(W["valid_len"], np.int64), fp8=False)
    lens = sequence_lengths(o)
    g = torch.Generator(device=device)
    g.manual_seed(o["seed"])
    total_q = B * s_q
    q = torch.randn(total_q, H, D_QK, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    idx = torch.full((total_q, topk), -1, dtype=torch.int32, device=device)
    valid = np.zeros(total_q, np.int64)
    for b in range(B):
        n = int(min(topk, lens[b]))
        n_keep = n - int(o["pad_frac"] * n)
        keys = torch.rand(s_q, int(lens[b]), generator=g, device=device)
        idx[b * s_q:(b + 1) * s_q, :n_keep] = keys.argsort(dim=1)[:, :n_keep].to(torch.int32)
        valid[b * s_q:(b + 1) * s_q] = n_keep
    if o["dtype"] == "fp8":
        page = o["page"]
        pages = (s + page - 1) // page
        cache = workloads.make_fp8_cache(B * pages * page, o["seed"] + 1, device)
        bt = torch.randperm(B * pages, generator=g, device=device).to(torch.int32).view(B, pages).contiguous()
        return dict(q=q, kv=cache, indices=idx, block_table=bt, page=page, kv_batch_stride_rows=0, s_q=s_q, valid_len=valid, fp8=True)
    kv = torch.randn(B * s, D_QK, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    return dict(q=q, kv=kv, indices=idx, block_table=None, page=1, kv_batch_stride_rows=s, s_q=s_q, valid_len=valid, fp8=False)


def report_out(ref_bits, gpu_bits, rtol, atol):
    """The reference validator's report (host.cc:322-374) with this build's bar: no mismatch budget."""
    import numpy as np
    r = (ref_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    g = (gpu_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    delta = np.abs(g - r)
    bad = ~np.isfinite(g) | (delta > atol + rtol * np.abs(r))
    nrms = math.sqrt(float((delta[np.isfinite(delta)] ** 2).sum()) / max(float((r ** 2).sum()), 1e-12))
    n_bad, n = int(bad.sum()), bad.size
    print("  rtol=%.0e atol=%.0e | max_abs_delta=%.6f nrms=%.3e | mismatch %d/%d (%.2f%%)" % (
        rtol, atol, float(np.nanmax(delta)) if n else 0.0, nrms, n_bad, n, 100.0 * n_bad / max(n, 1)))
    print(("✓ Validation passed (checked %d elements)" % n) if n_bad == 0 else
          ("✗ Validation failed (mismatch ratio %.2f%% > 0.00%%)" % (100.0 * n_bad / max(n, 1))))
    return n_bad == 0


def report_lse(ref, gpu, rtol=1e-3, atol=1e-3):
    import numpy as np
    ri, gi = np.isinf(ref), np.isinf(gpu)
    inf_bad = (ri != gi) | (ri & gi & (np.signbit(ref) != np.signbit(gpu)))
    fin = ~ri & ~gi
    delta = np.abs(gpu[fin].astype(np.float64) - ref[fin].astype(np.float64))
    bad = int(inf_bad.sum()) + int((np.isnan(gpu[fin]) | (delta > atol + rtol * np.abs(ref[fin]))).sum())
    print("  LSE: rtol=%.0e atol=%.0e | max_abs_delta=%.6f | mismatch %d/%d" % (
        rtol, atol, float(delta.max()) if delta.size else 0.0, bad, ref.size))
    print("✓ LSE validation passed (checked %d elements)" % ref.size if bad == 0 else "✗ LSE validation failed")
    return bad == 0


def main(argv=None):
    try:
        o = parse_args(sys.argv[1:] if argv is None else argv)
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 1
    import ctypes as C
    import numpy as np
    import torch
    from opfoundry_b200 import api
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")
        o = dict(o, seed=o["seed"] + rank)          # every rank its own sequences, nothing exchanged
    sm_scale = 1.0 / math.sqrt(192.0)
    case = build_case(o)
    total_q, H, topk = case["q"].shape[0], o["h_q"], o["topk"]
    plan = api.mla_decode_plan_create(total_q, H, topk, case["s_q"], valid_len_hint=case["valid_len"])
    out = torch.empty(total_q, H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(total_q, H, dtype=torch.float32, device="cuda")
    a = api.make_args(case["q"], case["kv"], case["indices"], plan, sm_scale, out=out, lse=lse, block_table=case["block_table"],
                      page_block_size=case["page"], kv_batch_stride_rows=case["kv_batch_stride_rows"])
    L = api.lib()
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    api._check(L.dsa_v32_decode_pipeline(C.byref(a), 0, st()), "pipeline")
    api._check(L.dsa_v32_device_status(C.byref(a), st()), "device status")
    ok = True
    if o["verify"] and rank == 0:
        from oracle import build as obuild
        obuild.build_oracle()
        from oracle import oracle as O
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
        # the CPU oracle is ~0.6 us per (query-head, row): verify every query while that stays within ~20 s
        budget_rows = int(3e7 / max(H, 1))
        csum = np.cumsum(case["valid_len"])
        n_ver = int(max(1, min(total_q, np.searchsorted(csum, budget_rows, side="right"))))
        subset = np.unique(np.round(np.linspace(0, total_q - 1, n_ver)).astype(np.int32)) if n_ver < total_q else None
        kv_host = case["kv"].cpu().numpy() if case["fp8"] else bits(case["kv"])
        r_out, r_lse = O.sparse_mla(bits(case["q"]), kv_host, case["indices"].cpu().numpy(), sm_scale, kv_is_fp8=case["fp8"],
                                    block_table=None if case["block_table"] is None else case["block_table"].cpu().numpy(),
                                    page_block_size=case["page"], s_q=case["s_q"], kv_batch_stride_rows=case["kv_batch_stride_rows"],
                                    subset=subset)
        sel = slice(None) if subset is None else subset
        print("verify: %d of %d query rows against the CPU oracle" % (total_q if subset is None else len(subset), total_q))
        ok = report_out(r_out[sel], bits(out)[sel], 1e-2, 5e-2 if case["fp8"] else 2e-2)
        ok = report_lse(r_lse[sel], lse.cpu().numpy()[sel]) and ok
    # ---- benchmark: the reference's protocol
    for _ in range(o["warmup"]):
        L.dsa_v32_decode_pipeline(C.byref(a), 0, st())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(o["iters"]):
        L.dsa_v32_decode_pipeline(C.byref(a), 0, st())
    e1.record()
    torch.cuda.synchronize()
    api._check(L.dsa_v32_device_status(C.byref(a), st()), "device status")
    avg_ms = e0.elapsed_time(e1) / max(o["iters"], 1)
    total_kv = float(np.sum(case["valid_len"]))
    flops = 2.0 * H * total_kv * (D_QK + D_V)
    row_bytes = 656 if case["fp8"] else 1152
    nbytes = total_q * H * D_QK * 2 + total_q * H * D_V * 2 + total_kv * row_bytes
    if rank == 0:
        print("MLA decode performance: avg_time=%.3f ms, %.2f TFlops, %.2f TB/s" % (avg_ms, flops / (avg_ms * 1e-3) / 1e12,
                                                                                    nbytes / (avg_ms * 1e-3) / 1e12))
        print(json.dumps(dict(harness="mla_decode", options={k: o[k] for k in sorted(o)}, avg_ms=avg_ms,
                              tflops=flops / (avg_ms * 1e-3) / 1e12, pairs=total_kv, verified=bool(o["verify"]), ok=bool(ok),
                              num_lists=plan.info.num_lists, num_works=plan.info.num_works, num_partials=plan.info.num_partials)))
    if world > 1:
        dist.destroy_process_group()
    return 0 if ok else 2


if __name__ == "__main__":
    sys.exit(main())
