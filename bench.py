#!/usr/bin/env python
"""Benchmark of the sparse-MLA hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this library (one process per GPU)
    python bench.py --impl reference --steps K --warmup W    the reference's CPU path on the host cores

A step is one pass of the decode pipeline (attention kernel + split merge; the plan is built once
outside the loop, as the reference keeps its metadata kernel out of the timed loop) over one batch of
the fp8 decode workload: batch 64, 128 heads, top-k 2048 (last 5 % of slots -1), kv_len 32768 in a
paged fp8 cache of 64-token blocks with a permuted block table.  Successive steps use different
batches (queries and index lists) so the rows gathered by consecutive steps exceed the L2.
With N > 1 every rank runs its own batch of 64 sequences against its own cache (the path shards by
sequence with no exchange), so scaling is weak and `value` is the sum over ranks.

Prints one JSON line (rank 0).  `value` is TFLOP/s of algorithmic work, 2 * H * (576 + 512) * pairs,
pairs = valid (query, position) slots, with inputs resident in HBM; `e2e` is the same through the
host-buffer C-ABI call with pinned host queries / index lists in and outputs back every step.
"""
import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_QK, D_V = 576, 512
CFG = dict(B=64, H=128, kv_len=32768, topk=2048, page=64, pad_frac=0.05, n_batches=4)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)
# dram bytes (read + write) of one attention-kernel launch on the workload above, from the ncu
# capture summarised in profiles/ (null until a capture exists for the current kernel)
NCU_TRAFFIC_BYTES_AT_BATCH16 = 28.46e6  # dram read + write of one launch captured at batch 16 (profiles/sparse_mla_fp8_decode_cluster_kernel.md)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]), source="measured")
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _once(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        for bit, name in names.items():
            if r & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._once()
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
            try:
                self._once()
            except Exception:
                pass

    def summary(self):
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=[], samples=0)
        s = sorted(self.samples)
        return dict(sm_mhz=s[len(s) // 2], sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons), samples=len(s))


def flops_of(pairs, H):
    return 2.0 * H * (D_QK + D_V) * pairs


# --------------------------------------------------------------------------- reference CPU path
def reference_cpu(sample_queries, n_valid, H, repeats=1):
    """Times the reference's own CPU function (host.cc:459-506, compiled as oracle/_ref) on
    `sample_queries` decode queries of n_valid rows each, in its own input format (MXFP8 tensors
    made by its own generator), on all host threads it uses.  Returns (seconds per pass, cores)."""
    import numpy as np
    from oracle import oracle as O
    R = O.ref_lib()
    kind = "reference"
    if R is None:
        kind = "port"
    B = sample_queries
    rows = B * n_valid
    cores = int(os.environ.get("MLA_DECODE_NUM_THREADS", os.cpu_count() or 1))
    if R is not None:
        qn = np.zeros((B * H, 512), np.uint8); qs = np.zeros((B * H, 16), np.uint8); qr = np.zeros((B * H, 64), np.uint16)
        kn = np.zeros((rows, 512), np.uint8); ks = np.zeros((rows, 16), np.uint8); kr = np.zeros((rows, 64), np.uint16)
        R.ref_init_fp8_split(O._p(qn), O._p(qs), O._p(qr), B * H)
        R.ref_init_fp8_split(O._p(kn), O._p(ks), O._p(kr), rows)
        ip = (np.arange(B + 1) * n_valid).astype(np.int32)
        ix = np.random.default_rng(0).permutation(rows).astype(np.int32)
        out = np.zeros((B, H, 512), np.uint16); lse = np.zeros((B, H), np.float32)
        best = None
        for _ in range(repeats):
            t0 = time.perf_counter()
            R.ref_attention_fp8(O._p(qn), O._p(qs), O._p(qr), O._p(kn), O._p(ks), O._p(kr), O._p(out), O._p(lse),
                                O._p(ip), O._p(ix), B, H, 1)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best, cores, kind
    # the reference build is absent: time the restatement on the same amount of work
    from opfoundry_b200 import synth
    case = synth.make_decode_case(B, H, max(n_valid, 64), n_valid, fp8=True, seed=1)
    t0 = time.perf_counter()
    O.sparse_mla(case["q"], case["kv"], case["indices"], 1 / math.sqrt(192), kv_is_fp8=True, kv_batch_stride_rows=case["kv_batch_stride_rows"],
                 num_threads=cores)
    return time.perf_counter() - t0, cores, kind


def cpu_baseline_block(budget_s=15.0):
    H, n_valid = CFG["H"], CFG["topk"] - int(CFG["pad_frac"] * CFG["topk"])
    t1, cores, kind = reference_cpu(1, n_valid, H)
    n = max(1, min(CFG["B"], int(budget_s / max(t1, 1e-3))))
    t, cores, kind = reference_cpu(n, n_valid, H)
    tf = flops_of(n * n_valid, H) / t / 1e12
    return dict(value=tf, unit="TFLOP/s", cores=cores, kind=kind, seconds=round(t, 3),
                sample="%d of %d decode queries x %d heads x %d valid rows, reference fp8 CPU function" % (n, CFG["B"], H, n_valid))


def run_reference_arm(args, rank):
    if rank != 0:
        return
    H, n_valid = CFG["H"], CFG["topk"] - int(CFG["pad_frac"] * CFG["topk"])
    t1, cores, kind = reference_cpu(1, n_valid, H)
    total_passes = args.steps + args.warmup
    n = max(1, min(CFG["B"], int(150.0 / max(t1 * total_passes, 1e-3))))
    for _ in range(args.warmup):
        reference_cpu(n, n_valid, H)
    times = [reference_cpu(n, n_valid, H)[0] for _ in range(args.steps)]
    t = sum(times) / len(times)
    tf = flops_of(n * n_valid, H) / t / 1e12
    sample = "each step = %d of %d decode queries x %d heads x %d valid rows through the reference's CPU function" % (n, CFG["B"], H, n_valid)
    line = dict(impl="reference", metric="sparse_mla_decode_fp8_tflops", value=tf, unit="TFLOP/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=t * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="fp32 (CPU reference arithmetic)", data="synthetic",
                config=workload_config(), cpu_baseline=dict(value=tf, unit="TFLOP/s", cores=cores, kind=kind, sample=sample),
                e2e=dict(value=tf, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def workload_config():
    return dict(workload="decode_fp8_b64_h128_topk2048_kv32768_paged64", batch=CFG["B"], heads=CFG["H"], topk=CFG["topk"],
                kv_len=CFG["kv_len"], page_block=CFG["page"], pad_frac=CFG["pad_frac"], d_qk=D_QK, d_v=D_V,
                sm_scale="1/sqrt(192)", sharding="one batch of 64 sequences per GPU, no exchange",
                l2="%d rotating batches gather %.0f MB of distinct rows > 126 MB L2" % (
                    CFG["n_batches"], CFG["n_batches"] * CFG["B"] * (CFG["topk"] * (1 - CFG["pad_frac"])) * 656 / 1e6),
                valid_len_hint="given to the planner (the analogue of the reference's kv_indptr lengths)")


def run_prefill(args, rank, world, local_rank, torch, dist, api, workloads):
    """bf16 causal prefill: one sequence of T tokens, 128 heads, top-k 2048; a step = the whole prefill.
    With N > 1 ranks the query tokens are cut into contiguous chunks of equal work, the latent cache is
    replicated and nothing is exchanged (strong scaling of one sequence)."""
    from opfoundry_b200 import shard
    import numpy as np
    T, H, topk = args.tokens, CFG["H"], CFG["topk"]
    valid_all = np.minimum(np.arange(T) + 1, topk)
    bounds = shard.shard_queries_equal_work(valid_all, world)
    q0, q1 = bounds[rank], bounds[rank + 1]
    W = workloads.prefill_bf16(T=T, H=H, topk=topk, seed=2026, q_begin=q0, q_end=q1)
    nq = q1 - q0
    plan = api.mla_decode_plan_create(nq, H, topk, nq, valid_len_hint=W["valid_len"])
    out = torch.empty(nq, H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(nq, H, dtype=torch.float32, device="cuda")
    a = api.make_args(W["q"], W["kv"], W["indices"], plan, 1.0 / math.sqrt(192.0), out=out, lse=lse)
    L = api.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        api._check(L.dsa_v32_decode_pipeline(C.byref(a), 0, stream), "prefill")
    torch.cuda.synchronize()
    api._check(L.dsa_v32_device_status(C.byref(a), stream), "device status")
    K = args.steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0.record()
    for _ in range(K):
        api._check(L.dsa_v32_decode_pipeline(C.byref(a), 0, stream), "prefill")
    e1.record()
    barrier()
    sampler.stop()
    ms = shard.max_over_ranks([e0.elapsed_time(e1)], "cuda")[0] / K
    total_pairs = float(valid_all.sum())
    if rank == 0:
        pk = peaks()
        flops = flops_of(total_pairs, H)
        tf = flops / (ms * 1e-3) / 1e12
        print(json.dumps(dict(
            metric="sparse_mla_prefill_bf16_tflops", value=tf, unit="TFLOP/s", n_gpus=world, steps=K, warmup=args.warmup,
            ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16 MMA, fp32 accumulate",
            data="synthetic",
            config=dict(workload="prefill_bf16_t%d_h128_topk2048_causal" % T, tokens=T, heads=H, topk=topk, pairs=total_pairs,
                        sharding="contiguous query chunks of equal work, latent cache replicated, no exchange",
                        l2="gathered rows per step %.1f GB from a %.1f MB cache (L2-resident by construction of the config)" % (
                            total_pairs * 1152 / 1e9, T * 1152 / 1e6)),
            roofline=dict(bound="tensor", achieved=tf, peak=pk["bf16_tflops"], unit="TFLOP/s", frac=tf / pk["bf16_tflops"],
                          traffic=None, peak_source=pk["source"], kernel="sparse_mla_kernel<bf16>",
                          flops_per_launch=flops, gathered_bytes_per_launch=total_pairs * 1152.0),
            gpu_launches=K * (2 if plan.info.num_partials > 0 else 1), clocks=sampler.summary())), flush=True)


def run_decode_tp(args, rank, world, local_rank, torch, dist, api, workloads):
    """fp8 decode with one MTP token, head-sharded (the TP layout of a serving stack): batch 128, two
    query rows per sequence (half of the sequences share one index list between their rows), 128 heads in
    total of which every rank attends 128 / N, kv_len 65536 in 64-token pages, top-k 2048, the latent cache
    replicated on every rank; a step = attention on the local heads + one NCCL all-gather of the outputs.
    Strong scaling: the total work is fixed.  Note what the layout costs: the tensor-core tile has 128 rows
    (heads), so a rank with 128 / N heads still pays for 128, while its gathered bytes stay the same."""
    from opfoundry_b200 import shard
    B, s_q, H_all, kv_len, topk, page = args.batch if args.batch != 64 else 128, 2, 128, 65536, 2048, 64
    h0, h1 = shard.shard_heads(H_all, world, rank)
    Hl = h1 - h0
    W = workloads.decode_fp8(B=B, H=H_all, kv_len=kv_len, topk=topk, page=page, pad_frac=0.0, n_batches=2, seed=2026, s_q=s_q)
    total_q = B * s_q
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    share = torch.rand(B, generator=g, device="cuda") < 0.5          # sequences whose two rows share a list
    steps = []
    for q, idx in W["steps"]:
        idx = idx.clone().view(B, s_q, topk)
        idx[share, 1] = idx[share, 0]
        steps.append((q[:, h0:h1].contiguous(), idx.view(total_q, topk).contiguous()))
    plan = api.mla_decode_plan_create(total_q, Hl, topk, s_q)
    out = torch.empty(total_q, Hl, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(total_q, Hl, dtype=torch.float32, device="cuda")
    gathered = torch.empty(world, total_q, Hl, D_V, dtype=torch.bfloat16, device="cuda")   # rank-major; heads of rank r = block r
    arg_sets = [api.make_args(q, W["cache"], idx, plan, 1.0 / math.sqrt(192.0), out=out, lse=lse, block_table=W["block_table"],
                              page_block_size=page) for q, idx in steps]
    L = api.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def step(i):
        api._check(L.dsa_v32_decode_pipeline(C.byref(arg_sets[i % len(arg_sets)]), 0, stream), "decode step")
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    api._check(L.dsa_v32_device_status(C.byref(arg_sets[0]), stream), "device status")
    K = args.steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0.record()
    for i in range(K):
        step(i)
    e1.record()
    barrier()
    sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / K
    if rank == 0:
        pk = peaks()
        pairs = float(total_q * topk)
        flops = flops_of(pairs, H_all)
        tf = flops / (ms * 1e-3) / 1e12
        launches = (2 if plan.info.num_partials > 0 else 1)
        print(json.dumps(dict(
            metric="sparse_mla_decode_fp8_mtp_tp_tflops", value=tf, unit="TFLOP/s", n_gpus=world, steps=K, warmup=args.warmup,
            ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None,
            dtype="bf16 MMA, fp32 accumulate (fp8 e4m3 cache)", data="synthetic",
            config=dict(workload="decode_fp8_mtp_b%d_sq2_h128_topk2048_kv65536_paged64_tp%d" % (B, world), batch=B, s_q=s_q,
                        heads_total=H_all, heads_per_gpu=Hl, topk=topk, kv_len=kv_len,
                        sharding="heads sharded %d per GPU, latent cache replicated, one NCCL all-gather of the outputs per step" % Hl,
                        l2="every step gathers %.0f MB of rows > 126 MB L2" % (pairs * 656 / 1e6)),
            roofline=dict(bound="tensor", achieved=tf, peak=world * pk["bf16_tflops"], unit="TFLOP/s",
                          frac=tf / (world * pk["bf16_tflops"]), traffic=None, peak_source=pk["source"],
                          kernel="sparse_mla_kernel<fp8> + all-gather", flops_per_launch=flops / world,
                          gathered_bytes_per_launch=pairs * 656.0),
            gpu_launches=K * launches, clocks=sampler.summary())), flush=True)


def e2e_leg(api, torch, W, plan, sm_scale, out, lse, K, barrier):
    """K steps through the host-buffer C-ABI call: pinned host q / index lists in, out / lse back,
    the caller synchronising on every step's result."""
    B, H = W["B"], W["H"]
    q_host = [q.cpu().pin_memory() for (q, _) in W["steps"]]
    i_host = [idx.cpu().pin_memory() for (_, idx) in W["steps"]]
    out_host = torch.empty(B, H, D_V, dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty(B, H, dtype=torch.float32).pin_memory()
    q_dev = torch.empty_like(W["steps"][0][0])
    i_dev = torch.empty_like(W["steps"][0][1])
    a_e2e = api.make_args(q_dev, W["cache"], i_dev, plan, sm_scale, out=out, lse=lse, block_table=W["block_table"],
                          page_block_size=W["page"])
    for i in range(3):
        api.mla_decode_step_host(a_e2e, q_host[i % len(q_host)], i_host[i % len(i_host)], out_host, lse_host)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record()
    for i in range(K):
        api.mla_decode_step_host(a_e2e, q_host[i % len(q_host)], i_host[i % len(i_host)], out_host, lse_host)
        torch.cuda.current_stream().synchronize()   # the caller reads the step's result before the next step
    g1.record()
    barrier()
    h2d = q_host[0].numel() * 2 + i_host[0].numel() * 4
    d2h = out_host.numel() * 2 + lse_host.numel() * 4
    return g0.elapsed_time(g1), h2d, d2h


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--batch", type=int, default=CFG["B"], help="sequences per GPU (smaller only for profiler captures)")
    ap.add_argument("--workload", default="decode_fp8", choices=["decode_fp8", "prefill_bf16", "decode_fp8_tp"],
                    help="decode_fp8: the headline; prefill_bf16: one causal prefill (second half of the metric; --tokens 131072 "
                         "with --gpus 8 is the query-chunk-sharded long prefill); decode_fp8_tp: MTP decode with the heads "
                         "sharded over the GPUs and an all-gather of the outputs")
    ap.add_argument("--tokens", type=int, default=4096, help="prefill_bf16: sequence length")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    CFG["B"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    from opfoundry_b200 import api, build, workloads
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not os.path.exists(api.LIB_PATH):
        if rank == 0:
            build.build()
        if world > 1:
            dist.barrier()
    api.lib()
    if args.workload == "prefill_bf16":
        run_prefill(args, rank, world, local_rank, torch, dist, api, workloads)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "decode_fp8_tp":
        run_decode_tp(args, rank, world, local_rank, torch, dist, api, workloads)
        if world > 1:
            dist.destroy_process_group()
        return

    W = workloads.decode_fp8(B=CFG["B"], H=CFG["H"], kv_len=CFG["kv_len"], topk=CFG["topk"], page=CFG["page"],
                             pad_frac=CFG["pad_frac"], n_batches=CFG["n_batches"], seed=2026 + rank)
    B, H, topk, n_valid = W["B"], W["H"], W["topk"], W["n_valid"]
    pairs = B * n_valid
    step_flops = flops_of(pairs, H)
    plan = api.mla_decode_plan_create(B, H, topk, 1, valid_len_hint=[n_valid] * B)
    out = torch.empty(B, H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
    sm_scale = 1.0 / math.sqrt(192.0)
    arg_sets = [api.make_args(q, W["cache"], idx, plan, sm_scale, out=out, lse=lse, block_table=W["block_table"],
                              page_block_size=W["page"]) for (q, idx) in W["steps"]]
    L = api.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def step(i):
        a = arg_sets[i % len(arg_sets)]
        rc = L.dsa_v32_decode_fp8(C.byref(a), stream)
        if rc == 0:
            rc = L.dsa_v32_combine(C.byref(a), stream)
        if rc:
            raise api.DsaError(rc, "decode step")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    st = L.dsa_v32_device_status(C.byref(arg_sets[0]), stream)
    if st:
        raise api.DsaError(st, "device status after warm-up")

    K = args.steps
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0.record()
    for i in range(K):
        a = arg_sets[i % len(arg_sets)]
        ev_a[i].record()
        rc = L.dsa_v32_decode_fp8(C.byref(a), stream)
        ev_b[i].record()
        rc = rc or L.dsa_v32_combine(C.byref(a), stream)
        if rc:
            raise api.DsaError(rc, "decode step")
    e1.record()
    barrier()
    sampler.stop()
    total_ms = e0.elapsed_time(e1)
    attn_ms = sum(a.elapsed_time(b) for a, b in zip(ev_a, ev_b)) / K
    st = L.dsa_v32_device_status(C.byref(arg_sets[0]), stream)
    if st:
        raise api.DsaError(st, "device status after the timed region")

    e2e_ms, h2d, d2h = float("nan"), 0, 0
    if not args.no_e2e:
        e2e_ms, h2d, d2h = e2e_leg(api, torch, W, plan, sm_scale, out, lse, K, barrier)

    t = torch.tensor([total_ms, attn_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, attn_ms, e2e_ms = (float(x) for x in t.tolist())
    clocks = sampler.summary()
    if rank == 0:
        pk = peaks()
        ms_per_step = total_ms / K
        value = world * step_flops / (ms_per_step * 1e-3) / 1e12
        attn_tf = step_flops / (attn_ms * 1e-3) / 1e12
        gathered = pairs * 656.0
        line = dict(metric="sparse_mla_decode_fp8_tflops", value=value, unit="TFLOP/s", n_gpus=world, steps=K,
                    warmup=args.warmup, ms_per_step=ms_per_step, us_per_step=ms_per_step * 1e3, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="bf16 MMA, fp32 accumulate (fp8 e4m3 cache)", data="synthetic",
                    config=workload_config(),
                    roofline=dict(bound="tensor", achieved=attn_tf, peak=pk["bf16_tflops"], unit="TFLOP/s",
                                  frac=attn_tf / pk["bf16_tflops"], traffic=NCU_TRAFFIC_BYTES_AT_BATCH16 * B / 16.0,
                                  peak_source=pk["source"], kernel="sparse_mla_kernel<fp8>", kernel_us=attn_ms * 1e3,
                                  flops_per_launch=step_flops, gathered_bytes_per_launch=gathered,
                                  gathered_gbs=gathered / (attn_ms * 1e-3) / 1e9, hbm_peak_gbs=pk["hbm_gbs"],
                                  t_flop_us=step_flops / (pk["bf16_tflops"] * 1e12) * 1e6,
                                  t_mem_us=gathered / (pk["hbm_gbs"] * 1e9) * 1e6),
                    e2e=None if args.no_e2e else dict(value=world * step_flops / (e2e_ms / K * 1e-3) / 1e12, unit="TFLOP/s",
                                                      ms_per_step=e2e_ms / K, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
                    gpu_launches=K * (2 if plan.info.num_partials > 0 else 1), clocks=clocks)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_block()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
