#!/usr/bin/env python
"""Benchmark of the sparse-MLA hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this library (one process per GPU)
    python bench.py --impl reference --steps K --warmup W    the reference's CPU path on the host cores

Headline (the JSON line's `value`): a step is one pass of the decode pipeline (attention kernel + split
merge; the plan is built once outside the loop, as the reference keeps its metadata kernel out of the timed
loop) over one batch of the fp8 decode workload: batch 64, 128 heads, top-k 2048 (last 5 % of slots -1),
kv_len 32768 in a paged fp8 cache of 64-token blocks with a permuted block table.  Successive steps use
different batches (queries and index lists) so the rows gathered by consecutive steps exceed the L2.
With N > 1 every rank runs its own batch of 64 sequences against its own cache (replicas: the path shards
by sequence with no exchange), so that number scales weakly and `value` is the sum over ranks.

The same line carries, measured in the same run:
  `prefill`  (N = 1)  the other half of the metric: the 4096-token causal bf16 prefill, with its own
                      roofline and CPU baseline;
  `sharded`  (every N) the configurations that are partitioned over the GPUs of the box, each over the
                      same problem size at every N (strong scaling):
        cfg4_tp     MTP fp8 decode, batch 128 x 2 query rows, 128 heads sharded 128 / N per GPU, cache
                    replicated, NCCL all-gather of the outputs (timed with and without the gather)
        cfg4_batch  the same problem sharded by sequence: 128 / N sequences per GPU, all 128 heads
        cfg5        131072-token causal bf16 prefill, queries cut into contiguous chunks of equal work,
                    latent cache replicated, no collective

`value` is TFLOP/s of algorithmic work, 2 * H * (576 + 512) * pairs, pairs = valid (query, position)
slots, with inputs resident in HBM; `e2e` is the same through the host-buffer C-ABI call with pinned host
queries / index lists in and outputs back every step.
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
CFG4 = dict(B=128, s_q=2, H=128, kv_len=65536, topk=2048, page=64)
CFG5_TOKENS = 131072
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
SM_SCALE = 1.0 / math.sqrt(192.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(FALLBACK_PEAKS, source="fallback")


def measured_traffic(batch):
    """DRAM bytes (read + write) of one attention launch of the headline workload, from the ncu capture
    recorded beside its summary (taken at a smaller batch; traffic is proportional to the batch because
    every sequence has its own cache pages).  None when no capture of the current kernel is recorded."""
    path = os.path.join(ROOT, "profiles", "sparse_mla_fp8_decode_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        d = json.load(f)
    return float(d["dram_bytes_per_launch"]) * batch / float(d["batch"])


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
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
            self._thread = None
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
    O.sparse_mla(case["q"], case["kv"], case["indices"], SM_SCALE, kv_is_fp8=True, kv_batch_stride_rows=case["kv_batch_stride_rows"],
                 num_threads=cores)
    return time.perf_counter() - t0, cores, kind


def reference_cpu_prefill(valid_lens, H, kv_rows):
    """The reference's bf16 CPU function (host.cc:508-548) on a sample of prefill queries: every sampled
    query is one 'batch' of its CSR page table with its own list of `valid_lens[i]` rows.  Returns
    (seconds, cores, kind)."""
    import numpy as np
    from oracle import oracle as O
    R = O.ref_lib()
    cores = int(os.environ.get("MLA_DECODE_NUM_THREADS", os.cpu_count() or 1))
    n = len(valid_lens)
    rng = np.random.default_rng(1)
    ip = np.concatenate([[0], np.cumsum(valid_lens)]).astype(np.int32)
    ix = np.concatenate([rng.permutation(kv_rows)[:v] for v in valid_lens]).astype(np.int32)
    if R is not None:
        q = np.zeros((n, H, D_QK), np.uint16)
        kv = np.zeros((kv_rows, D_QK), np.uint16)
        R.ref_rand_bf16(O._p(q), q.size)
        R.ref_rand_bf16(O._p(kv), kv.size)
        out = np.zeros((n, H, D_V), np.uint16); lse = np.zeros((n, H), np.float32)
        t0 = time.perf_counter()
        R.ref_attention_bf16(O._p(q), O._p(kv), O._p(out), O._p(lse), O._p(ip), O._p(ix), n, H, 1)
        return time.perf_counter() - t0, cores, "reference"
    q = rng.integers(0x3c00, 0x4000, size=(n, H, D_QK)).astype(np.uint16)
    kv = rng.integers(0x3c00, 0x4000, size=(kv_rows, D_QK)).astype(np.uint16)
    topk = int(max(valid_lens))
    idx = np.full((n, topk), -1, np.int32)
    for i, v in enumerate(valid_lens):
        idx[i, :v] = ix[ip[i]:ip[i + 1]]
    t0 = time.perf_counter()
    O.sparse_mla(q, kv, idx, SM_SCALE, s_q=n, num_threads=cores)
    return time.perf_counter() - t0, cores, "port"


def cpu_baseline_block(budget_s=15.0):
    H, n_valid = CFG["H"], CFG["topk"] - int(CFG["pad_frac"] * CFG["topk"])
    t1, cores, kind = reference_cpu(1, n_valid, H)
    n = max(1, min(CFG["B"], int(budget_s / max(t1, 1e-3))))
    t, cores, kind = reference_cpu(n, n_valid, H)
    tf = flops_of(n * n_valid, H) / t / 1e12
    return dict(value=tf, unit="TFLOP/s", cores=cores, kind=kind, seconds=round(t, 3),
                sample="%d of %d decode queries x %d heads x %d valid rows, reference fp8 CPU function" % (n, CFG["B"], H, n_valid))


def cpu_baseline_prefill(T, topk, H, budget_s=10.0):
    """A deterministic sample of the prefill's queries (short ones, the tile-boundary ones, then evenly
    spaced ones) through the reference's bf16 CPU function; the rate is per (query-head, position) pair, so
    the whole prefill's CPU time follows by the pair count."""
    import numpy as np
    probe = [min(T, topk)]
    t1, cores, kind = reference_cpu_prefill(probe, H, T)
    n = int(max(4, min(64, budget_s / max(t1, 1e-3))))
    qs = sorted(set([0, 31, 32, 63, 64] + [int(x) for x in np.linspace(0, T - 1, n)]))
    lens = [min(t + 1, topk) for t in qs]
    t, cores, kind = reference_cpu_prefill(lens, H, T)
    pairs = float(sum(lens))
    tf = flops_of(pairs, H) / t / 1e12
    total_pairs = float(np.minimum(np.arange(T) + 1, topk).sum())
    return dict(value=tf, unit="TFLOP/s", cores=cores, kind=kind, seconds=round(t, 3),
                sample="%d of %d prefill queries (%d of %d pairs) x %d heads, reference bf16 CPU function" % (
                    len(qs), T, int(pairs), int(total_pairs), H),
                extrapolated_seconds_whole_prefill=round(t * total_pairs / pairs, 1))


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


# --------------------------------------------------------------------------- timing helper
class Env:
    """What every leg needs: rank facts, the library, and a timed loop that follows the timing rules
    (warm-up, barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks)."""

    def __init__(self, rank, world, local_rank, torch, dist, api, workloads):
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.torch, self.dist, self.api, self.workloads = torch, dist, api, workloads
        self.L = api.lib()
        self.sampler = ClockSampler(local_rank)

    def stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_ms(self, ms):
        t = self.torch.tensor([ms], dtype=self.torch.float64, device="cuda")
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, step, steps, warmup, status_args=None):
        """ms per step, max over ranks."""
        torch = self.torch
        for i in range(max(3, warmup)):
            step(i)
        torch.cuda.synchronize()
        if status_args is not None:
            self.api._check(self.L.dsa_v32_device_status(C.byref(status_args), self.stream()), "device status after warm-up")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        self.sampler.start()
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        self.barrier()
        self.sampler.stop()
        if status_args is not None:
            self.api._check(self.L.dsa_v32_device_status(C.byref(status_args), self.stream()), "device status after the timed region")
        return self.max_ms(e0.elapsed_time(e1)) / steps

    def free(self):
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()


def roofline_block(flops_per_gpu, bytes_per_gpu, ms, pk, kernel, sustained=False):
    """The slower of the two bounds sets the roofline of one GPU's share of a step."""
    peak_tf = pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"]
    t_flop = flops_per_gpu / (peak_tf * 1e12) * 1e6
    t_mem = bytes_per_gpu / (pk["hbm_gbs"] * 1e9) * 1e6
    bound = "tensor" if t_flop >= t_mem else "hbm"
    t_us = ms * 1e3
    if bound == "tensor":
        achieved, peak, unit = flops_per_gpu / (t_us * 1e-6) / 1e12, peak_tf, "TFLOP/s"
    else:
        achieved, peak, unit = bytes_per_gpu / (t_us * 1e-6) / 1e9, pk["hbm_gbs"], "GB/s"
    return dict(bound=bound, achieved=achieved, peak=peak, unit=unit, frac=achieved / peak, traffic=None,
                peak_source=pk["source"] + (" (sustained)" if sustained else " (burst)"), kernel=kernel,
                t_flop_us=t_flop, t_mem_us=t_mem, flops_per_gpu=flops_per_gpu, gathered_bytes_per_gpu=bytes_per_gpu)


# --------------------------------------------------------------------------- prefill (config 3 / config 5)
def prefill_leg(env, T, steps, warmup, label):
    """bf16 causal prefill of one T-token sequence, 128 heads, top-k 2048; a step = the whole prefill.  With
    N > 1 ranks the query tokens are cut into contiguous chunks of equal work, the latent cache is replicated
    and nothing is exchanged (strong scaling of one sequence)."""
    import numpy as np
    from opfoundry_b200 import shard
    torch, api = env.torch, env.api
    H, topk = CFG["H"], CFG["topk"]
    valid_all = np.minimum(np.arange(T) + 1, topk)
    bounds = shard.shard_queries_equal_work(valid_all, env.world)
    q0, q1 = bounds[env.rank], bounds[env.rank + 1]
    W = env.workloads.prefill_bf16(T=T, H=H, topk=topk, seed=2026, q_begin=q0, q_end=q1)
    nq = q1 - q0
    plan = api.mla_decode_plan_create(nq, H, topk, nq, valid_len_hint=W["valid_len"])
    out = torch.empty(nq, H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(nq, H, dtype=torch.float32, device="cuda")
    a = api.make_args(W["q"], W["kv"], W["indices"], plan, SM_SCALE, out=out, lse=lse)

    def step(i):
        api._check(env.L.dsa_v32_decode_pipeline(C.byref(a), 0, env.stream()), "prefill")

    ms = env.timed(step, steps, warmup, a)
    total_pairs = float(valid_all.sum())
    local_pairs = float(valid_all[q0:q1].sum())
    pk = peaks()
    flops = flops_of(total_pairs, H)
    tf = flops / (ms * 1e-3) / 1e12
    # the whole job's rate against N GPUs' tensor peak; a long prefill runs under the power cap, so the
    # sustained peak is given beside the burst one
    block = dict(workload="%s_prefill_bf16_t%d_h128_topk2048_causal" % (label, T), tokens=T, heads=H, topk=topk, n_gpus=env.world,
                 ms_per_step=ms, tflops=tf, steps=steps, pairs=total_pairs, pairs_rank0=local_pairs,
                 sharding="contiguous query chunks of equal work, latent cache replicated, no exchange",
                 l2="gathered rows per step %.1f GB from a %.1f MB cache (the cache is L2-resident by construction of the config)" % (
                     total_pairs * 1152 / 1e9, T * 1152 / 1e6),
                 roofline=dict(bound="tensor", achieved=tf, peak=env.world * pk["bf16_tflops"], unit="TFLOP/s",
                               frac=tf / (env.world * pk["bf16_tflops"]),
                               frac_of_sustained=tf / (env.world * pk["bf16_tflops_sustained"]), traffic=None,
                               peak_source=pk["source"], kernel="sparse_mla_kernel<bf16>", flops_per_step=flops,
                               gathered_bytes_per_step=total_pairs * 1152.0,
                               t_flop_us=flops / env.world / (pk["bf16_tflops"] * 1e12) * 1e6),
                 gpu_launches=steps * (2 if plan.info.num_partials > 0 else 1), clocks=env.sampler.summary())
    del W, plan, out, lse, a
    env.free()
    return block


# --------------------------------------------------------------------------- config 4 (MTP fp8 decode)
def cfg4_problem(env, seq_begin, seq_end, n_batches=2):
    """Sequences [seq_begin, seq_end) of the config-4 problem: paged fp8 cache of those sequences, and for
    each of `n_batches` steps the queries [seqs * 2, 128, 576] and their index lists (the two rows of a
    sequence share one list for the sequences a seeded coin picks)."""
    torch = env.torch
    c = CFG4
    n = seq_end - seq_begin
    W = env.workloads.decode_fp8(B=n, H=c["H"], kv_len=c["kv_len"], topk=c["topk"], page=c["page"], pad_frac=0.0,
                                 n_batches=n_batches, seed=4000 + seq_begin, s_q=c["s_q"])
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    share = (torch.rand(c["B"], generator=g, device="cuda") < 0.5)[seq_begin:seq_end]
    steps = []
    for q, idx in W["steps"]:
        idx = idx.clone().view(n, c["s_q"], c["topk"])
        idx[share, 1] = idx[share, 0]
        steps.append((q, idx.view(n * c["s_q"], c["topk"]).contiguous()))
    W["steps"] = steps
    W["share_frac"] = float(share.float().mean().item()) if n else 0.0
    W["mtp_shared"] = [bool(x) for x in share.cpu().tolist()]
    return W


def fused_gather_leg(env, mode, W, plan, step_in, out, lse, gathered, attn_gather, steps, warmup, status_args, s0, h0, total_q):
    """The config-4 step with the gather fused into the kernels: finished rows are stored straight into every
    peer's gathered buffer (peer-mapped pointers, plain stores), then one flag round.  Returns (ms per step,
    whether one more step of it equals attention + NCCL all-gather bit for bit on every rank)."""
    from opfoundry_b200 import shard
    torch, api, dist = env.torch, env.api, env.dist
    c = CFG4
    pg = shard.PeerGather(c["B"] * c["s_q"], c["H"])
    try:
        row0 = s0 * c["s_q"]
        fused_args = []
        for q, idx in step_in:
            a = api.make_args(q, W["cache"], idx, plan, SM_SCALE, out=out, lse=lse, block_table=W["block_table"], page_block_size=c["page"])
            a.stride_o_row, a.stride_o_head = pg.out.stride(0), pg.out.stride(1)
            fused_args.append(a)

        def fused(i):
            po = pg.targets(row0, h0)
            api._check(env.L.dsa_v32_decode_pipeline_allgather(C.byref(fused_args[i % len(fused_args)]), C.byref(po), env.stream()),
                       "fused decode step")

        ms_fused = env.timed(fused, steps, warmup, status_args)
        # same numbers as the NCCL path: one more step of each on the same inputs
        attn_gather(0)
        fused(0)
        torch.cuda.synchronize()
        dist.barrier()
        if mode == "tp":
            ref = gathered.permute(1, 0, 2, 3).reshape(total_q, c["H"], D_V)          # [rank, q, heads, d] -> [q, H, d]
        else:
            ref = gathered.reshape(c["B"] * c["s_q"], c["H"], D_V)
        same = bool(torch.equal(ref.view(torch.int16), pg.out.view(torch.int16)))
        t = torch.tensor([1.0 if same else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return ms_fused, bool(t.item() > 0.5)
    finally:
        torch.cuda.synchronize()
        pg.close()


def cfg4_leg(env, mode, steps, warmup):
    """mode "tp": every rank attends all 128 x 2 query rows with its 128 / N heads over the replicated cache;
    mode "batch": every rank attends its 128 / N sequences with all 128 heads over its own sequences' cache.
    Both end with the all-gather of the bf16 outputs (the only exchange the path has): the step is timed
    without it, with the gather fused into the kernels (peer stores + flags; the block's `ms_per_step`) and
    with an NCCL all-gather after the kernels (the cross-check; both must give the same bytes)."""
    from opfoundry_b200 import shard
    torch, api, dist = env.torch, env.api, env.dist
    c = CFG4
    world, rank = env.world, env.rank
    if mode == "tp":
        h0, h1 = shard.shard_heads(c["H"], world, rank)
        s0, s1 = 0, c["B"]
    else:
        h0, h1 = 0, c["H"]
        s0, s1 = shard.shard_batch(c["B"], world, rank)
    Hl, nseq = h1 - h0, s1 - s0
    W = cfg4_problem(env, s0, s1)
    total_q = nseq * c["s_q"]
    step_in = [(q[:, h0:h1].contiguous(), idx) for q, idx in W["steps"]]
    # rows of a sequence that share a list are gathered once when both fit one 128-row tile (128 / N heads <= 64)
    plan = api.mla_decode_plan_create(total_q, Hl, c["topk"], c["s_q"], mtp_shared=W["mtp_shared"])
    out = torch.empty(total_q, Hl, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(total_q, Hl, dtype=torch.float32, device="cuda")
    gathered = torch.empty(world, total_q, Hl, D_V, dtype=torch.bfloat16, device="cuda") if world > 1 else None
    arg_sets = [api.make_args(q, W["cache"], idx, plan, SM_SCALE, out=out, lse=lse, block_table=W["block_table"],
                              page_block_size=c["page"]) for q, idx in step_in]

    def attn(i):
        api._check(env.L.dsa_v32_decode_pipeline(C.byref(arg_sets[i % len(arg_sets)]), 0, env.stream()), "decode step")

    def attn_gather(i):
        attn(i)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)   # rank-major: block r = rank r's heads (tp) or sequences (batch)

    ms_attn = env.timed(attn, steps, warmup, arg_sets[0])
    ms_full = env.timed(attn_gather, steps, warmup, arg_sets[0]) if world > 1 else ms_attn
    # the same step with the gather fused into the kernels: finished rows are stored straight into every
    # peer's gathered buffer (peer-mapped pointers, plain stores), then one flag round
    ms_fused, fused_ok, fused_note = None, None, None
    if world > 1:
        try:
            ms_fused, fused_ok = fused_gather_leg(env, mode, W, plan, step_in, out, lse, gathered, attn_gather, steps, warmup,
                                                  arg_sets[0], s0, h0, total_q)
        except Exception as ex:          # the NCCL number stands on its own; say why the fused one is missing
            ms_fused, fused_ok, fused_note = None, False, "%s: %s" % (type(ex).__name__, ex)
        ok = torch.tensor([0.0 if ms_fused is None else 1.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() < 0.5:
            ms_fused = None
    clocks = env.sampler.summary()
    pk = peaks()
    ms_step = ms_fused if ms_fused is not None else ms_full
    pairs_total = float(c["B"] * c["s_q"] * c["topk"])
    flops_total = flops_of(pairs_total, c["H"])
    # per GPU: tp keeps every GPU's gathered bytes and divides the flops; batch divides both
    pairs_gpu = float(total_q * c["topk"])
    roof = roofline_block(flops_of(pairs_gpu, Hl), pairs_gpu * 656.0, ms_attn, pk, "sparse_mla_kernel<fp8>")
    block = dict(workload="cfg4_%s_decode_fp8_mtp_b%d_sq2_h128_topk2048_kv65536_paged64" % (mode, c["B"]), n_gpus=world,
                 heads_per_gpu=Hl, sequences_per_gpu=nseq, shared_list_fraction=W["share_frac"],
                 ms_per_step=ms_step, ms_per_step_without_gather=ms_attn, ms_per_step_nccl_gather=ms_full,
                 ms_per_step_fused_gather=ms_fused, nccl_all_gather_ms=ms_full - ms_attn, fused_equals_nccl=fused_ok,
                 fused_gather_note=fused_note,
                 gather="stores into the peers' gathered buffers from the attention kernels + one flag round (the NCCL all-gather "
                        "is timed beside it as the cross-check)" if world > 1 else "none (one GPU)",
                 all_gather_bytes_per_gpu=(out.numel() * 2 if world > 1 else 0),
                 tflops=flops_total / (ms_step * 1e-3) / 1e12, tflops_without_gather=flops_total / (ms_attn * 1e-3) / 1e12,
                 tflops_nccl_gather=flops_total / (ms_full * 1e-3) / 1e12,
                 steps=steps, pairs=pairs_total, roofline=roof,
                 sharding=("heads sharded %d per GPU, latent cache replicated" % Hl if mode == "tp" else
                           "sequences sharded %d per GPU with their cache, all 128 heads" % nseq) + ", one NCCL all-gather of the outputs per step",
                 l2="every step gathers %.0f MB of rows per GPU > 126 MB L2" % (pairs_gpu * 656 / 1e6),
                 gpu_launches=steps * (2 if plan.info.num_partials > 0 else 1), clocks=clocks)
    del W, plan, out, lse, gathered, arg_sets, step_in
    env.free()
    return block


# --------------------------------------------------------------------------- host-buffer leg of the headline
def e2e_leg(env, W, out, lse, K, num_chunks, num_lanes=1):
    """K steps through the host-buffer C-ABI call: pinned host q / index lists in, out / lse back, the caller
    synchronising on every step's result.  num_chunks > 1: the call that cuts the batch into groups of
    sequences whose PCIe copies overlap the other groups' kernels (its plan is for one group's shape);
    num_lanes > 1: that many groups' kernels side by side, each on its share of the SMs."""
    api, torch = env.api, env.torch
    B, H = W["B"], W["H"]
    hint = [W["n_valid"]] * (B // num_chunks)
    plan = api.mla_decode_plan_create(B // num_chunks, H, W["topk"], 1, valid_len_hint=hint)
    lane_plans = None
    if num_lanes > 1:
        sms = torch.cuda.get_device_properties(0).multi_processor_count // num_lanes // 2 * 2
        lane_plans = [api.mla_decode_plan_create(B // num_chunks, H, W["topk"], 1, valid_len_hint=hint, num_sms=sms)
                      for _ in range(num_lanes)]
    q_host = [q.cpu().pin_memory() for (q, _) in W["steps"]]
    i_host = [idx.cpu().pin_memory() for (_, idx) in W["steps"]]
    out_host = torch.empty(B, H, D_V, dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty(B, H, dtype=torch.float32).pin_memory()
    q_dev = torch.empty_like(W["steps"][0][0])
    i_dev = torch.empty_like(W["steps"][0][1])
    a_e2e = api.make_args(q_dev, W["cache"], i_dev, plan, SM_SCALE, out=out, lse=lse, block_table=W["block_table"],
                          page_block_size=W["page"])
    for i in range(3):
        api.mla_decode_step_host(a_e2e, q_host[i % len(q_host)], i_host[i % len(i_host)], out_host, lse_host, num_chunks,
                                 lane_plans=lane_plans)
    torch.cuda.synchronize()
    api._check(env.L.dsa_v32_device_status(C.byref(a_e2e), env.stream()), "device status (host-buffer leg)")
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    g0.record()
    for i in range(K):
        api.mla_decode_step_host(a_e2e, q_host[i % len(q_host)], i_host[i % len(i_host)], out_host, lse_host, num_chunks,
                                 lane_plans=lane_plans)
        torch.cuda.current_stream().synchronize()   # the caller reads the step's result before the next step
    g1.record()
    env.barrier()
    h2d = q_host[0].numel() * 2 + i_host[0].numel() * 4
    d2h = out_host.numel() * 2 + lse_host.numel() * 4
    return g0.elapsed_time(g1), h2d, d2h


# --------------------------------------------------------------------------- headline (config 2)
def headline_leg(env, args):
    torch, api = env.torch, env.api
    W = env.workloads.decode_fp8(B=CFG["B"], H=CFG["H"], kv_len=CFG["kv_len"], topk=CFG["topk"], page=CFG["page"],
                                 pad_frac=CFG["pad_frac"], n_batches=CFG["n_batches"], seed=2026 + env.rank)
    B, H, topk, n_valid = W["B"], W["H"], W["topk"], W["n_valid"]
    pairs = B * n_valid
    step_flops = flops_of(pairs, H)
    plan = api.mla_decode_plan_create(B, H, topk, 1, valid_len_hint=[n_valid] * B)
    out = torch.empty(B, H, D_V, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
    arg_sets = [api.make_args(q, W["cache"], idx, plan, SM_SCALE, out=out, lse=lse, block_table=W["block_table"],
                              page_block_size=W["page"]) for (q, idx) in W["steps"]]
    L = env.L

    def step(i):
        a = arg_sets[i % len(arg_sets)]
        rc = L.dsa_v32_decode_fp8(C.byref(a), env.stream())
        if rc == 0:
            rc = L.dsa_v32_combine(C.byref(a), env.stream())
        if rc:
            raise api.DsaError(rc, "decode step")

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    api._check(L.dsa_v32_device_status(C.byref(arg_sets[0]), env.stream()), "device status after warm-up")

    K = args.steps
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = env.stream()
    env.barrier()
    env.sampler.start()
    # the timed region: K steps of the pipeline call a user makes (attention + merge, launched back to back)
    e0.record()
    for i in range(K):
        rc = L.dsa_v32_decode_pipeline(C.byref(arg_sets[i % len(arg_sets)]), 0, stream)
        if rc:
            raise api.DsaError(rc, "decode step")
    e1.record()
    env.barrier()
    # the same K steps once more with an event pair around every attention launch: the kernel's own duration
    # for the roofline (events between the launches keep the merge kernel from overlapping the attention
    # kernel's tail, so this pass is a little slower than the timed one and is not the reported step time)
    for i in range(K):
        a = arg_sets[i % len(arg_sets)]
        ev_a[i].record()
        rc = L.dsa_v32_decode_fp8(C.byref(a), stream)
        ev_b[i].record()
        rc = rc or L.dsa_v32_combine(C.byref(a), stream)
        if rc:
            raise api.DsaError(rc, "decode step")
    env.barrier()
    env.sampler.stop()
    total_ms = e0.elapsed_time(e1)
    attn_ms = sum(a.elapsed_time(b) for a, b in zip(ev_a, ev_b)) / K
    api._check(L.dsa_v32_device_status(C.byref(arg_sets[0]), env.stream()), "device status after the timed region")
    clocks = env.sampler.summary()

    e2e_ms, e2e1_ms, h2d, d2h = float("nan"), float("nan"), 0, 0
    e2e_chunks = 4 if B % 4 == 0 and B >= 16 else 1
    e2e_lanes = 1
    if not args.no_e2e:
        e2e1_ms, h2d, d2h = e2e_leg(env, W, out, lse, K, 1)
        e2e_ms = e2e_leg(env, W, out, lse, K, e2e_chunks)[0] if e2e_chunks > 1 else e2e1_ms
        if e2e_chunks > 1:   # two groups' kernels side by side on half the SMs each; the faster form is reported
            e2e2_ms = e2e_leg(env, W, out, lse, K, e2e_chunks, 2)[0]
            if e2e2_ms < e2e_ms:
                e2e_ms, e2e_lanes = e2e2_ms, 2

    t = torch.tensor([total_ms, attn_ms, e2e_ms, e2e1_ms], dtype=torch.float64, device="cuda")
    if env.world > 1:
        env.dist.all_reduce(t, op=env.dist.ReduceOp.MAX)
    total_ms, attn_ms, e2e_ms, e2e1_ms = (float(x) for x in t.tolist())
    world = env.world
    pk = peaks()
    ms_per_step = total_ms / K
    value = world * step_flops / (ms_per_step * 1e-3) / 1e12
    # The attention kernel's duration: the event pairs of the second pass keep the next launch's set-up from
    # overlapping the kernel before it, so a launch there takes longer than a whole step of the timed region;
    # the step time (attention + merge when the plan splits items) is then the tighter upper bound of the two.
    attn_events_ms = attn_ms
    attn_ms = min(attn_ms, ms_per_step)
    attn_tf = step_flops / (attn_ms * 1e-3) / 1e12
    gathered = pairs * 656.0
    line = dict(metric="sparse_mla_decode_fp8_tflops", value=value, unit="TFLOP/s", n_gpus=world, steps=K,
                warmup=args.warmup, ms_per_step=ms_per_step, us_per_step=ms_per_step * 1e3, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="bf16 MMA, fp32 accumulate (fp8 e4m3 cache)", data="synthetic",
                config=workload_config(),
                roofline=dict(bound="tensor", achieved=attn_tf, peak=pk["bf16_tflops"], unit="TFLOP/s",
                              frac=attn_tf / pk["bf16_tflops"], traffic=measured_traffic(B),
                              peak_source=pk["source"], kernel="sparse_mla_kernel<fp8>", kernel_us=attn_ms * 1e3,
                              kernel_us_between_events=attn_events_ms * 1e3,
                              flops_per_launch=step_flops, gathered_bytes_per_launch=gathered,
                              gathered_gbs=gathered / (attn_ms * 1e-3) / 1e9, hbm_peak_gbs=pk["hbm_gbs"],
                              t_flop_us=step_flops / (pk["bf16_tflops"] * 1e12) * 1e6,
                              t_mem_us=gathered / (pk["hbm_gbs"] * 1e9) * 1e6),
                e2e=None if args.no_e2e else dict(value=world * step_flops / (e2e_ms / K * 1e-3) / 1e12, unit="TFLOP/s",
                                                  ms_per_step=e2e_ms / K, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                                                  call=("dsa_v32_decode_pipeline_host_chunked, %d groups of sequences "
                                                        "(copies overlap the other groups' kernels)" % e2e_chunks)
                                                  if e2e_lanes == 1 else
                                                  ("dsa_v32_decode_pipeline_host_lanes, %d groups of sequences, the kernels "
                                                   "of %d groups side by side" % (e2e_chunks, e2e_lanes)),
                                                  ms_per_step_unchunked=e2e1_ms / K),
                gpu_launches=K * (2 if plan.info.num_partials > 0 else 1), clocks=clocks)
    del W, plan, out, lse, arg_sets
    env.free()
    return line


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the `prefill` block")
    ap.add_argument("--no-sharded", action="store_true", help="skip the `sharded` block")
    ap.add_argument("--batch", type=int, default=CFG["B"], help="sequences per GPU (smaller only for profiler captures)")
    ap.add_argument("--workload", default="all", choices=["all", "decode_fp8", "prefill_bf16", "decode_fp8_tp", "decode_fp8_batch"],
                    help="all: the headline with the prefill and sharded blocks; the others run one leg alone and print "
                         "its block (profiler captures, quick checks)")
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
        import datetime
        # a short collective timeout: a rank that fails must not hold the others for the default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=90))
    if not os.path.exists(api.LIB_PATH):
        if rank == 0:
            build.build()
        if world > 1:
            dist.barrier()
    api.lib()
    env = Env(rank, world, local_rank, torch, dist, api, workloads)
    short = max(5, min(args.steps, 20))

    if args.workload == "prefill_bf16":
        block = prefill_leg(env, args.tokens, args.steps, args.warmup, "single")
        if rank == 0:
            print(json.dumps(dict(metric="sparse_mla_prefill_bf16_tflops", value=block["tflops"], unit="TFLOP/s", n_gpus=world,
                                  steps=args.steps, warmup=args.warmup, ms_per_step=block["ms_per_step"], higher_is_better=True,
                                  scaling="strong", vs_baseline=None, dtype="bf16 MMA, fp32 accumulate", data="synthetic",
                                  config=dict(workload=block["workload"]), roofline=block["roofline"],
                                  gpu_launches=block["gpu_launches"], clocks=block["clocks"])), flush=True)
    elif args.workload in ("decode_fp8_tp", "decode_fp8_batch"):
        block = cfg4_leg(env, "tp" if args.workload == "decode_fp8_tp" else "batch", short, args.warmup)
        if rank == 0:
            print(json.dumps(dict(metric="sparse_mla_decode_fp8_mtp_tflops", value=block["tflops"], unit="TFLOP/s", n_gpus=world,
                                  steps=short, warmup=args.warmup, ms_per_step=block["ms_per_step"], higher_is_better=True,
                                  scaling="strong", vs_baseline=None, dtype="bf16 MMA, fp32 accumulate (fp8 e4m3 cache)",
                                  data="synthetic", config=dict(workload=block["workload"]), block=block,
                                  gpu_launches=block["gpu_launches"], clocks=block["clocks"])), flush=True)
    else:
        line = headline_leg(env, args)
        if args.workload == "all":
            if world == 1 and not args.no_prefill:
                # a short burst (15 launches, 35 ms): the kernel timed alone, against the burst peak; hundreds of
                # launches in a row run under the power cap (--workload prefill_bf16 --steps 200 shows that figure)
                pre = prefill_leg(env, 4096, min(short, 10), min(args.warmup, 5), "cfg3")
                if not args.no_cpu_baseline:
                    pre["cpu_baseline"] = cpu_baseline_prefill(4096, CFG["topk"], CFG["H"])
                line["prefill"] = pre
            if not args.no_sharded:
                sharded = dict(note="strong scaling: the same total problem at every N; ms are device-timed, max over ranks")
                sharded["cfg4_tp"] = cfg4_leg(env, "tp", short, args.warmup)
                sharded["cfg4_batch"] = cfg4_leg(env, "batch", short, args.warmup)
                sharded["cfg5"] = prefill_leg(env, CFG5_TOKENS, 3, 3, "cfg5")
                line["sharded"] = sharded
        if rank == 0:
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline_block()
            print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
