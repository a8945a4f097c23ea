"""Full-size synthetic workloads, generated on the device (the host generators in synth.py are
for small parity cases).  Shapes and value distributions follow the benchmark configurations:

  decode_fp8   batch 64, 128 heads, kv_len 32768 per sequence in a paged fp8 cache of 64-token
               blocks with a randomly permuted block table, top-k 2048 unique positions per query
               with the last 5 % of slots -1, Q ~ N(0,1) bf16, latent ~ N(0,1) quantised per 128
               values (scale = amax / 448), rope ~ N(0,1) bf16
  prefill_bf16 one sequence of T tokens, 128 heads, causal top-k 2048 (query t draws from [0, t];
               fewer than 2048 positions -> all of them, rest -1), bf16 cache
"""
import torch

from . import api

D_QK, D_V, D_ROPE = 576, 512, 64


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_fp8_cache(num_rows, seed, device="cuda", chunk=1 << 18):
    """[num_rows, 656] uint8 cache rows from N(0,1) latent / rope values, packed by the library's
    cache-write kernel."""
    g = _gen(seed, device)
    cache = torch.empty(num_rows, api.FP8_ROW_BYTES, dtype=torch.uint8, device=device)
    for r0 in range(0, num_rows, chunk):
        n = min(chunk, num_rows - r0)
        latent = torch.randn(n, D_V, generator=g, device=device, dtype=torch.float32)
        rope = torch.randn(n, D_ROPE, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        api.pack_fp8_rows(latent, rope, out=cache[r0:r0 + n])
    return cache


def unique_topk(batch, kv_len, topk, g, device):
    """[batch, topk] int32: distinct uniform positions in random order (argsort of uniform keys)."""
    keys = torch.rand(batch, kv_len, generator=g, device=device)
    return keys.argsort(dim=1)[:, :topk].to(torch.int32).contiguous()


def decode_fp8(B=64, H=128, kv_len=32768, topk=2048, page=64, pad_frac=0.05, n_batches=4, seed=2026, device="cuda",
               s_q=1):
    """Returns a dict: cache, block_table, and `n_batches` different (q, indices) steps so successive
    timed steps gather different rows (together more than the L2 holds)."""
    blocks_per_seq = kv_len // page
    n_rows = B * kv_len
    cache = make_fp8_cache(n_rows, seed, device)
    g = _gen(seed + 1, device)
    block_table = torch.randperm(B * blocks_per_seq, generator=g, device=device).to(torch.int32).view(B, blocks_per_seq)
    n_pad = int(pad_frac * topk)
    steps = []
    for _ in range(n_batches):
        q = torch.randn(B * s_q, H, D_QK, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        idx = unique_topk(B * s_q, kv_len, topk, g, device)
        if n_pad:
            idx[:, topk - n_pad:] = -1
        steps.append((q, idx))
    return dict(cache=cache, block_table=block_table.contiguous(), steps=steps, B=B, H=H, kv_len=kv_len, topk=topk,
                page=page, n_valid=topk - n_pad, s_q=s_q)


def prefill_bf16(T=4096, H=128, topk=2048, seed=2026, device="cuda", q_begin=0, q_end=None, block=1024):
    """Causal prefill of queries [q_begin, q_end) of a T-token sequence (the whole cache is built).
    Queries and index lists are drawn per block of `block` absolute query positions from a generator
    seeded by (seed, block number), so any query range is a slice of the same T-token problem."""
    q_end = T if q_end is None else q_end
    kv = torch.randn(T, D_QK, generator=_gen(seed, device), device=device, dtype=torch.float32).to(torch.bfloat16)
    nq = q_end - q_begin
    q = torch.empty(nq, H, D_QK, dtype=torch.bfloat16, device=device)
    idx = torch.full((nq, topk), -1, dtype=torch.int32, device=device)
    for b in range(q_begin // block, (q_end + block - 1) // block):
        g = _gen(seed * 1000003 + 17 * b + 1, device)
        t0, t1 = b * block, min(T, (b + 1) * block)
        qb = torch.randn(t1 - t0, H, D_QK, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        tt = torch.arange(t0, t1, device=device)
        width = t1
        keys = torch.rand(t1 - t0, width, generator=g, device=device)
        keys[torch.arange(width, device=device)[None, :] > tt[:, None]] = 2.0  # positions after t sort last
        k = min(topk, width)
        order = keys.topk(k, dim=1, largest=False).indices.to(torch.int32)
        del keys
        valid = torch.arange(k, device=device)[None, :] <= tt[:, None]
        ib = torch.full((t1 - t0, topk), -1, dtype=torch.int32, device=device)
        ib[:, :k] = torch.where(valid, order, torch.full_like(order, -1))
        lo, hi = max(t0, q_begin), min(t1, q_end)
        q[lo - q_begin:hi - q_begin] = qb[lo - t0:hi - t0]
        idx[lo - q_begin:hi - q_begin] = ib[lo - t0:hi - t0]
    t = torch.arange(q_begin, q_end, device=device)
    valid_len = torch.minimum(t + 1, torch.tensor(topk, device=device)).to(torch.int32)
    return dict(q=q, kv=kv, indices=idx.contiguous(), valid_len=valid_len.cpu().numpy(), T=T, H=H, topk=topk,
                n_pairs=int(valid_len.sum().item()))
