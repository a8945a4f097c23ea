"""How the path is partitioned across the GPUs of one box (one process per GPU, torch.distributed).

The path shards only where it does so naturally:
  * decode by sequence (batch): every rank owns whole sequences and their cache; no exchange at all.
  * decode by heads (the TP layout of the 8-GPU decode configuration): rank r owns heads
    [r*H/world, (r+1)*H/world) of every query; cache, block table and index lists are replicated
    (one shared latent KV head: there is nothing to shard on the KV side); outputs are all-gathered.
  * long prefill by query chunks: contiguous ranges of query tokens with equal numbers of valid
    (query, position) pairs, latent cache replicated, no exchange.
Timing of any multi-GPU number is the maximum over ranks of a device-side duration.
"""
import numpy as np
import torch
import torch.distributed as dist


def shard_batch(num_seqs, world, rank):
    """Contiguous block of sequences for `rank`; sizes differ by at most one."""
    base, extra = divmod(num_seqs, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_heads(H, world, rank):
    if H % world != 0:
        raise ValueError("heads (%d) must divide evenly over %d ranks" % (H, world))
    per = H // world
    return rank * per, (rank + 1) * per


def shard_queries_equal_work(valid_len, world):
    """Cut query rows [0, n) into `world` contiguous ranges holding equal shares of sum(valid_len)
    (the first queries of a causal prefill have fewer valid positions).  Returns world+1 bounds."""
    v = np.asarray(valid_len, dtype=np.int64)
    csum = np.concatenate([[0], np.cumsum(v)])
    total = csum[-1]
    bounds = [0]
    for r in range(1, world):
        target = total * r / world
        bounds.append(int(np.searchsorted(csum, target, side="left")))
    bounds.append(len(v))
    for i in range(1, len(bounds)):           # keep the bounds monotone for degenerate inputs
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


def max_over_ranks(values, device):
    """Element-wise maximum over all ranks of a list of floats (identity without a process group)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


def all_gather_heads(local_out, world):
    """[rows, H/world, D] per rank -> [rows, H, D] on every rank (heads are the middle dimension, so
    the gathered blocks are interleaved back into place)."""
    if world == 1:
        return local_out
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous())
    return torch.cat(parts, dim=1)
