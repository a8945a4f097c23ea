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


class PeerGather:
    """The gathered output of a sharded decode step, written by the attention kernels themselves.

    Every rank owns a full [total_q, H_all, 512] bf16 buffer (+ lse [total_q, H_all] and eight arrival
    flags) and maps every peer's through CUDA IPC (plain peer mappings; no multicast object).  `targets`
    builds the argument of dsa_v32_decode_pipeline_allgather for this rank's slice - rows [row0, ...) and
    heads [head0, ...) of the full layout - so the kernels store finished rows into all buffers directly
    and the NCCL all-gather after the step disappears.
    """

    def __init__(self, total_q, H_all, device="cuda"):
        from . import api
        self.api = api
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if self.world > api.MAX_PEERS:
            raise ValueError("at most %d peers" % api.MAX_PEERS)
        self.total_q, self.H_all = total_q, H_all
        self.out = torch.zeros(total_q, H_all, 512, dtype=torch.bfloat16, device=device)
        self.lse = torch.zeros(total_q, H_all, dtype=torch.float32, device=device)
        self.flags = torch.zeros(api.MAX_PEERS, dtype=torch.int32, device=device)
        self.step = 0
        torch.cuda.synchronize()
        # export: (64-byte handle of the allocation, byte offset of the tensor inside it); the tensors keep it alive
        import ctypes as C
        mine = []
        for t in (self.out, self.lse, self.flags):
            hb = C.create_string_buffer(64)
            off = C.c_int64(0)
            api._check(api.lib().dsa_v32_ipc_export(t.data_ptr(), hb, C.byref(off)), "dsa_v32_ipc_export")
            mine.append((hb.raw, int(off.value)))
        everyone = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(everyone, mine)
        else:
            everyone[0] = mine
        # import: every distinct allocation is opened once, for THIS device (peer access is enabled by the open)
        self._opened = {}
        self.ptrs = []          # per peer: (out, lse, flags) device addresses usable from this GPU
        for r in range(self.world):
            if r == self.rank:
                self.ptrs.append((self.out.data_ptr(), self.lse.data_ptr(), self.flags.data_ptr()))
                continue
            addrs = []
            for handle, offset in everyone[r]:
                if handle not in self._opened:
                    base = C.c_void_p()
                    api._check(api.lib().dsa_v32_ipc_open(handle, C.byref(base)), "dsa_v32_ipc_open")
                    self._opened[handle] = base.value
                addrs.append(self._opened[handle] + offset)
            self.ptrs.append(tuple(addrs))
        if self.world > 1:
            dist.barrier()      # nobody stores into a peer before every mapping exists

    def close(self):
        """Unmaps the peers' buffers (call on every rank, after a barrier, before the buffers are freed)."""
        for base in self._opened.values():
            self.api.lib().dsa_v32_ipc_close(base)
        self._opened = {}

    def targets(self, row0, head0):
        """PeerOutputs for the next step of this rank's slice starting at (row0, head0) of the full layout.
        The matching strides for the attention arguments are out.stride(0), out.stride(1)."""
        po = self.api.PeerOutputs()
        po.num_peers, po.my_rank = self.world, self.rank
        o_off = (row0 * self.out.stride(0) + head0 * self.out.stride(1)) * 2
        l_off = (row0 * self.H_all + head0) * 4
        for r, (o, l, f) in enumerate(self.ptrs):
            po.out[r], po.lse[r], po.flags[r] = o + o_off, l + l_off, f
        po.lse_stride_row = self.H_all
        self.step += 1
        po.step = self.step
        return po
