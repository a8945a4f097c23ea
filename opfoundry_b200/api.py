"""Host-side mirror of the reference lab's launcher interface, bound to libdsa_v32.so over its C ABI.

Names follow opus_attn/dsa_v32/common/host.cc: `mla_decode_plan_create` (:151-178) sizes and fills
the split workspace, `mla_decode_launch_pipeline` (:114-138) runs metadata (optional) -> decode ->
reduce on one stream.  torch is used only to own device memory and to name the stream; all work
happens in the CUDA library, and importing this module without the built library raises.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdsa_v32.so")

D_QK, D_V, D_ROPE = 576, 512, 64
BF16_ROW_BYTES, FP8_ROW_BYTES = 1152, 656
KV_BF16, KV_FP8 = 0, 1
ERR_DEVICE_WAIT = 1001
ERR_SCRATCH_TOO_SMALL = -7
STATIC_SCRATCH_BYTES = 48 << 20


class WorkInfo(C.Structure):
    _fields_ = [("q_row", C.c_int32), ("partial_slot", C.c_int32), ("k_begin", C.c_int32), ("k_end", C.c_int32),
                ("head_block", C.c_int32), ("reduce_row", C.c_int32), ("stacked_rows", C.c_int32), ("_pad", C.c_int32)]


class Shape(C.Structure):
    _fields_ = [("total_q", C.c_int32), ("H", C.c_int32), ("topk", C.c_int32), ("s_q", C.c_int32),
                ("num_sms", C.c_int32), ("flags", C.c_int32), ("valid_len_hint", C.c_void_p), ("mtp_shared", C.c_void_p)]


class PlanInfo(C.Structure):
    _fields_ = [("workspace_bytes", C.c_int64), ("num_lists", C.c_int32), ("num_works", C.c_int32),
                ("num_partials", C.c_int32), ("num_reduce_rows", C.c_int32)]


MAX_PEERS = 8


class PeerOutputs(C.Structure):
    _fields_ = [("num_peers", C.c_int32), ("my_rank", C.c_int32), ("out", C.c_void_p * MAX_PEERS), ("lse", C.c_void_p * MAX_PEERS),
                ("flags", C.c_void_p * MAX_PEERS), ("lse_stride_row", C.c_int64), ("step", C.c_uint32), ("_pad", C.c_uint32)]


class V4Ext(C.Structure):
    _fields_ = [("attn_sink", C.c_void_p), ("kv2", C.c_void_p), ("pool_split", C.c_void_p), ("num_kv2_rows", C.c_int64)]


class AttnArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("kv", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
                ("indices", C.c_void_p), ("block_table", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_int64), ("num_kv_rows", C.c_int64), ("kv_batch_stride_rows", C.c_int64),
                ("stride_q_row", C.c_int64), ("stride_q_head", C.c_int64), ("stride_o_row", C.c_int64),
                ("stride_o_head", C.c_int64), ("total_q", C.c_int32), ("H", C.c_int32), ("topk", C.c_int32),
                ("s_q", C.c_int32), ("block_table_stride", C.c_int32), ("page_block_size", C.c_int32),
                ("kv_dtype", C.c_int32), ("sm_scale", C.c_float)]


class HostIO(C.Structure):
    _fields_ = [("q_host", C.c_void_p), ("indices_host", C.c_void_p), ("out_host", C.c_void_p),
                ("lse_host", C.c_void_p), ("q_bytes", C.c_int64), ("out_bytes", C.c_int64)]


EXPORTS = ["dsa_v32_abi_version", "dsa_v32_error_string", "dsa_v32_plan_info_get", "dsa_v32_plan",
           "dsa_v32_plan_host", "dsa_v32_plan_read", "dsa_v32_plan_release", "dsa_v32_decode_bf16", "dsa_v32_decode_fp8",
           "dsa_v32_prefill_bf16", "dsa_v32_combine", "dsa_v32_decode_pipeline", "dsa_v32_device_status",
           "dsa_v32_debug_rows", "dsa_v32_pack_fp8_rows", "dsa_v32_decode_pipeline_host",
           "dsa_v32_decode_pipeline_static", "dsa_v32_static_scratch_address", "dsa_v32_selftest_wait_expiry", "dsa_v32_decode_pipeline_allgather", "dsa_v32_ipc_export", "dsa_v32_ipc_open", "dsa_v32_ipc_close", "dsa_v32_decode_pipeline_host_chunked", "dsa_v32_decode_pipeline_host_lanes", "dsa_v32_decode_pipeline_v4", "dsa_v32_topk_select"]

_lib = None


class DsaError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = lib().dsa_v32_error_string(status).decode()
        super().__init__("%s failed with status %d: %s" % (where, status, msg))


def lib():
    """Loads the CUDA library; there is no fallback of any kind."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libdsa_v32.so is not built; run `python -m opfoundry_b200.build` "
                              "(the package has no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        L.dsa_v32_error_string.restype = C.c_char_p
        L.dsa_v32_error_string.argtypes = [C.c_int]
        L.dsa_v32_plan_info_get.argtypes = [C.POINTER(Shape), C.POINTER(PlanInfo)]
        L.dsa_v32_plan.argtypes = [C.POINTER(Shape), C.c_void_p, C.c_int64, C.c_void_p]
        L.dsa_v32_plan_host.argtypes = [C.POINTER(Shape), C.c_void_p, C.c_int64, C.POINTER(C.c_int64)]
        L.dsa_v32_plan_read.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]
        L.dsa_v32_plan_release.argtypes = [C.c_void_p]
        L.dsa_v32_selftest_wait_expiry.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        for name in ("dsa_v32_decode_bf16", "dsa_v32_decode_fp8", "dsa_v32_prefill_bf16", "dsa_v32_combine",
                     "dsa_v32_device_status"):
            getattr(L, name).argtypes = [C.POINTER(AttnArgs), C.c_void_p]
        L.dsa_v32_decode_pipeline.argtypes = [C.POINTER(AttnArgs), C.c_int, C.c_void_p]
        L.dsa_v32_decode_pipeline_host.argtypes = [C.POINTER(AttnArgs), C.POINTER(HostIO), C.c_void_p]
        L.dsa_v32_decode_pipeline_static.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
        L.dsa_v32_decode_pipeline_v4.argtypes = [C.POINTER(AttnArgs), C.POINTER(V4Ext), C.c_void_p]
        L.dsa_v32_decode_pipeline_host_chunked.argtypes = [C.POINTER(AttnArgs), C.POINTER(HostIO), C.c_int32, C.c_void_p]
        L.dsa_v32_decode_pipeline_host_lanes.argtypes = [C.POINTER(AttnArgs), C.POINTER(HostIO), C.c_int32, C.POINTER(C.c_void_p),
                                                         C.POINTER(C.c_int64), C.c_int32, C.c_void_p]
        L.dsa_v32_decode_pipeline_allgather.argtypes = [C.POINTER(AttnArgs), C.POINTER(PeerOutputs), C.c_void_p]
        L.dsa_v32_ipc_export.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64)]
        L.dsa_v32_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        L.dsa_v32_ipc_close.argtypes = [C.c_void_p]
        L.dsa_v32_static_scratch_address.restype = C.c_void_p
        L.dsa_v32_static_scratch_address.argtypes = []
        L.dsa_v32_debug_rows.argtypes = [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p]
        L.dsa_v32_topk_select.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        L.dsa_v32_pack_fp8_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        _lib = L
    return _lib


def _check(status, where):
    if status != 0:
        raise DsaError(status, where)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class MlaDecodePlan:
    """Counterpart of the reference's `mla_decode_plan` (common/host.cc:69-88): shape facts plus the
    caller-owned device workspace holding the work list, reduce tables and split partials."""

    def __init__(self, total_q, H, topk, s_q, info, workspace, hint):
        self.total_q, self.H, self.topk, self.s_q = total_q, H, topk, s_q
        self.info = info
        self.workspace = workspace
        self._hint = hint

    @property
    def num_lists(self):
        return self.info.num_lists

    def read_works(self):
        works = (WorkInfo * self.info.num_works)()
        indptr = (C.c_int32 * (self.info.num_lists + 1))()
        _check(lib().dsa_v32_plan_read(self.workspace.data_ptr(), self.workspace.numel(), works, self.info.num_works,
                                       indptr, self.info.num_lists + 1, _stream()), "dsa_v32_plan_read")
        return list(works), list(indptr)


PLAN_AUTO_SPLIT = 1


def _shape(total_q, H, topk, s_q, num_sms, hint, flags=0, mtp_shared=None):
    sh = Shape(total_q, H, topk, s_q, num_sms, flags, None, None)
    keep = []
    if hint is not None:
        k = (C.c_int32 * total_q)(*[int(x) for x in hint])
        sh.valid_len_hint = C.cast(k, C.c_void_p)
        keep.append(k)
    if mtp_shared is not None:
        k = (C.c_uint8 * (total_q // s_q))(*[1 if x else 0 for x in mtp_shared])
        sh.mtp_shared = C.cast(k, C.c_void_p)
        keep.append(k)
    return sh, keep


def mla_decode_plan_create(total_q, H, topk, s_q=1, *, device="cuda", valid_len_hint=None, num_sms=0, auto_split=False,
                           mtp_shared=None):
    """Sizes the workspace, allocates it (torch owns it) and runs the metadata stage once.
    auto_split: the reference scheduler's option of the same name (fewer work lists for small problems).
    mtp_shared: per sequence, whether its s_q query rows carry the same index list (then, when s_q * H <= 128,
    they are planned as one item that gathers the rows once)."""
    sh, keep = _shape(total_q, H, topk, s_q, num_sms, valid_len_hint, PLAN_AUTO_SPLIT if auto_split else 0, mtp_shared)
    info = PlanInfo()
    _check(lib().dsa_v32_plan_info_get(C.byref(sh), C.byref(info)), "dsa_v32_plan_info_get")
    ws = torch.empty(int(info.workspace_bytes) + 256, dtype=torch.uint8, device=device)
    off = (-ws.data_ptr()) % 256
    ws = ws[off:off + int(info.workspace_bytes)]
    _check(lib().dsa_v32_plan(C.byref(sh), ws.data_ptr(), ws.numel(), _stream()), "dsa_v32_plan")
    return MlaDecodePlan(total_q, H, topk, s_q, info, ws, keep)


def plan_host(total_q, H, topk, s_q=1, *, num_sms=148, valid_len_hint=None, auto_split=False, mtp_shared=None):
    """Runs the planner on the host only and returns the raw metadata blob (bytes) - no GPU needed."""
    sh, keep = _shape(total_q, H, topk, s_q, num_sms, valid_len_hint, PLAN_AUTO_SPLIT if auto_split else 0, mtp_shared)
    need = C.c_int64(0)
    _check(lib().dsa_v32_plan_host(C.byref(sh), None, 0, C.byref(need)), "dsa_v32_plan_host")
    buf = (C.c_uint8 * need.value)()
    _check(lib().dsa_v32_plan_host(C.byref(sh), buf, need.value, C.byref(need)), "dsa_v32_plan_host")
    return bytes(buf)


def make_args(q, kv, indices, plan, sm_scale, *, out, lse, block_table=None, page_block_size=64,
              kv_batch_stride_rows=0):
    assert q.dtype == torch.bfloat16 and q.dim() == 3 and q.shape[2] == D_QK and q.stride(2) == 1
    assert indices.dtype == torch.int32 and indices.is_contiguous()
    total_q, H = q.shape[0], q.shape[1]
    a = AttnArgs()
    a.q = q.data_ptr()
    a.kv = kv.data_ptr()
    a.out = out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.indices = indices.data_ptr()
    if kv.dtype == torch.uint8:
        assert kv.is_contiguous() and kv.shape[-1] == FP8_ROW_BYTES
        a.kv_dtype = KV_FP8
        a.num_kv_rows = kv.numel() // FP8_ROW_BYTES
    else:
        assert kv.dtype == torch.bfloat16 and kv.is_contiguous() and kv.shape[-1] == D_QK
        a.kv_dtype = KV_BF16
        a.num_kv_rows = kv.numel() // D_QK
    if block_table is not None:
        assert block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2
        a.block_table = block_table.data_ptr()
        a.block_table_stride = block_table.shape[1]
        a.page_block_size = page_block_size
    else:
        a.block_table = None
        a.block_table_stride = 0
        a.page_block_size = 1
    a.kv_batch_stride_rows = kv_batch_stride_rows
    a.workspace = plan.workspace.data_ptr()
    a.workspace_bytes = plan.workspace.numel()
    a.stride_q_row, a.stride_q_head = q.stride(0), q.stride(1)
    a.stride_o_row, a.stride_o_head = out.stride(0), out.stride(1)
    a.total_q, a.H, a.topk, a.s_q = total_q, H, indices.shape[1], plan.s_q
    a.sm_scale = float(sm_scale)
    return a


def mla_decode_launch_pipeline(q, kv, indices, plan, sm_scale, *, block_table=None, page_block_size=64,
                               kv_batch_stride_rows=0, out=None, lse=None, run_metadata=False, check=True):
    """metadata (optional) -> attention -> merge on the current stream; returns (out, lse).

    q [total_q, H, 576] bf16; kv [rows, 576] bf16 or [rows, 656] uint8 (fp8 cache rows);
    indices [total_q, topk] int32 with -1 padding.  `check` reads the device status word back
    (one stream synchronisation); pass False inside timed loops.
    """
    total_q, H = q.shape[0], q.shape[1]
    if out is None:
        out = torch.empty(total_q, H, D_V, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(total_q, H, dtype=torch.float32, device=q.device)
    a = make_args(q, kv, indices, plan, sm_scale, out=out, lse=lse, block_table=block_table,
                  page_block_size=page_block_size, kv_batch_stride_rows=kv_batch_stride_rows)
    _check(lib().dsa_v32_decode_pipeline(C.byref(a), 1 if run_metadata else 0, _stream()), "dsa_v32_decode_pipeline")
    if check:
        _check(lib().dsa_v32_device_status(C.byref(a), _stream()), "dsa_v32_device_status")
    return out, lse


def mla_v4_launch_pipeline(q, kv, indices, plan, sm_scale, *, attn_sink=None, kv2=None, pool_split=None, block_table=None,
                           page_block_size=64, kv_batch_stride_rows=0, out=None, lse=None, check=True):
    """The pipeline with an attention sink per head (fp32 [H]) and / or a second pool of bf16 rows for the
    slots at or beyond pool_split[q] (int32 [total_q], physical rows of kv2): the two features of the
    reference's v4 prefill kernels."""
    total_q, H = q.shape[0], q.shape[1]
    if out is None:
        out = torch.empty(total_q, H, D_V, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(total_q, H, dtype=torch.float32, device=q.device)
    a = make_args(q, kv, indices, plan, sm_scale, out=out, lse=lse, block_table=block_table,
                  page_block_size=page_block_size, kv_batch_stride_rows=kv_batch_stride_rows)
    ext = V4Ext()
    if attn_sink is not None:
        assert attn_sink.dtype == torch.float32 and attn_sink.numel() == H and attn_sink.is_contiguous()
        ext.attn_sink = attn_sink.data_ptr()
    if kv2 is not None:
        assert kv2.dtype == torch.bfloat16 and kv2.is_contiguous() and kv2.shape[-1] == D_QK
        assert pool_split is not None and pool_split.dtype == torch.int32 and pool_split.numel() == total_q
        ext.kv2, ext.pool_split, ext.num_kv2_rows = kv2.data_ptr(), pool_split.data_ptr(), kv2.numel() // D_QK
    _check(lib().dsa_v32_decode_pipeline_v4(C.byref(a), C.byref(ext), _stream()), "dsa_v32_decode_pipeline_v4")
    if check:
        _check(lib().dsa_v32_device_status(C.byref(a), _stream()), "dsa_v32_device_status")
    return out, lse


def sparse_mla_prefill(q, kv, indices, plan, sm_scale, **kw):
    """Prefill is the same pipeline with one query row per token (bf16 cache)."""
    return mla_decode_launch_pipeline(q, kv, indices, plan, sm_scale, **kw)


def debug_rows(indices, *, s_q=1, num_kv_rows, block_table=None, page_block_size=64, kv_batch_stride_rows=0):
    """Physical row the kernel's translation resolves every (query, slot) to; -1 = masked."""
    a = AttnArgs()
    a.indices = indices.data_ptr()
    a.total_q, a.topk, a.s_q = indices.shape[0], indices.shape[1], s_q
    a.num_kv_rows = num_kv_rows
    a.kv_batch_stride_rows = kv_batch_stride_rows
    if block_table is not None:
        a.block_table = block_table.data_ptr()
        a.block_table_stride = block_table.shape[1]
        a.page_block_size = page_block_size
    rows = torch.empty_like(indices)
    _check(lib().dsa_v32_debug_rows(C.byref(a), rows.data_ptr(), _stream()), "dsa_v32_debug_rows")
    return rows


def topk_select(scores, topk, valid_len=None, out=None):
    """scores fp32 [total_q, kv_len] (device) -> int32 [total_q, topk]: the positions of the topk largest scores of
    every row among its first valid_len[q] positions, ascending, -1 padded."""
    assert scores.dtype == torch.float32 and scores.dim() == 2 and scores.stride(1) == 1
    total_q, kv_len = scores.shape
    if out is None:
        out = torch.empty(total_q, topk, dtype=torch.int32, device=scores.device)
    vl = None
    if valid_len is not None:
        assert valid_len.dtype == torch.int32 and valid_len.numel() == total_q
        vl = valid_len.data_ptr()
    _check(lib().dsa_v32_topk_select(scores.data_ptr(), scores.stride(0), vl, total_q, kv_len, topk, out.data_ptr(), _stream()),
           "dsa_v32_topk_select")
    return out


def pack_fp8_rows(latent, rope, out=None, dst_rows=None):
    """latent [n,512] fp32 + rope [n,64] bf16 (device) -> fp8 cache rows [n or given, 656] uint8."""
    n = latent.shape[0]
    assert latent.dtype == torch.float32 and latent.is_contiguous() and latent.shape[1] == D_V
    assert rope.dtype == torch.bfloat16 and rope.is_contiguous() and rope.shape == (n, D_ROPE)
    if out is None:
        out = torch.empty(n, FP8_ROW_BYTES, dtype=torch.uint8, device=latent.device)
    dr = dst_rows.data_ptr() if dst_rows is not None else None
    _check(lib().dsa_v32_pack_fp8_rows(latent.data_ptr(), rope.data_ptr(), dr, out.data_ptr(), n, _stream()),
           "dsa_v32_pack_fp8_rows")
    return out


def mla_decode_step_host(args, q_host, indices_host, out_host, lse_host, num_chunks=1, lane_plans=None):
    """One serving step with pinned HOST tensors: H2D of q / indices, attention + merge, D2H of
    out / lse, all on the current stream (asynchronous; synchronise the stream to read results).
    `args` comes from make_args and names the resident device buffers.  num_chunks > 1 cuts the batch
    into that many groups of sequences whose copies overlap the other groups' kernels; the plan in
    `args` must then be for one group's shape (total_q / num_chunks rows).  lane_plans: plans for one
    group's shape made with num_sms = SMs / len(lane_plans); their kernels run side by side."""
    io = HostIO()
    io.q_host = q_host.data_ptr()
    io.indices_host = indices_host.data_ptr()
    io.out_host = out_host.data_ptr()
    io.lse_host = lse_host.data_ptr()
    io.q_bytes = q_host.numel() * q_host.element_size()
    io.out_bytes = out_host.numel() * out_host.element_size()
    if lane_plans:
        n = len(lane_plans)
        ws = (C.c_void_p * n)(*[p.workspace.data_ptr() for p in lane_plans])
        wb = (C.c_int64 * n)(*[p.workspace.numel() for p in lane_plans])
        _check(lib().dsa_v32_decode_pipeline_host_lanes(C.byref(args), C.byref(io), num_chunks, ws, wb, n, _stream()),
               "dsa_v32_decode_pipeline_host_lanes")
        return
    if num_chunks > 1:
        _check(lib().dsa_v32_decode_pipeline_host_chunked(C.byref(args), C.byref(io), num_chunks, _stream()),
               "dsa_v32_decode_pipeline_host_chunked")
        return
    _check(lib().dsa_v32_decode_pipeline_host(C.byref(args), C.byref(io), _stream()), "dsa_v32_decode_pipeline_host")


def mla_decode_launch_pipeline_static(q, kv, indices, sm_scale, *, s_q=1, block_table=None, page_block_size=64,
                                      kv_batch_stride_rows=0, out=None, lse=None, check=True):
    """The pipeline for callers that may not allocate device memory: the split workspace is a fixed
    array inside the library (48 MiB per GPU, shared by all calls, so calls must not overlap on the
    GPU).  The first call for a shape plans it - make that call before any stream capture.  Shapes
    whose plan does not fit raise DsaError with status ERR_SCRATCH_TOO_SMALL.  `out` / `lse` should be
    passed in by such a caller; they are only created here for convenience when omitted."""
    total_q, H = q.shape[0], q.shape[1]
    if out is None:
        out = torch.empty(total_q, H, D_V, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(total_q, H, dtype=torch.float32, device=q.device)

    class _NoPlan:   # make_args only needs the shape facts of a plan
        pass
    np_ = _NoPlan()
    np_.s_q = s_q
    np_.workspace = torch.empty(0, dtype=torch.uint8)   # ignored by the entry point
    a = make_args(q, kv, indices, np_, sm_scale, out=out, lse=lse, block_table=block_table,
                  page_block_size=page_block_size, kv_batch_stride_rows=kv_batch_stride_rows)
    a.workspace = None
    a.workspace_bytes = 0
    _check(lib().dsa_v32_decode_pipeline_static(C.byref(a), _stream()), "dsa_v32_decode_pipeline_static")
    if check:
        a.workspace = lib().dsa_v32_static_scratch_address()
        _check(lib().dsa_v32_device_status(C.byref(a), _stream()), "dsa_v32_device_status")
    return out, lse
