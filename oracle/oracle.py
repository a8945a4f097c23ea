"""ctypes front-end of the test-only CPU oracle (dsa_oracle.c) and, when built, of the
reference's own CPU functions (ref_wrap.cu -> _ref/libdsa_ref.so).

bf16 tensors travel as numpy uint16 arrays holding the raw bit patterns.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

D_QK, D_V, D_ROPE, FP8_ROW_BYTES = 576, 512, 64, 656

_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = C.CDLL(path)
        L.dsa_oracle_f32_to_e4m3.restype = C.c_uint8
        L.dsa_oracle_f32_to_e4m3.argtypes = [C.c_float]
        L.dsa_oracle_e4m3_to_f32.restype = C.c_float
        L.dsa_oracle_e4m3_to_f32.argtypes = [C.c_uint8]
        L.dsa_oracle_f32_to_bf16.restype = C.c_uint16
        L.dsa_oracle_f32_to_bf16.argtypes = [C.c_float]
        L.dsa_oracle_pack_fp8_rows.restype = None
        L.dsa_oracle_pack_fp8_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
        L.dsa_oracle_dequant_fp8_rows.restype = None
        L.dsa_oracle_dequant_fp8_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.dsa_oracle_sparse_mla.restype = C.c_int
        L.dsa_oracle_sparse_mla.argtypes = [
            C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64,
            C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
            C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int]
        L.dsa_oracle_sparse_mla_v4.restype = C.c_int
        L.dsa_oracle_sparse_mla_v4.argtypes = [
            C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64,
            C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
            C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int]
        L.dsa_oracle_merge.restype = None
        L.dsa_oracle_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def ref_lib():
    """The reference's host.cc compiled as a library, or None when it was never built."""
    global _ref
    if _ref is None:
        path = _build.REF_SO
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.ref_attention_bf16.restype = None
        R.ref_attention_bf16.argtypes = [C.c_void_p] * 6 + [C.c_int] * 3
        R.ref_attention_fp8.restype = None
        R.ref_attention_fp8.argtypes = [C.c_void_p] * 10 + [C.c_int] * 3
        R.ref_rand_bf16.restype = None
        R.ref_rand_bf16.argtypes = [C.c_void_p, C.c_size_t]
        R.ref_init_fp8_split.restype = None
        R.ref_init_fp8_split.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        R.ref_init_kv_page_table.restype = C.c_int
        R.ref_init_kv_page_table.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint]
        R.ref_float_to_e4m3.restype = C.c_uint8
        R.ref_float_to_e4m3.argtypes = [C.c_float]
        R.ref_e4m3_to_float.restype = C.c_float
        R.ref_e4m3_to_float.argtypes = [C.c_uint8]
        R.ref_num_qo_tiles.restype = C.c_int
        R.ref_num_qo_tiles.argtypes = [C.c_int, C.c_int]
        _ref = R
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f32_to_bf16(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def pack_fp8_rows(latent_f32, rope_bf16):
    """[rows,512] fp32 latent + [rows,64] bf16 rope -> [rows,656] uint8 cache rows."""
    latent_f32 = np.ascontiguousarray(latent_f32, dtype=np.float32)
    rope_bf16 = np.ascontiguousarray(rope_bf16, dtype=np.uint16)
    n = latent_f32.shape[0]
    assert latent_f32.shape == (n, D_V) and rope_bf16.shape == (n, D_ROPE)
    out = np.empty((n, FP8_ROW_BYTES), dtype=np.uint8)
    lib().dsa_oracle_pack_fp8_rows(_p(latent_f32), _p(rope_bf16), _p(out), n)
    return out


def dequant_fp8_rows(rows):
    rows = np.ascontiguousarray(rows, dtype=np.uint8)
    n = rows.shape[0]
    out = np.empty((n, D_QK), dtype=np.float32)
    lib().dsa_oracle_dequant_fp8_rows(_p(rows), _p(out), n)
    return out


def sparse_mla(q, kv, indices, sm_scale, *, kv_is_fp8=False, block_table=None, page_block_size=1, s_q=1,
               kv_batch_stride_rows=0, subset=None, num_threads=None, want_rows=False):
    """q uint16 [total_q,H,576]; kv uint16 [rows,576] or uint8 [rows,656]; indices int32 [total_q,topk].

    Returns (out uint16 [total_q,H,512], lse float32 [total_q,H]) and, with want_rows, the physical
    row every slot resolved to.  Raises ValueError on an index the path treats as a caller error.
    """
    q = np.ascontiguousarray(q, dtype=np.uint16)
    total_q, H, dq = q.shape
    assert dq == D_QK
    if kv_is_fp8:
        kv = np.ascontiguousarray(kv, dtype=np.uint8).reshape(-1, FP8_ROW_BYTES)
        row_bytes = FP8_ROW_BYTES
    else:
        kv = np.ascontiguousarray(kv, dtype=np.uint16).reshape(-1, D_QK)
        row_bytes = D_QK * 2
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    assert indices.shape[0] == total_q
    topk = indices.shape[1]
    bt = None
    bt_stride = 0
    if block_table is not None:
        bt = np.ascontiguousarray(block_table, dtype=np.int32)
        bt_stride = bt.shape[1]
    out = np.zeros((total_q, H, D_V), dtype=np.uint16)
    lse = np.zeros((total_q, H), dtype=np.float32)
    rows = np.full((total_q, topk), -2, dtype=np.int32) if want_rows else None
    sub = None
    if subset is not None:
        sub = np.ascontiguousarray(subset, dtype=np.int32)
    if num_threads is None:
        num_threads = int(os.environ.get("DSA_NUM_THREADS", os.cpu_count() or 1))
    rc = lib().dsa_oracle_sparse_mla(_p(q), H * D_QK, D_QK, _p(kv), int(kv_is_fp8), row_bytes, kv.shape[0],
                                     int(kv_batch_stride_rows), _p(indices), topk, _p(bt), bt_stride,
                                     int(page_block_size), int(s_q), float(sm_scale), _p(out), _p(lse), _p(rows),
                                     total_q, H, _p(sub), 0 if sub is None else len(sub), int(num_threads))
    if rc:
        raise ValueError("oracle rejected the inputs, code %d" % rc)
    return (out, lse, rows) if want_rows else (out, lse)


def sparse_mla_v4(q, kv, indices, sm_scale, *, attn_sink=None, kv2=None, pool_split=None, kv_is_fp8=False, block_table=None,
                  page_block_size=1, s_q=1, kv_batch_stride_rows=0, num_threads=None):
    """sparse_mla with the two v4 features: attn_sink float32 [H]; kv2 uint16 [rows2, 576] + pool_split int32
    [total_q] (slots >= pool_split[q] index kv2 by physical row)."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    total_q, H, _ = q.shape
    if kv_is_fp8:
        kv = np.ascontiguousarray(kv, dtype=np.uint8).reshape(-1, FP8_ROW_BYTES)
        row_bytes = FP8_ROW_BYTES
    else:
        kv = np.ascontiguousarray(kv, dtype=np.uint16).reshape(-1, D_QK)
        row_bytes = D_QK * 2
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    topk = indices.shape[1]
    bt, bt_stride = None, 0
    if block_table is not None:
        bt = np.ascontiguousarray(block_table, dtype=np.int32)
        bt_stride = bt.shape[1]
    sink = None if attn_sink is None else np.ascontiguousarray(attn_sink, dtype=np.float32)
    k2 = None if kv2 is None else np.ascontiguousarray(kv2, dtype=np.uint16).reshape(-1, D_QK)
    ps = None if pool_split is None else np.ascontiguousarray(pool_split, dtype=np.int32)
    out = np.zeros((total_q, H, D_V), dtype=np.uint16)
    lse = np.zeros((total_q, H), dtype=np.float32)
    if num_threads is None:
        num_threads = int(os.environ.get("DSA_NUM_THREADS", os.cpu_count() or 1))
    rc = lib().dsa_oracle_sparse_mla_v4(_p(q), H * D_QK, D_QK, _p(kv), int(kv_is_fp8), row_bytes, kv.shape[0],
                                        int(kv_batch_stride_rows), _p(indices), topk, _p(bt), bt_stride, int(page_block_size),
                                        int(s_q), float(sm_scale), _p(out), _p(lse), total_q, H, _p(sink), _p(k2),
                                        0 if k2 is None else k2.shape[0], _p(ps), int(num_threads))
    if rc:
        raise ValueError("oracle rejected the inputs, code %d" % rc)
    return out, lse


def merge(o_parts, lse_parts):
    o_parts = np.ascontiguousarray(o_parts, dtype=np.float32)
    lse_parts = np.ascontiguousarray(lse_parts, dtype=np.float32)
    ns = lse_parts.shape[0]
    out = np.empty(D_V, dtype=np.float32)
    lse = np.empty(1, dtype=np.float32)
    lib().dsa_oracle_merge(_p(o_parts), _p(lse_parts), ns, _p(out), _p(lse))
    return out, float(lse[0])
