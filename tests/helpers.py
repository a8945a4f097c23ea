"""Shared helpers of the test-suite: golden loading, conversions between the reference's CSR /
MXFP8 inputs and the inputs this library takes, and the parity criteria."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Parity bar: every element |gpu - ref| <= atol + rtol * |ref|, no mismatch budget.
TOL_BF16 = dict(atol=2e-2, rtol=1e-2)   # bf16 cache
TOL_FP8 = dict(atol=5e-2, rtol=1e-2)    # fp8 cache
LSE_ATOL = 1e-3
LSE_RTOL = 1e-3


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def csr_to_lists(kv_indptr, kv_indices, B, s_q, topk=None):
    """The reference selects rows per batch through a CSR page table and trims token t of an s_q
    group causally (host.cc:482,526).  Returns the equivalent per-query lists with -1 padding."""
    lens = []
    for i in range(B * s_q):
        b = i // s_q
        lens.append(int(kv_indptr[b + 1]) - (s_q - 1 - i % s_q) - int(kv_indptr[b]))
    if topk is None:
        topk = max(1, max(lens))
    ind = np.full((B * s_q, topk), -1, np.int32)
    for i, n in enumerate(lens):
        if n > 0:
            b = i // s_q
            ind[i, :n] = kv_indices[kv_indptr[b]:kv_indptr[b] + n]
    return ind


def mxfp8_q_to_bf16(q_nope, q_scale, q_rope, decode_table):
    """fp8 value x 2^(e-127) is exactly representable in bf16, so the reference's quantised query
    converts without rounding."""
    rows = q_nope.shape[0]
    val = decode_table[q_nope.astype(np.int64)] * np.exp2(np.repeat(q_scale.astype(np.int32) - 127, 32, axis=1)).astype(np.float32)
    f = np.concatenate([val.astype(np.float32), (q_rope.astype(np.uint32) << 16).view(np.float32)], axis=1)
    bits = f.view(np.uint32)
    assert np.all((bits & 0xFFFF) == 0), "not exactly representable in bf16"
    return (bits >> 16).astype(np.uint16).reshape(rows, 576)


def mxfp8_kv_to_rows(kv_nope, kv_scale, kv_rope):
    """Reference layout (three tensors, one E8M0 byte per 32 values) -> packed 656-byte rows.
    Requires the scale bytes to be equal inside each group of 128 values."""
    n = kv_nope.shape[0]
    s = kv_scale.reshape(n, 4, 4)
    assert np.all(s == s[:, :, :1])
    scale = np.exp2(s[:, :, 0].astype(np.int32) - 127).astype(np.float32)
    rows = np.empty((n, 656), np.uint8)
    rows[:, :512] = kv_nope
    rows[:, 512:528] = scale.view(np.uint8).reshape(n, 16)
    rows[:, 528:] = kv_rope.view(np.uint8).reshape(n, 128)
    return rows


def check_out(gpu_bits, ref_bits, atol, rtol, what="out"):
    g = (gpu_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    r = (ref_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.all(np.isfinite(g)), "%s: NaN/Inf on the GPU side" % what
    assert np.all(np.isfinite(r)), "%s: NaN/Inf in the reference" % what
    err = np.abs(g - r)
    bad = err > atol + rtol * np.abs(r)
    assert not bad.any(), "%s: %d / %d elements out of tolerance, max abs err %.5f" % (what, bad.sum(), bad.size, err.max())
    return float(err.max())


def check_lse(gpu, ref):
    gi, ri = np.isinf(gpu), np.isinf(ref)
    assert np.array_equal(gi, ri), "lse: infinities differ"
    assert np.array_equal(np.sign(gpu[gi]), np.sign(ref[ri])), "lse: sign of infinities differs"
    g, r = gpu[~gi].astype(np.float64), ref[~ri].astype(np.float64)
    assert np.all(np.isfinite(g)), "lse: NaN on the GPU side"
    err = np.abs(g - r)
    bad = err > LSE_ATOL + LSE_RTOL * np.abs(r)
    assert not bad.any(), "lse: %d / %d out of tolerance, max err %.6f" % (bad.sum(), bad.size, err.max() if err.size else 0)
    return float(err.max()) if err.size else 0.0
