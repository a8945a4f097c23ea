"""Pins the CPU oracle (oracle/dsa_oracle.c) to the reference: against golden vectors produced by the
reference's own CPU functions (tests/golden/make_golden.py) and, when the reference build is present
(oracle/_ref), against those functions live.  Bit-exact in both cases."""
import numpy as np
import pytest

from helpers import csr_to_lists, load_golden, mxfp8_kv_to_rows, mxfp8_q_to_bf16

REF_SCALE = np.float32(1.0) / np.sqrt(np.float32(576.0))  # host.cc:437


def test_codec_decode_table(oracle):
    g = load_golden("codec_e4m3.npz")
    dec = np.array([oracle.lib().dsa_oracle_e4m3_to_f32(b) for b in range(256)], dtype=np.float32)
    assert np.array_equal(dec.view(np.uint32), g["decode"])


def test_codec_encode_probes(oracle):
    g = load_golden("codec_e4m3.npz")
    probes = g["probes"].view(np.float32)
    enc = np.array([oracle.lib().dsa_oracle_f32_to_e4m3(float(x)) for x in probes], dtype=np.uint8)
    assert np.array_equal(enc, g["encode"])


def test_bf16_golden(oracle):
    g = load_golden("ref_bf16_csr.npz")
    B, H, sq = int(g["B"]), int(g["H"]), int(g["s_q"])
    ind = csr_to_lists(g["kv_indptr"], g["kv_indices"], B, sq)
    out, lse = oracle.sparse_mla(g["q"], g["kv"], ind, REF_SCALE, s_q=sq, kv_batch_stride_rows=0)
    assert np.array_equal(out, g["out"])
    assert np.array_equal(lse.view(np.uint32), g["lse"].view(np.uint32))


def test_bf16_empty_selection_golden(oracle):
    g = load_golden("ref_bf16_empty.npz")
    B, H, sq = int(g["B"]), int(g["H"]), int(g["s_q"])
    ind = csr_to_lists(g["kv_indptr"], g["kv_indices"], B, sq)
    out, lse = oracle.sparse_mla(g["q"], g["kv"], ind, REF_SCALE, s_q=sq)
    assert np.isposinf(g["lse"]).any(), "fixture must contain an empty selection"
    assert np.array_equal(out, g["out"])
    assert np.array_equal(lse.view(np.uint32), g["lse"].view(np.uint32))


def test_fp8_golden(oracle):
    g = load_golden("ref_fp8_csr.npz")
    codec = load_golden("codec_e4m3.npz")
    B, H, sq = int(g["B"]), int(g["H"]), int(g["s_q"])
    q = mxfp8_q_to_bf16(g["q_nope"], g["q_scale"], g["q_rope"], codec["decode"].view(np.float32)).reshape(B * sq, H, 576)
    rows = mxfp8_kv_to_rows(g["kv_nope"], g["kv_scale"], g["kv_rope"])
    ind = csr_to_lists(g["kv_indptr"], g["kv_indices"], B, sq)
    out, lse = oracle.sparse_mla(q, rows, ind, REF_SCALE, kv_is_fp8=True, s_q=sq)
    assert np.array_equal(out, g["out"])
    assert np.array_equal(lse.view(np.uint32), g["lse"].view(np.uint32))


def test_live_reference_bf16(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("reference build (oracle/_ref) not present")
    B, H, S, sq = 4, 16, 200, 2
    ip = np.zeros(B + 1, np.int32)
    ix = np.zeros(B * S, np.int32)
    n = R.ref_init_kv_page_table(oracle._p(ip), oracle._p(ix), B * S, B, S, 1, 4321)
    ix = ix[:n].copy()
    rng = np.random.default_rng(5)
    q = oracle.f32_to_bf16(rng.standard_normal((B * sq, H, 576)).astype(np.float32))
    kv = np.zeros((n, 576), np.uint16)
    R.ref_rand_bf16(oracle._p(kv), kv.size)  # the reference's own generator (host.cc:194-205)
    out = np.zeros((B * sq, H, 512), np.uint16)
    lse = np.zeros((B * sq, H), np.float32)
    R.ref_attention_bf16(oracle._p(q), oracle._p(kv), oracle._p(out), oracle._p(lse), oracle._p(ip), oracle._p(ix), B, H, sq)
    ind = csr_to_lists(ip, ix, B, sq)
    o2, l2 = oracle.sparse_mla(q, kv, ind, REF_SCALE, s_q=sq)
    assert np.array_equal(out, o2) and np.array_equal(lse.view(np.uint32), l2.view(np.uint32))


def test_live_reference_codec(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("reference build (oracle/_ref) not present")
    rng = np.random.default_rng(9)
    xs = np.concatenate([rng.standard_normal(20000) * 200, rng.standard_normal(20000) * 0.02]).astype(np.float32)
    a = np.array([R.ref_float_to_e4m3(float(x)) for x in xs], np.uint8)
    b = np.array([oracle.lib().dsa_oracle_f32_to_e4m3(float(x)) for x in xs], np.uint8)
    assert np.array_equal(a, b)


def test_oracle_semantics_padding_and_paging(oracle):
    """-1 anywhere in the list is skipped and order is preserved; the block table is honoured; an
    all-padding query gives out = 0 and lse = +inf; other bad indices are rejected."""
    rng = np.random.default_rng(3)
    H, pbs, nblk = 3, 4, 6
    kv = oracle.f32_to_bf16(rng.standard_normal((nblk * pbs, 576)).astype(np.float32))
    q = oracle.f32_to_bf16(rng.standard_normal((2, H, 576)).astype(np.float32))
    bt = np.array([[5, 2, 0], [1, 3, 4]], np.int32)
    ind = np.array([[7, -1, 0, 11, -1, 3], [-1, -1, -1, -1, -1, -1]], np.int32)
    out, lse, rows = oracle.sparse_mla(q, kv, ind, 0.07, block_table=bt, page_block_size=pbs, want_rows=True)
    assert rows[0].tolist() == [2 * 4 + 3, -1, 5 * 4 + 0, 0 * 4 + 3, -1, 5 * 4 + 3]
    assert np.all(out[1] == 0) and np.all(np.isposinf(lse[1]))
    # same selection expressed as physical rows without a table and without the padding
    phys = np.array([[11, 20, 3, 23]], np.int32)
    o2, l2 = oracle.sparse_mla(q[:1], kv, phys, 0.07)
    assert np.array_equal(out[0], o2[0]) and np.array_equal(lse[0], l2[0])
    with pytest.raises(ValueError):
        oracle.sparse_mla(q[:1], kv, np.array([[-2]], np.int32), 0.07)
    with pytest.raises(ValueError):
        oracle.sparse_mla(q[:1], kv, np.array([[nblk * pbs]], np.int32), 0.07)


def test_split_and_merge_matches_unsplit(oracle):
    """Splitting a list and merging the normalised partials with their lse (the reduce stage,
    mla_reduce.hpp:92-156) reproduces the unsplit result."""
    rng = np.random.default_rng(11)
    kv = oracle.f32_to_bf16(rng.standard_normal((300, 576)).astype(np.float32))
    q = oracle.f32_to_bf16(rng.standard_normal((1, 2, 576)).astype(np.float32))
    ind = rng.permutation(300)[:200].astype(np.int32)[None, :]
    full, lse_full = oracle.sparse_mla(q, kv, ind, 0.0721)
    parts, lses = [], []
    for a, b in ((0, 64), (64, 160), (160, 200)):
        o, l = oracle.sparse_mla(q, kv, ind[:, a:b], 0.0721)
        parts.append(oracle.bf16_to_f32(o[0, 0]))
        lses.append(l[0, 0])
    merged, lse_m = oracle.merge(np.stack(parts), np.array(lses, np.float32))
    assert abs(lse_m - lse_full[0, 0]) < 1e-5
    assert np.max(np.abs(merged - oracle.bf16_to_f32(full[0, 0]))) < 2e-2
