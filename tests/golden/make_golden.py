"""Generates the golden fixtures in this directory by running the reference's own CPU functions
(opus_attn/dsa_v32/common/host.cc compiled through oracle/ref_wrap.cu) on small seeded inputs.

Run where a checkout of the reference is present:  python tests/golden/make_golden.py
The fixtures store inputs and the reference's outputs, so the tests need neither the reference
checkout nor this script at run time.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import build as obuild  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    obuild.build_oracle()
    assert obuild.build_ref(), "reference checkout not found"
    R = O.ref_lib()
    rng = np.random.default_rng(20261125)

    # ---- codec tables (defs.h:11-52)
    decode = np.array([R.ref_e4m3_to_float(b) for b in range(256)], dtype=np.float32)
    probes = np.concatenate([
        np.array([0.0, -0.0, 1.0, -1.0, 448.0, 449.0, 464.0, 480.0, 1e9, -1e9, np.inf, -np.inf, np.nan,
                  2.0 ** -6, 2.0 ** -7, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 0.3, 0.3125, 0.0009765625 * 3], dtype=np.float32),
        rng.standard_normal(2000).astype(np.float32) * np.float32(100.0),
        rng.standard_normal(2000).astype(np.float32) * np.float32(0.01),
        decode[np.isfinite(decode)],
        ((decode[:-1] + decode[1:]) / 2)[np.isfinite(decode[:-1] + decode[1:])].astype(np.float32),  # ties
    ]).astype(np.float32)
    encode = np.array([R.ref_float_to_e4m3(float(x)) for x in probes], dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "codec_e4m3.npz"), decode=decode.view(np.uint32), probes=probes.view(np.uint32),
                        encode=encode)

    # ---- bf16 decode, CSR page table, s_q = 2, variable lengths (host.cc:508-548)
    B, H, S, sq = 3, 5, 40, 2
    ip = np.zeros(B + 1, np.int32)
    ix = np.zeros(B * S, np.int32)
    n = R.ref_init_kv_page_table(O._p(ip), O._p(ix), B * S, B, S, 1, 1234)
    ix = ix[:n].copy()
    q = O.f32_to_bf16(rng.standard_normal((B * sq, H, 576)).astype(np.float32))
    kv = O.f32_to_bf16(rng.standard_normal((n, 576)).astype(np.float32))
    out = np.zeros((B * sq, H, 512), np.uint16)
    lse = np.zeros((B * sq, H), np.float32)
    R.ref_attention_bf16(O._p(q), O._p(kv), O._p(out), O._p(lse), O._p(ip), O._p(ix), B, H, sq)
    np.savez_compressed(os.path.join(HERE, "ref_bf16_csr.npz"), q=q, kv=kv, kv_indptr=ip, kv_indices=ix, out=out,
                        lse=lse, B=B, H=H, s_q=sq)

    # ---- one sequence shorter than s_q-1 rows: empty selection -> out 0, lse +inf (host.cc:530-534)
    B, H, sq = 2, 3, 3
    ip = np.array([0, 1, 9], np.int32)
    ix = rng.permutation(9).astype(np.int32)
    q = O.f32_to_bf16(rng.standard_normal((B * sq, H, 576)).astype(np.float32))
    kv = O.f32_to_bf16(rng.standard_normal((9, 576)).astype(np.float32))
    out = np.zeros((B * sq, H, 512), np.uint16)
    lse = np.zeros((B * sq, H), np.float32)
    R.ref_attention_bf16(O._p(q), O._p(kv), O._p(out), O._p(lse), O._p(ip), O._p(ix), B, H, sq)
    np.savez_compressed(os.path.join(HERE, "ref_bf16_empty.npz"), q=q, kv=kv, kv_indptr=ip, kv_indices=ix, out=out,
                        lse=lse, B=B, H=H, s_q=sq)

    # ---- fp8 (host.cc:459-506) with scale bytes constant inside every group of 128 values, so the
    #      same numbers can be expressed in the packed row format (one fp32 scale per 128)
    B, H, S, sq = 2, 4, 24, 1
    ip = np.zeros(B + 1, np.int32)
    ix = np.zeros(B * S, np.int32)
    n = R.ref_init_kv_page_table(O._p(ip), O._p(ix), B * S, B, S, 0, 77)
    ix = ix[:n].copy()

    def fp8_tensor(rows):
        e = rng.integers(0, 4, size=(rows, 4))
        scale = np.repeat(e + 127, 4, axis=1).astype(np.uint8)  # 16 E8M0 bytes, equal inside each 128-group
        x = rng.standard_normal((rows, 512)).astype(np.float32) * np.exp2(-np.repeat(e, 128, axis=1)).astype(np.float32)
        nope = np.array([R.ref_float_to_e4m3(float(v)) for v in x.reshape(-1)], dtype=np.uint8).reshape(rows, 512)
        rope = O.f32_to_bf16(rng.standard_normal((rows, 64)).astype(np.float32))
        return nope, scale, rope

    qn, qs, qr = fp8_tensor(B * sq * H)
    kn, ks, kr = fp8_tensor(n)
    out = np.zeros((B * sq, H, 512), np.uint16)
    lse = np.zeros((B * sq, H), np.float32)
    R.ref_attention_fp8(O._p(qn), O._p(qs), O._p(qr), O._p(kn), O._p(ks), O._p(kr), O._p(out), O._p(lse), O._p(ip),
                        O._p(ix), B, H, sq)
    np.savez_compressed(os.path.join(HERE, "ref_fp8_csr.npz"), q_nope=qn, q_scale=qs, q_rope=qr, kv_nope=kn, kv_scale=ks,
                        kv_rope=kr, kv_indptr=ip, kv_indices=ix, out=out, lse=lse, B=B, H=H, s_q=sq)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
