"""Seeded synthetic inputs for the sparse-MLA path (host side, numpy).

Plays the role of the reference harness's generators (opus_attn/dsa_v32/common/host.cc:191-261:
`rand_vector`, `init_fp8_mla_split`, `init_kv_page_table`) for the inputs this library takes:
bf16 queries, a bf16 or packed-fp8 latent cache, a randomly permuted block table and one top-k
list per query with -1 padding.  Unlike the reference (which seeds Q and KV identically, so Q
row r equals KV row r), every tensor draws from its own counter-based stream, keyed by
(seed, tensor tag), so results do not depend on generation order or thread count.

bf16 values are carried as uint16 bit patterns and fp8 cache rows as uint8 so the same bytes
can be handed to the CPU checker and uploaded to the GPU.
"""
import numpy as np

D_QK, D_V, D_ROPE = 576, 512, 64
FP8_ROW_BYTES = 656

_TAGS = {"q": 1, "kv": 2, "rope": 3, "indices": 4, "block_table": 5, "share": 6, "kv2": 7}


def stream(seed, tag, sub=0):
    return np.random.Generator(np.random.Philox(key=[int(seed), (_TAGS[tag] << 32) | int(sub)]))


def f32_to_bf16_bits(x):
    """fp32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3_bits(x):
    """fp32 -> e4m3 bytes: round to nearest even, saturate to +-448 (0x7E), NaN/Inf -> 0x7F,
    subnormals in steps of 2^-9 (the codec of opus_attn/dsa_v32/common/defs.h:11-38)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    mag = bits & 0x7FFFFFFF
    exp = (mag >> 23).astype(np.int32) - 127
    mant = mag & 0x7FFFFF
    # normal range (exp >= -6)
    pay_n = (((exp + 7) << 3).astype(np.int64) | (mant >> 20)).astype(np.int64)
    drop_n = (mant & 0xFFFFF).astype(np.int64)
    half_n = np.int64(0x80000)
    # subnormal range
    shift = np.clip(-exp - 6, 1, 12).astype(np.int64)
    full = (mant | 0x800000).astype(np.int64)
    width = 20 + shift
    pay_s = full >> width
    drop_s = full & ((np.int64(1) << width) - 1)
    half_s = np.int64(1) << (width - 1)
    normal = exp >= -6
    pay = np.where(normal, pay_n, pay_s)
    drop = np.where(normal, drop_n, drop_s)
    half = np.where(normal, half_n, half_s)
    pay = pay + ((drop > half) | ((drop == half) & ((pay & 1) == 1)))
    pay = np.where((~normal) & ((-exp - 6) > 11), 0, pay)
    pay = np.where(mag >= 0x43E00000, 0x7E, pay)
    pay = np.where(mag >= 0x7F800000, 0x7F, pay)
    return (sign | pay.astype(np.uint8)).astype(np.uint8)


def pack_fp8_rows(latent_f32, rope_bits):
    """[n,512] fp32 + [n,64] bf16 bits -> [n,656] uint8: per 128 values scale = amax/448 (fp32, 1.0 for
    an all-zero group) and e4m3(x / scale); then the 4 scales; then the rope values."""
    latent = np.ascontiguousarray(latent_f32, dtype=np.float32)
    n = latent.shape[0]
    g = latent.reshape(n, 4, 128)
    amax = np.abs(g).max(axis=2)
    scale = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    qv = (g / scale[:, :, None]).astype(np.float32)
    rows = np.empty((n, FP8_ROW_BYTES), dtype=np.uint8)
    rows[:, :D_V] = f32_to_e4m3_bits(qv).reshape(n, D_V)
    rows[:, D_V:D_V + 16] = scale.view(np.uint8).reshape(n, 16)
    rows[:, D_V + 16:] = np.ascontiguousarray(rope_bits, dtype=np.uint16).view(np.uint8).reshape(n, 128)
    return rows


def normal_bf16(seed, tag, shape, sub=0):
    return f32_to_bf16_bits(stream(seed, tag, sub).standard_normal(size=shape, dtype=np.float32))


def unique_indices(rng, n_choices, k):
    """k distinct positions drawn uniformly from [0, n_choices) in random order (partial shuffle)."""
    if k >= n_choices:
        return rng.permutation(n_choices).astype(np.int32)
    return rng.choice(n_choices, size=k, replace=False).astype(np.int32)


def make_decode_case(B, H, kv_len, topk, *, s_q=1, fp8=False, paged=False, page_block_size=64, pad_frac=0.0,
                     share_mtp=None, seed=2026, scatter_pad=False):
    """Decode inputs.  Returns a dict:
       q [B*s_q,H,576] u16 | kv [rows,576] u16 or [rows,656] u8 | indices [B*s_q,topk] i32 |
       block_table [B,blocks] i32 or None | page_block_size | kv_batch_stride_rows | s_q.
    pad_frac: that fraction of the slots (the tail, or random positions with scatter_pad) is -1.
    share_mtp: None = independent lists per query row; 'coin' = per sequence a seeded coin flip
    decides whether its s_q rows share one list."""
    total_q = B * s_q
    q = normal_bf16(seed, "q", (total_q, H, D_QK))
    if paged:
        assert kv_len % page_block_size == 0
        blocks_per_seq = kv_len // page_block_size
        n_blocks = B * blocks_per_seq
        block_table = stream(seed, "block_table").permutation(n_blocks).astype(np.int32).reshape(B, blocks_per_seq)
        n_rows = n_blocks * page_block_size
        stride_rows = 0
    else:
        block_table = None
        n_rows = B * kv_len
        stride_rows = kv_len
    if fp8:
        latent = stream(seed, "kv").standard_normal(size=(n_rows, D_V), dtype=np.float32)
        rope = normal_bf16(seed, "rope", (n_rows, D_ROPE))
        kv = pack_fp8_rows(latent, rope)
    else:
        kv = normal_bf16(seed, "kv", (n_rows, D_QK))
    n_pad = int(pad_frac * topk)
    indices = np.full((total_q, topk), -1, dtype=np.int32)
    coin = stream(seed, "share").integers(0, 2, size=B) if share_mtp == "coin" else np.zeros(B, dtype=np.int64)
    for b in range(B):
        for t in range(s_q):
            r = b * s_q + t
            if t > 0 and coin[b]:
                indices[r] = indices[b * s_q]
                continue
            rng = stream(seed, "indices", r)
            sel = unique_indices(rng, kv_len, min(topk, kv_len))
            row = np.full(topk, -1, dtype=np.int32)
            row[:len(sel)] = sel
            if n_pad:
                if scatter_pad:
                    row[rng.choice(topk, size=n_pad, replace=False)] = -1
                else:
                    row[topk - n_pad:] = -1
            indices[r] = row
    return dict(q=q, kv=kv, indices=indices, block_table=block_table, page_block_size=page_block_size,
                kv_batch_stride_rows=stride_rows, s_q=s_q, fp8=fp8, H=H, topk=topk, kv_len=kv_len, B=B,
                mtp_shared=(coin != 0))


def make_prefill_case(T, H, topk, *, seed=2026, q_rows=None):
    """Causal prefill: one sequence of T tokens, query t draws min(t+1, topk) distinct positions from
    [0, t]; unused slots are -1.  q_rows (optional) limits generation to a subset of query rows
    (the other rows of `indices` stay -1 and q stays zero) to keep large cases cheap."""
    kv = normal_bf16(seed, "kv", (T, D_QK))
    q = np.zeros((T, H, D_QK), dtype=np.uint16)
    indices = np.full((T, topk), -1, dtype=np.int32)
    rows = range(T) if q_rows is None else q_rows
    for t in rows:
        q[t] = normal_bf16(seed, "q", (H, D_QK), sub=t)
        rng = stream(seed, "indices", t)
        sel = unique_indices(rng, t + 1, min(topk, t + 1))
        indices[t, :len(sel)] = sel
    valid_len = np.minimum(np.arange(T) + 1, topk).astype(np.int32)
    return dict(q=q, kv=kv, indices=indices, block_table=None, page_block_size=1, kv_batch_stride_rows=0, s_q=T,
                fp8=False, H=H, topk=topk, kv_len=T, B=1, valid_len=valid_len)
