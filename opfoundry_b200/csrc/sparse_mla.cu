// Sparse MLA attention for sm_100a: decode (split over the top-k list) and prefill share one
// warp-specialised kernel.
//
// What it computes is the reference lab's decode kernel family
// (opus_attn/dsa_v32/gfx950/mla_decode_a16w16_16mx4_64nx1_template.hpp:815-926 and the mxfp8
// variant mla_decode_mxfp8_16mx8_32nx1_template.hpp:1362-1490): for one work item = one query
// row x one block of 128 heads x a slice of the query's top-k list, an online-softmax attention
// over the gathered latent rows, K = all 576 columns of a row, V = its first 512 columns.
// How it does it is specific to Blackwell:
//
//   * one CTA pair per work list; the two CTAs of a pair walk the same list and each accumulates
//     one 256-column half of the output (the full 128 x 512 fp32 output would fill all of TMEM);
//   * warp 4 (producer): reads 32 top-k slots, translates them through the block table, and
//     gathers the rows with TMA tile::gather4 into 128-byte-swizzled shared memory; the query
//     block is loaded once per item with a tiled TMA load;
//   * warp 5 (MMA issuer): S = Q K^T as 36 tcgen05.mma (M=128, N=32, K=16) with both operands in
//     shared memory and the accumulator in TMEM, then O += P V as 2 tcgen05.mma (M=128, N=256,
//     K=16) whose A operand is P in TMEM and whose B operand is the same gathered tile described
//     MN-major;
//   * warps 0-3 (softmax): one thread per head row; tcgen05.ld of S, log2-domain online softmax
//     with lazy rescaling (the reference's threshold of 8: ..16mx4_64nx1_template.hpp:700-725),
//     P -> bf16 -> tcgen05.st, epilogue O / l -> bf16 (or fp32 partial + lse for split items);
//   * fp8 cache rows add warps 6-9 (convert): raw 656-byte rows are gathered unswizzled and the
//     e4m3 bytes are converted to bf16 exactly (no rounding: e4m3 has 4 significant bits) into the
//     swizzled MMA tile (the reference's LDS round trip: ..mxfp8_16mx8_32nx1_template.hpp:852-864).
//     The per-128 fp32 scales never touch the operands: Q K^T accumulates one fp32 score per scale
//     group (plus one for the rope part) and the softmax warps form s = sum_g scale_g S_g + S_rope
//     in fp32; for P V the softmax warps store one copy of P per scale group, pre-multiplied by
//     that group's scale, and each copy multiplies its own 128 output columns.
//
// Every mbarrier wait is bounded; on expiry the CTA records DSA_V32_ERR_DEVICE_WAIT in the
// workspace status word and drains to its normal exit, where TMEM is released.
#include <cuda_bf16.h>
#include <cfloat>
#include "defs.h"
#include "ptx.cuh"

namespace dsa {

// ------------------------------------------------------------------ shared-memory map
constexpr int kQKBlocks = kDQK / 64;                        // 9 blocks of 64 columns (128 bytes)
constexpr int kQBlockBytes = kHeadsPerBlock * 128;          // 16384
constexpr int kQBytes = kQKBlocks * kQBlockBytes;           // 147456
constexpr int kKvBlockBytes = kTileRows * 128;              // 4096: one 64-column block of a tile
constexpr int kKvTileBytes = kQKBlocks * kKvBlockBytes;     // 36864
constexpr int kRawGroupBytes = 2688;                        // 4 rows: 4x256 | 4x256 | 4x144 (+pad to 128)
constexpr int kRawTileBytes = (kTileRows / 4) * kRawGroupBytes;  // 21504
constexpr int kRawTxBytes = kTileRows * kFp8RowBytes;       // bytes the three gathers deliver per tile

template <bool kFp8>
struct Cfg {
    static constexpr int kKvStages = kFp8 ? 1 : 2;
    static constexpr int kRawStages = kFp8 ? 2 : 0;
    static constexpr int kThreads = kFp8 ? 320 : 192;
    static constexpr int kOffKv = kQBytes;
    static constexpr int kOffRaw = kOffKv + kKvStages * kKvTileBytes;
    static constexpr int kOffCtl = kOffRaw + kRawStages * kRawTileBytes;
    static constexpr int kSmemBytes = kOffCtl + 1536 + 1024;  // control block + slack for 1024-byte alignment
};

// control block (after the tiles)
struct Ctl {
    float row_scale[2][kTileRows][4];  // fp8 cache: the four fp32 scales of every row of a tile
    uint64_t q_full, q_empty, o_free;
    uint64_t kv_full[2], kv_empty[2];
    uint64_t s_full[2], s_empty[2], p_full[2], pv_done[2];
    uint64_t raw_full[2], raw_empty[2];
    uint32_t tile_mask[4];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Ctl) <= 1536, "control block");

// TMEM columns.
//   bf16 cache: O [0,256) | S double-buffered 2 x 32 | P double-buffered 2 x 16 (packed bf16 pairs)
//   fp8 cache:  O [0,256) | five S accumulators of 32 columns (one per 128-value scale group of
//               the latent part, one for the rope part) | two P variants of 16 columns (P times
//               the scale of each of the two scale groups this CTA's output half covers)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0;
constexpr uint32_t kColS = 256;
template <bool kFp8> __host__ __device__ constexpr uint32_t col_p() { return kFp8 ? 256 + 5 * 32 : 256 + 2 * 32; }

// ------------------------------------------------------------------ index translation
// Top-k slot value -> physical cache row, or -1 when the slot is padding / unusable.
__device__ __forceinline__ int translate_row(int idx, int seq, const AttnParams& p) {
    if (idx < 0) return -1;
    long long row;
    if (p.block_table != nullptr) {
        const int blk = idx / p.page_block_size;
        if (blk >= p.block_table_stride) return -1;
        const int phys = __ldg(p.block_table + (size_t)seq * p.block_table_stride + blk);
        if (phys < 0) return -1;
        row = (long long)phys * p.page_block_size + (idx - blk * p.page_block_size);
    } else {
        row = (long long)seq * p.kv_batch_stride_rows + idx;
    }
    if (row < 0 || row >= p.num_kv_rows) return -1;
    return (int)row;
}

__global__ void debug_rows_kernel(AttnParams p, int total_q, int32_t* rows_out) {
    const long long n = (long long)total_q * p.topk;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i / p.topk);
        rows_out[i] = translate_row(__ldg(p.indices + i), q / p.s_q, p);
    }
}

// ------------------------------------------------------------------ the kernel
template <bool kFp8>
__global__ void __launch_bounds__(Cfg<kFp8>::kThreads, 1)
sparse_mla_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_kv_tail, const AttnParams p) {
    using C = Cfg<kFp8>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sKV = smem + C::kOffKv;
    uint8_t* sRaw = smem + C::kOffRaw;
    Ctl* ctl = reinterpret_cast<Ctl*>(smem + C::kOffCtl);
    volatile int* abort_flag = &ctl->abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int list = blockIdx.x >> 1;
    const int half = blockIdx.x & 1;  // which 256 output columns this CTA accumulates
    const int w_begin = __ldg(p.list_indptr + list);
    const int w_end = __ldg(p.list_indptr + list + 1);

    if (tid == 0) {
        mbar_init(smem_u32(&ctl->q_full), 1);
        mbar_init(smem_u32(&ctl->q_empty), 1);
        mbar_init(smem_u32(&ctl->o_free), 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctl->kv_full[i]), kFp8 ? 4 : 1);
            mbar_init(smem_u32(&ctl->kv_empty[i]), 1);
            mbar_init(smem_u32(&ctl->s_full[i]), 1);
            mbar_init(smem_u32(&ctl->s_empty[i]), 4);
            mbar_init(smem_u32(&ctl->p_full[i]), 4);
            mbar_init(smem_u32(&ctl->pv_done[i]), 1);
            mbar_init(smem_u32(&ctl->raw_full[i]), 1);
            mbar_init(smem_u32(&ctl->raw_empty[i]), 4);
        }
        ctl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_kv);
        if (kFp8) prefetch_tensormap(&tm_kv_tail);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 4) {
        // ============================================================ producer
        uint32_t it = 0;
        int item_n = 0;
        const int oob_row = (int)p.num_kv_rows;  // first row outside the tensor: the gather zero-fills it
        for (int w = w_begin; w < w_end; ++w, ++item_n) {
            const dsa_v32_work_info wi = p.works[w];
            const int seq = wi.q_row / p.s_q;
            if (!mbar_wait(smem_u32(&ctl->q_empty), (item_n & 1) ^ 1, abort_flag)) goto done;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&ctl->q_full);
                mbar_arrive_expect_tx(bar, kQBytes);
                for (int kb = 0; kb < kQKBlocks; ++kb)
                    tma_load_3d(smem_u32(sQ + kb * kQBlockBytes), &tm_q, bar, kb * 64, wi.head_block * kHeadsPerBlock,
                                wi.q_row);
            }
            const int32_t* idx_row = p.indices + (size_t)wi.q_row * p.topk;
            for (int k0 = wi.k_begin; k0 < wi.k_end; k0 += kTileRows, ++it) {
                const int k = k0 + lane;
                const int idx = (k < wi.k_end) ? __ldg(idx_row + k) : -1;
                const int row = translate_row(idx, seq, p);
                const uint32_t mask = __ballot_sync(0xffffffffu, row >= 0);
                const int coord = row >= 0 ? row : oob_row;
                const int g = lane & 7;
                const int r0 = __shfl_sync(0xffffffffu, coord, 4 * g + 0);
                const int r1 = __shfl_sync(0xffffffffu, coord, 4 * g + 1);
                const int r2 = __shfl_sync(0xffffffffu, coord, 4 * g + 2);
                const int r3 = __shfl_sync(0xffffffffu, coord, 4 * g + 3);
                if (!kFp8) {
                    const int s = it & 1;
                    if (!mbar_wait(smem_u32(&ctl->kv_empty[s]), ((it >> 1) & 1) ^ 1, abort_flag)) goto done;
                    const uint32_t bar = smem_u32(&ctl->kv_full[s]);
                    if (lane == 0) {
                        ctl->tile_mask[it & 3] = mask;
                        mbar_arrive_expect_tx(bar, kKvTileBytes);
                    }
                    __syncwarp();
                    if (lane < 8) {
                        const uint32_t dst = smem_u32(sKV + s * kKvTileBytes + g * 512);
                        for (int kb = 0; kb < kQKBlocks; ++kb)
                            tma_gather4(dst + kb * kKvBlockBytes, &tm_kv, bar, kb * 64, r0, r1, r2, r3);
                    }
                } else {
                    const int s = it & 1;
                    if (!mbar_wait(smem_u32(&ctl->raw_empty[s]), ((it >> 1) & 1) ^ 1, abort_flag)) goto done;
                    const uint32_t bar = smem_u32(&ctl->raw_full[s]);
                    if (lane == 0) {
                        ctl->tile_mask[it & 3] = mask;
                        mbar_arrive_expect_tx(bar, kRawTxBytes);
                    }
                    __syncwarp();
                    if (lane < 8) {
                        const uint32_t dst = smem_u32(sRaw + s * kRawTileBytes + g * kRawGroupBytes);
                        tma_gather4(dst, &tm_kv, bar, 0, r0, r1, r2, r3);
                        tma_gather4(dst + 1024, &tm_kv, bar, 256, r0, r1, r2, r3);
                        tma_gather4(dst + 2048, &tm_kv_tail, bar, 512, r0, r1, r2, r3);
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ============================================================ MMA issuer (one lane)
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_bf16(kHeadsPerBlock, kTileRows, false);
            constexpr uint32_t idesc_pv = make_idesc_bf16(kHeadsPerBlock, kDvHalf, true);
            constexpr uint32_t idesc_pv128 = make_idesc_bf16(kHeadsPerBlock, 128, true);
            constexpr int S = C::kKvStages;
            constexpr int SB = kFp8 ? 1 : 2;  // S / P buffers
            constexpr uint32_t kColP = col_p<kFp8>();
            uint32_t it_base = 0;
            int item_n = 0;
            bool ok = true;
            auto issue_qk = [&](uint32_t it, bool last_of_item) {
                const int s = it % S, sb = it % SB;
                if (!mbar_wait(smem_u32(&ctl->kv_full[s]), (it / S) & 1, abort_flag)) { ok = false; return; }
                if (!mbar_wait(smem_u32(&ctl->s_empty[sb]), ((it / SB) & 1) ^ 1, abort_flag)) { ok = false; return; }
                tc_fence_after();
                const uint32_t kv = smem_u32(sKV + s * kKvTileBytes);
                const uint32_t q = smem_u32(sQ);
#pragma unroll 4
                for (int ks = 0; ks < kDQK / 16; ++ks) {
                    const int kb = ks >> 2, kin = ks & 3;
                    const uint64_t a = make_smem_desc_sw128(q + kb * kQBlockBytes + kin * 32, 16, 1024);
                    const uint64_t b = make_smem_desc_sw128(kv + kb * kKvBlockBytes + kin * 32, 16, 1024);
                    if (kFp8) {
                        // one accumulator per 128-value scale group (two 64-column blocks), one for rope
                        umma_ss(tmem + kColS + (kb >> 1) * 32, a, b, idesc_qk, (ks & 7) ? 1u : 0u);
                    } else {
                        umma_ss(tmem + kColS + sb * 32, a, b, idesc_qk, ks > 0 ? 1u : 0u);
                    }
                }
                tc_commit(smem_u32(&ctl->s_full[sb]));
                if (last_of_item) tc_commit(smem_u32(&ctl->q_empty));
            };
            auto issue_pv = [&](uint32_t it, bool first_of_item) {
                const int s = it % S, sb = it % SB;
                if (!mbar_wait(smem_u32(&ctl->p_full[sb]), (it / SB) & 1, abort_flag)) { ok = false; return; }
                if (first_of_item && item_n > 0)
                    if (!mbar_wait(smem_u32(&ctl->o_free), (item_n - 1) & 1, abort_flag)) { ok = false; return; }
                tc_fence_after();
                const uint32_t v = smem_u32(sKV + s * kKvTileBytes + (4 * half) * kKvBlockBytes);
#pragma unroll
                for (int ks = 0; ks < kTileRows / 16; ++ks) {
                    const uint32_t acc = (first_of_item && ks == 0) ? 0u : 1u;
                    if (kFp8) {
                        // two 128-column halves, each with P pre-multiplied by its scale group
#pragma unroll
                        for (int v2 = 0; v2 < 2; ++v2) {
                            const uint64_t b = make_smem_desc_sw128(v + v2 * 2 * kKvBlockBytes + ks * 2048, kKvBlockBytes, 1024);
                            umma_ts(tmem + kColO + v2 * 128, tmem + kColP + v2 * 16 + ks * 8, b, idesc_pv128, acc);
                        }
                    } else {
                        const uint64_t b = make_smem_desc_sw128(v + ks * 2048, kKvBlockBytes, 1024);
                        umma_ts(tmem + kColO, tmem + kColP + sb * 16 + ks * 8, b, idesc_pv, acc);
                    }
                }
                tc_commit(smem_u32(&ctl->kv_empty[s]));
                tc_commit(smem_u32(&ctl->pv_done[it & 1]));
            };
            for (int w = w_begin; w < w_end && ok; ++w, ++item_n) {
                const dsa_v32_work_info wi = p.works[w];
                const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
                if (!mbar_wait(smem_u32(&ctl->q_full), item_n & 1, abort_flag)) { ok = false; break; }
                if (S > 1) issue_qk(it_base, n_tiles == 1);
                for (int t = 0; t < n_tiles && ok; ++t) {
                    if (S > 1) {
                        if (t + 1 < n_tiles) issue_qk(it_base + t + 1, t + 2 == n_tiles);
                    } else {
                        issue_qk(it_base + t, t + 1 == n_tiles);
                    }
                    if (ok) issue_pv(it_base + t, t == 0);
                }
                it_base += n_tiles;
            }
        }
        __syncwarp();
    } else if (warp < 4) {
        // ============================================================ softmax + epilogue
        constexpr int S = C::kKvStages;
        constexpr int SB = kFp8 ? 1 : 2;
        constexpr uint32_t kColP = col_p<kFp8>();
        const int row = tid;  // head row inside the block == TMEM lane
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        uint32_t it = 0;
        for (int w = w_begin; w < w_end; ++w) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            float m_ref = -INFINITY;  // running reference maximum, log2 domain
            float l = 0.0f;
            for (int t = 0; t < n_tiles; ++t, ++it) {
                const int sb = it % SB;
                if (!mbar_wait(smem_u32(&ctl->kv_full[it % S]), (it / S) & 1, abort_flag)) goto done;
                const uint32_t mask = ctl->tile_mask[it & 3];
                if (!mbar_wait(smem_u32(&ctl->s_full[sb]), (it / SB) & 1, abort_flag)) goto done;
                tc_fence_after();
                float tv[32];
                if (kFp8) {
                    // s = sum_g scale[row][g] * S_g + S_rope : the cache values went through the MMA
                    // unscaled (e4m3 is exact in bf16), so nothing is rounded before this point
                    uint32_t sr[32];
                    tmem_ld32(lane_base + kColS + 4 * 32, sr);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) tv[j] = __uint_as_float(sr[j]);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        tmem_ld32(lane_base + kColS + g * 32, sr);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) tv[j] = fmaf(ctl->row_scale[it & 1][j][g], __uint_as_float(sr[j]), tv[j]);
                    }
                } else {
                    uint32_t sr[32];
                    tmem_ld32(lane_base + kColS + sb * 32, sr);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) tv[j] = __uint_as_float(sr[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[sb]));

                float mt = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float x = tv[j] * p.scale_log2;
                    tv[j] = ((mask >> j) & 1u) ? x : -INFINITY;
                    mt = fmaxf(mt, tv[j]);
                }
                // lazy rescale: move the reference maximum only when a row outgrows it by more than 8
                const bool need = mt > m_ref + 8.0f;
                if (__any_sync(0xffffffffu, need)) {
                    const float m_new = need ? mt : m_ref;
                    if (t > 0) {
                        const float f = (m_ref == -INFINITY) ? 0.0f : ex2_approx(m_ref - m_new);
                        l *= f;
                        // O of this item so far is complete once the previous PV has finished
                        const uint32_t pit = it - 1;
                        if (!mbar_wait(smem_u32(&ctl->pv_done[pit & 1]), (pit >> 1) & 1, abort_flag)) goto done;
                        tc_fence_after();
#pragma unroll 1
                        for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
                            uint32_t o[32];
                            tmem_ld32(lane_base + kColO + c0, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
                            tmem_st32(lane_base + kColO + c0, o);
                        }
                        tmem_wait_st();
                    }
                    m_ref = m_new;
                }
                const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
                float lsum = 0.0f;
                if (kFp8) {
                    uint32_t pk0[16], pk1[16];
                    const int g0 = 2 * half;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float p0 = ex2_approx(tv[2 * j] - m_use);
                        const float p1 = ex2_approx(tv[2 * j + 1] - m_use);
                        lsum += p0 + p1;
                        const float* sc0 = ctl->row_scale[it & 1][2 * j];
                        const float* sc1 = ctl->row_scale[it & 1][2 * j + 1];
                        pk0[j] = pack_bf16x2(p0 * sc0[g0], p1 * sc1[g0]);
                        pk1[j] = pack_bf16x2(p0 * sc0[g0 + 1], p1 * sc1[g0 + 1]);
                    }
                    tmem_st16(lane_base + kColP, pk0);
                    tmem_st16(lane_base + kColP + 16, pk1);
                } else {
                    uint32_t pk[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float p0 = ex2_approx(tv[2 * j] - m_use);
                        const float p1 = ex2_approx(tv[2 * j + 1] - m_use);
                        lsum += p0 + p1;
                        pk[j] = pack_bf16x2(p0, p1);
                    }
                    tmem_st16(lane_base + kColP + sb * 16, pk);
                }
                l += lsum;
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[sb]));
            }
            // ---- epilogue of the item
            {
                const uint32_t pit = it - 1;
                if (!mbar_wait(smem_u32(&ctl->pv_done[pit & 1]), (pit >> 1) & 1, abort_flag)) goto done;
                tc_fence_after();
                const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
                const int head = wi.head_block * kHeadsPerBlock + row;
                const bool live = head < p.H;
                const float lse_nat = (l > 0.0f) ? (m_ref + __log2f(l)) * 0.69314718055994531f : INFINITY;
                if (wi.partial_slot < 0) {
                    __nv_bfloat16* o_dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)wi.q_row * p.stride_o_row +
                                           (size_t)head * p.stride_o_head + half * kDvHalf;
#pragma unroll 1
                    for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + c0, o);
                        tmem_wait_ld();
                        if (live) {
                            uint4* d4 = reinterpret_cast<uint4*>(o_dst + c0);
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 u;
                                u.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                                u.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                                u.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                                u.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                                d4[v] = u;
                            }
                        }
                    }
                    if (live && half == 0 && p.lse != nullptr) p.lse[(size_t)wi.q_row * p.H + head] = lse_nat;
                } else {
                    float* o_dst = p.o_accum + ((size_t)wi.partial_slot * kHeadsPerBlock + row) * kDV + half * kDvHalf;
#pragma unroll 1
                    for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + c0, o);
                        tmem_wait_ld();
                        float4* d4 = reinterpret_cast<float4*>(o_dst + c0);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            d4[v] = make_float4(__uint_as_float(o[4 * v + 0]) * inv, __uint_as_float(o[4 * v + 1]) * inv,
                                                __uint_as_float(o[4 * v + 2]) * inv, __uint_as_float(o[4 * v + 3]) * inv);
                    }
                    if (half == 0)
                        p.lse_accum[(size_t)wi.partial_slot * kHeadsPerBlock + row] = (l > 0.0f) ? lse_nat : -FLT_MAX;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->o_free));
            }
        }
    } else if (kFp8) {
        // ============================================================ dequantise (warps 6-9)
        const int dt = tid - 192;        // 0..127
        const int r = dt >> 2;           // tile row 0..31
        const int qd = dt & 3;           // which 128-value scale group of the row
        const int dwarp_lane0 = (lane == 0);
        uint32_t it = 0;
        for (int w = w_begin; w < w_end; ++w) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            for (int t = 0; t < n_tiles; ++t, ++it) {
                const int rs = it & 1;
                if (!mbar_wait(smem_u32(&ctl->raw_full[rs]), (it >> 1) & 1, abort_flag)) goto done;
                if (!mbar_wait(smem_u32(&ctl->kv_empty[0]), (it & 1) ^ 1, abort_flag)) goto done;
                const uint8_t* grp = sRaw + rs * kRawTileBytes + (r >> 2) * kRawGroupBytes;
                const int ri = r & 3;
                const uint8_t* src = grp + (qd >> 1) * 1024 + ri * 256 + (qd & 1) * 128;
                const uint8_t* tail = grp + 2048 + ri * 144;
                // values go to the MMA unscaled (every e4m3 value is exact in bf16); the row's scales
                // are applied to the fp32 scores and to P by the softmax warps
                ctl->row_scale[it & 1][r][qd] = reinterpret_cast<const float*>(tail)[qd];
                uint8_t* dst_row = sKV + r * 128;
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const int c = (cc + r) & 7;  // rotate so the 8 rows of a warp hit different banks
                    const uint4 raw = *reinterpret_cast<const uint4*>(src + c * 16);
                    const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
                    uint32_t o[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t h01, h23;
                        const uint16_t lo16 = (uint16_t)(wv[k] & 0xFFFFu), hi16 = (uint16_t)(wv[k] >> 16);
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"(lo16));
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"(hi16));
                        const __half2 a = *reinterpret_cast<const __half2*>(&h01);
                        const __half2 b = *reinterpret_cast<const __half2*>(&h23);
                        const float2 fa = __half22float2(a), fb = __half22float2(b);
                        o[2 * k + 0] = pack_bf16x2(fa.x, fa.y);
                        o[2 * k + 1] = pack_bf16x2(fb.x, fb.y);
                    }
                    // 16 fp8 -> 16 bf16 = two 16-byte chunks of the 64-column block (2*qd + c/4)
                    const int kb = 2 * qd + (c >> 2);
                    const int ch = (c & 3) * 2;
                    uint8_t* d = dst_row + kb * kKvBlockBytes;
                    *reinterpret_cast<uint4*>(d + (((ch + 0) ^ (r & 7)) * 16)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(d + (((ch + 1) ^ (r & 7)) * 16)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                // rope: 64 bf16 = 8 chunks; this thread copies chunks 2*qd, 2*qd+1 into block 8
                {
                    const uint4 a = *reinterpret_cast<const uint4*>(tail + 16 + (2 * qd + 0) * 16);
                    const uint4 b = *reinterpret_cast<const uint4*>(tail + 16 + (2 * qd + 1) * 16);
                    uint8_t* d = dst_row + 8 * kKvBlockBytes;
                    *reinterpret_cast<uint4*>(d + (((2 * qd + 0) ^ (r & 7)) * 16)) = a;
                    *reinterpret_cast<uint4*>(d + (((2 * qd + 1) ^ (r & 7)) * 16)) = b;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (dwarp_lane0) {
                    mbar_arrive(smem_u32(&ctl->kv_full[0]));
                    mbar_arrive(smem_u32(&ctl->raw_empty[rs]));
                }
            }
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ctl->abort_flag) atomicExch(p.status, DSA_V32_ERR_DEVICE_WAIT);
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ------------------------------------------------------------------ split merge
// One warp per (reduce row, head).  Same arithmetic as the reference's two-pass merge
// (opus_attn/dsa_v32/common/mla_reduce.hpp:92-156): m = max lse_i, w_i = exp2((lse_i - m) log2e)
// (0 for an empty split), out = sum w_i O_i / sum w_i, lse = m + ln(sum w_i); all empty -> 0, +inf.
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ o_accum, const float* __restrict__ lse_accum,
                                                      const int32_t* __restrict__ reduce_indptr,
                                                      const int32_t* __restrict__ reduce_slots,
                                                      const ReduceDst* __restrict__ reduce_dst, void* out, float* lse,
                                                      int64_t stride_o_row, int64_t stride_o_head, int H) {
    const int rr = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hrow = blockIdx.y * 8 + warp;  // head inside the 128-head block
    const ReduceDst dst = reduce_dst[rr];
    const int head = dst.head_block * kHeadsPerBlock + hrow;
    if (head >= H) return;
    const int s0 = reduce_indptr[rr], ns = reduce_indptr[rr + 1] - s0;
    float m = -FLT_MAX;
    for (int i = lane; i < ns; i += 32) m = fmaxf(m, lse_accum[(size_t)reduce_slots[s0 + i] * kHeadsPerBlock + hrow]);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
    float denom = 0.0f;
    for (int i = 0; i < ns; ++i) {
        const int slot = reduce_slots[s0 + i];
        const float li = lse_accum[(size_t)slot * kHeadsPerBlock + hrow];
        const float wgt = (li > -FLT_MAX) ? exp2f((li - m) * 1.4426950408889634f) : 0.0f;
        denom += wgt;
        const float4* src = reinterpret_cast<const float4*>(o_accum + ((size_t)slot * kHeadsPerBlock + hrow) * kDV);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const float4 x = src[v * 32 + lane];
            acc[4 * v + 0] += wgt * x.x;
            acc[4 * v + 1] += wgt * x.y;
            acc[4 * v + 2] += wgt * x.z;
            acc[4 * v + 3] += wgt * x.w;
        }
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)dst.q_row * stride_o_row + (size_t)head * stride_o_head;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        uint2 u;
        u.x = pack_bf16x2(acc[4 * v + 0] * inv, acc[4 * v + 1] * inv);
        u.y = pack_bf16x2(acc[4 * v + 2] * inv, acc[4 * v + 3] * inv);
        *reinterpret_cast<uint2*>(o + (v * 32 + lane) * 4) = u;
    }
    if (lane == 0 && lse != nullptr)
        lse[(size_t)dst.q_row * H + head] = denom > 0.0f ? m + log2f(denom) * 0.69314718055994531f : INFINITY;
}

// ------------------------------------------------------------------ cache write path
// One warp per row: per 128 values amax -> scale = amax / 448, e4m3(x / scale) with RNE and
// saturation (cvt.rn.satfinite), scales and rope appended.
__global__ void __launch_bounds__(256) pack_fp8_rows_kernel(const float* __restrict__ latent,
                                                            const __nv_bfloat16* __restrict__ rope,
                                                            const int64_t* __restrict__ dst_rows, uint8_t* __restrict__ out,
                                                            int64_t num_rows) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    const int64_t dr = dst_rows ? dst_rows[r] : r;
    uint8_t* row = out + dr * kFp8RowBytes;
    const float* x = latent + r * kDV;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const float4 v = reinterpret_cast<const float4*>(x + g * 128)[lane];
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float scale = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
        const float a = __fdiv_rn(v.x, scale), b = __fdiv_rn(v.y, scale), c = __fdiv_rn(v.z, scale), d = __fdiv_rn(v.w, scale);
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
        reinterpret_cast<uint32_t*>(row + g * 128)[lane] = (uint32_t)lo | ((uint32_t)hi << 16);
        if (lane == 0) reinterpret_cast<float*>(row + kDV)[g] = scale;
    }
    reinterpret_cast<uint32_t*>(row + kDV + 16)[lane] = reinterpret_cast<const uint32_t*>(rope + r * kDRope)[lane];
}

// ------------------------------------------------------------------ launch helpers (called from capi.cu)
int smem_bytes_attn(bool fp8) { return fp8 ? Cfg<true>::kSmemBytes : Cfg<false>::kSmemBytes; }

cudaError_t launch_attn(bool fp8, int num_lists, const CUtensorMap& tq, const CUtensorMap& tkv, const CUtensorMap& ttail,
                        const AttnParams& p, cudaStream_t stream) {
    static bool configured[2] = {false, false};
    cudaError_t e;
    if (fp8) {
        if (!configured[1]) {
            e = cudaFuncSetAttribute(sparse_mla_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true>::kSmemBytes);
            if (e != cudaSuccess) return e;
            configured[1] = true;
        }
        sparse_mla_kernel<true><<<2 * num_lists, Cfg<true>::kThreads, Cfg<true>::kSmemBytes, stream>>>(tq, tkv, ttail, p);
    } else {
        if (!configured[0]) {
            e = cudaFuncSetAttribute(sparse_mla_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false>::kSmemBytes);
            if (e != cudaSuccess) return e;
            configured[0] = true;
        }
        sparse_mla_kernel<false><<<2 * num_lists, Cfg<false>::kThreads, Cfg<false>::kSmemBytes, stream>>>(tq, tkv, ttail, p);
    }
    return cudaGetLastError();
}

cudaError_t launch_combine(const float* o_accum, const float* lse_accum, const int32_t* reduce_indptr,
                           const int32_t* reduce_slots, const ReduceDst* reduce_dst, int num_reduce_rows, void* out, float* lse,
                           int64_t stride_o_row, int64_t stride_o_head, int H, cudaStream_t stream) {
    if (num_reduce_rows <= 0) return cudaSuccess;
    dim3 grid(num_reduce_rows, kHeadsPerBlock / 8);
    combine_kernel<<<grid, 256, 0, stream>>>(o_accum, lse_accum, reduce_indptr, reduce_slots, reduce_dst, out, lse,
                                             stride_o_row, stride_o_head, H);
    return cudaGetLastError();
}

cudaError_t launch_debug_rows(const AttnParams& p, int total_q, int32_t* rows_out, cudaStream_t stream) {
    debug_rows_kernel<<<256, 256, 0, stream>>>(p, total_q, rows_out);
    return cudaGetLastError();
}

cudaError_t launch_pack_fp8(const float* latent, const void* rope, const int64_t* dst_rows, void* out, int64_t num_rows,
                            cudaStream_t stream) {
    if (num_rows <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((num_rows + 7) / 8);
    pack_fp8_rows_kernel<<<blocks, 256, 0, stream>>>(latent, reinterpret_cast<const __nv_bfloat16*>(rope), dst_rows,
                                                     reinterpret_cast<uint8_t*>(out), num_rows);
    return cudaGetLastError();
}

}  // namespace dsa
