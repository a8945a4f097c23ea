// Sparse MLA attention for sm_100a: decode (split over the top-k list) and prefill share one
// warp-specialised kernel run by clusters of two CTAs.
//
// What it computes is the reference lab's decode kernel family
// (opus_attn/dsa_v32/gfx950/mla_decode_a16w16_16mx4_64nx1_template.hpp:815-926 and the mxfp8
// variant mla_decode_mxfp8_16mx8_32nx1_template.hpp:1362-1490): for one work item = one query
// row x one block of 128 heads x a slice of the query's top-k list, an online-softmax attention
// over the gathered latent rows, K = all 576 columns of a row, V = its first 512 columns.
// How it does it is specific to Blackwell.
//
// The 128 x 512 fp32 output would fill all 512 TMEM columns, so two CTAs (a cluster) share a work
// item and split the 576 columns of the latent row between them:
//       fp8 cache:   CTA 0: columns [0, 256)                 CTA 1: columns [256, 512) + the 64 rope columns
//       bf16 cache:  CTA 0: [0, 256) + rope columns [0, 32)  CTA 1: [256, 512) + rope columns [32, 64)
// (a bf16 row can be cut anywhere, so both CTAs get four and a half 64-column blocks and neither waits for
// the other's partial scores; an fp8 row is gathered in one contiguous piece per CTA).
// Each CTA loads only its columns of Q, gathers only its columns of every selected row, computes
// the partial scores Q_c K_c^T over its columns and owns the 256 output columns that are the
// first 256 of its slice (V is a prefix of K), so no byte of the cache is fetched or converted
// twice.  The partial scores have to be summed across the pair through distributed shared memory,
// and the link between two SMs is narrow (measured: 17-20 bytes per clock one way, 11-16 each way
// when both send), so what crosses it is kept small: partial scores as 16-bit fixed point with a
// per-row step instead of fp32, and
//   bf16 cache: the softmax itself is split by head rows - CTA c computes it for rows [64 c, 64 c + 64),
//              receives the peer's partial scores for those rows and sends the finished P (bf16) and the
//              rare rescale factor back: 8.7 KB per 32-row tile and direction, half the exponentials;
//   fp8 cache:  both CTAs run the softmax of all 128 rows on the same (quantised) sums - the single score
//              buffer in TMEM and the four tile stages make the latency of a tile's chain the bound
//              there, and the row split would add a second hop to it.
//
// Warp roles inside a CTA (28 warps = seven warpgroups; after the role split setmaxnreg gives the four
// softmax warpgroups 88 registers per thread and the others 48 for a bf16 cache, 96 and 40 for an fp8 cache):
//   warps 0-15  softmax, as four teams of four warps (one per TMEM lane quadrant) that take the 32-slot
//              tiles round robin; thread = head row, holding its row's 32 scores of the tile: tcgen05.ld
//              of the partial scores, exchange with the peer CTA, row maximum; then the only ordered
//              step - the row's reference maximum in shared memory is read and moved when the tile's
//              maximum exceeds it by more than the lazy margin (the reference's threshold of 8:
//              ..16mx4_64nx1_template.hpp:700-725); P = 2^(s - reference) -> bf16 -> tcgen05.st.
//              Epilogue: O / l -> bf16 (to out, or to every peer GPU's gathered buffer when the all-gather
//              is fused), or the fp32 partial + lse of a split item; during its waits the next item's Q
//              slice is stored into TMEM (A operand of the score MMAs).
//   warp 16    score MMA issuer: S_c = Q_c K_c^T (tcgen05.mma M=128, N=32, K=16, A = the Q slice in TMEM,
//              accumulator in TMEM; fp8 cache: the 64 rope columns of Q stay in shared memory)
//   warp 17    P V MMA issuer: O_c += P V_c (A = P in TMEM, B = the same gathered tile described
//              MN-major).  Two issuers so that neither stream waits behind the other's barriers.
//   bf16 cache: warp 18 second score issuer (alternate tiles), warp 19 asks the next item's Q into L2 near the end of
//              an item; warps 20-27 loaders, two groups of four on alternate tiles, 8 rows of the tile per warp:
//              top-k slots -> block table -> the row's bytes of this CTA's slice as 16-byte cp.async copies
//              straight into the 128-byte swizzled MMA tile (a TMA tile::gather4 moves one 128-byte block
//              of four rows per request, 40 requests per tile, and the issue rate of those requests was
//              the period of the whole pipeline)
//   fp8 cache: warps 18-19 gather issuers on alternate tiles (lane = row; one TMA tile::gather4 per four
//              rows, the row's two scales by cp.async), warps 20-27 converters, four rows of every tile
//              each (all eight on one tile: the time a tile holds its stage is what bounds the pipeline):
//              e4m3 -> bf16 exactly (e4m3 has 4 significant bits) into the swizzled MMA
//              tile (the reference's LDS round trip: ..mxfp8_16mx8_32nx1_template.hpp:852-864).  The
//              per-128 fp32 scales never touch the operands: Q K^T keeps one fp32 accumulator per scale
//              group (plus one for rope) and the softmax warps form sum_g scale_g S_g in fp32 before the
//              exchange; for P V they store one copy of P per scale group, pre-multiplied by that group's
//              scale, and each copy multiplies its own 128 output columns.
//
// A work item may stack the query rows of one sequence that share an index list (MTP) along the heads
// when they fit the 128-row tile together: tile row r = query row q_row + r / H, head r % H.
//
// Every mbarrier wait is bounded; on expiry the CTA raises its own and its peer's abort flag,
// records DSA_V32_ERR_DEVICE_WAIT in the workspace status word and both drain to the normal exit
// (cluster barrier, TMEM release).  A parity wait is only issued on a barrier whose previous phase the
// waiting warp knows to be complete (rings it takes part in, or per-item barriers).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include <mutex>
#include "defs.h"
#include "ptx.cuh"

// Tile stages.  The period of the pipeline is (how long a tile occupies its stage) / (stages), so more stages are
// faster - until the CTA's shared memory no longer fits the 196 KB carve-out of the SM's 256 KB L1/shared array:
// the next carve-out leaves 28 instead of 60 KB of L1 and costs 5-10 % (measured).  fp8: 4 + 4 raw stages fill
// the 196 KB exactly; bf16: 7 stages are 188 KB (8 measured slower than 6).
#ifndef DSA_FP8_KV_STAGES
#define DSA_FP8_KV_STAGES 4
#endif
#ifndef DSA_BF16_KV_STAGES
#define DSA_BF16_KV_STAGES 7
#endif
#ifndef DSA_ROWSPLIT_FP8
#define DSA_ROWSPLIT_FP8 0
#endif
#ifndef DSA_ROWSPLIT_BF16
#define DSA_ROWSPLIT_BF16 1
#endif
#ifndef DSA_FP8_RAW_STAGES
#define DSA_FP8_RAW_STAGES 4
#endif

namespace dsa {



// ------------------------------------------------------------------ shared-memory map
constexpr int kMaxKBlocks = 5;                            // 64-column blocks per CTA: 4 (CTA 0) or 5 (CTA 1)
constexpr int kQBlockBytes = kHeadsPerBlock * 128;        // 16384
constexpr int kKvBlockBytes = kTileRows * 128;            // 4096: one 64-column block of a 32-row tile
constexpr int kKvTileBytes = kMaxKBlocks * kKvBlockBytes; // 20480
constexpr int kRawGroupBytes = 1024 + 640;                // 4 rows: 4 x 256 latent bytes | 4 x 144 tail (+pad)
constexpr int kRawTileBytes = (kTileRows / 4) * kRawGroupBytes;   // 13312
constexpr int kXWarpBytes = 32 * (kTileRows * 2 + 4);             // 2176: per softmax warp, a tile row's 32 values as 16-bit words (partial
                                                                  // scores in fixed point, or P in bf16) + one fp32 word per row
constexpr int kXbufBytes = 4 * kXWarpBytes;                       // 8704: the four warps of a team
constexpr float kQuantBias = 8421376.0f;                          // 2^23 + 2^15: adding it leaves round(x) + 32768 in the low mantissa bits
constexpr int kMaskSlots = 16;
constexpr int kGroups = 4;                                // softmax warpgroups sharing a tile's columns
constexpr int kSoftmaxWarps = 4 * kGroups;
constexpr int kMmaWarp = kSoftmaxWarps;                   // issues the score MMAs (and owns the TMEM allocation)
constexpr int kGatherWarp0 = kSoftmaxWarps + 2;           // fp8 cache: two gather issuers (idle for a bf16 cache) ...
constexpr int kGatherWarps = 2;
constexpr int kConvertWarp0 = kGatherWarp0 + kGatherWarps; // ... and eight converters (two warpgroups)
constexpr int kConvertWarps = 8;
constexpr int kLoaderWarp0 = kConvertWarp0;               // bf16 cache: eight loader warps, two groups of four
constexpr int kLoaderWarps = 8;
constexpr int kWarps = kConvertWarp0 + kConvertWarps;     // 28: seven warpgroups
// Registers per thread after the role split (setmaxnreg, per warpgroup): the softmax warpgroups hold a
// tile row in registers, everything else is light.  bf16 cache: 4 x 128 x 88 + 3 x 128 x 48 = 63 488;
// fp8 cache (scales, two copies of P): 4 x 128 x 96 + 3 x 128 x 40 = 64 512; both <= 65 536.
template <bool kFp8> constexpr int kRegsSoftmax = kFp8 ? 96 : 88;
template <bool kFp8> constexpr int kRegsOther = kFp8 ? 40 : 48;
constexpr int kScaleSlots = 16;                           // tiles whose row scales are kept (raw ring + tile ring <= 16)

template <bool kFp8>
struct Cfg {
    // The Q slice lives in TMEM (A operand of the score MMAs), written there by the softmax warps straight
    // from global memory.  Only the rope block of an fp8 item stays in shared memory (TMEM is full).
    static constexpr bool kQInTmem = true;
    static constexpr int kQSmemBytes = kFp8 ? kQBlockBytes : 0;
    static constexpr int kKvStages = kFp8 ? DSA_FP8_KV_STAGES : DSA_BF16_KV_STAGES;   // MMA-ready bf16 tiles
    static constexpr int kRawStages = kFp8 ? DSA_FP8_RAW_STAGES : 0; // raw fp8 tiles in flight
    // The raw ring must have an even number of buffers: a buffer is then always filled by the same issuer
    // warp, so a warp that waits for it to come back is never more than one phase ahead of its barrier (with
    // an odd ring the two issuers alternate on a buffer and a parity wait could pass on the phase before last).
    static_assert(!kFp8 || kRawStages % 2 == 0, "even raw ring");
    static_assert(kKvStages <= 8 && kRawStages <= 16, "kv_full/kv_empty hold 8 barriers, raw_full/raw_empty 16");
    static_assert(kKvStages + kRawStages <= kScaleSlots && kKvStages + kRawStages <= kMaskSlots,
                  "a tile's mask and scales stay in their slot from the gather to the softmax");
    static constexpr int kThreads = 32 * kWarps;
    static constexpr int kOffKv = kQSmemBytes;
    static constexpr int kOffRaw = kOffKv + kKvStages * kKvTileBytes;
    static constexpr int kOffX = kOffRaw + kRawStages * kRawTileBytes;
    static constexpr int kOffCtl = kOffX + kGroups * kXbufBytes;   // one exchange buffer per softmax team
    static constexpr int kCtlBytes = 12288;
    static constexpr int kSmemBytes = kOffCtl + kCtlBytes + 1024;  // + slack for 1024-byte alignment
};

struct Ctl {
    float l_part[2][kGroups][kHeadsPerBlock];   // per-team row sums at the end of an item, by item parity
    float row_scale[kScaleSlots][2][kTileRows];  // fp8 cache: per tile buffer, the scales of this CTA's two groups for every tile row
    uint64_t q_full, q_empty, o_free;
    uint64_t kv_full[8], kv_empty[8];
    uint64_t raw_full[16];   // fp8 cache, per raw buffer: the tile's rows and their scales have landed
    uint64_t raw_empty[16];  // ... and the four converter warps that read them are done
    uint64_t s_full[kGroups], s_empty[kGroups], p_full[kGroups], pv_done[kGroups];
    uint64_t l_bar;
    uint64_t e_bar;    // every softmax warp has committed its last tile of the item (its P stores and reference-maximum steps)
    uint64_t o_full;   // the item's last P V product has completed: O is final
    uint64_t m_bar[kGroups][4];        // [team][lane quadrant]: the tile's reference-maximum step is done
    // Exchange of partial scores with the peer CTA: one buffer per team, barriers per softmax warp.
    uint64_t x_full[kSoftmaxWarps];    // the peer's partial scores for this warp's rows have arrived (bytes)
    uint64_t x_free[kSoftmaxWarps];    // credit (4 bytes): the peer's same warp has read what this warp sent
    uint32_t x_sink[kSoftmaxWarps];    // where the credit word lands
    float m_shared[kHeadsPerBlock];    // reference maximum of every row, moved only at a tile's commit
    uint32_t tile_mask[kMaskSlots];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Ctl) <= 12288 - 256, "control block");

// TMEM columns (512 allocated).
//   bf16 cache: O [0,256) | Q slice [256,416) (packed bf16 pairs: 128 latent + 16 rope columns used) | S 2 x 32 | P 2 x 16
//   fp8 cache:  O [0,256) | latent Q slice [256,384) | one score buffer of 3 accumulators x 32 (scale
//               group a, scale group b, rope) | one P buffer of 2 variants x 16.  Single buffers: the
//               scores are drained into registers right after they complete, and P is rewritten right
//               after the product that read it.
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0;
constexpr uint32_t kColQ = 256;
template <bool kFp8> __host__ __device__ constexpr uint32_t col_s() { return kFp8 ? 384 : 416; }
template <bool kFp8> __host__ __device__ constexpr uint32_t col_p() { return 480; }
// The per-tile barriers (s_full, s_empty, p_full, pv_done) come in fours indexed by the softmax team that
// works on the tile (tile number mod 4), also where the TMEM buffer behind them is single or double: a
// team that runs ahead must not take another team's completion for its own.
template <bool kFp8> __device__ __forceinline__ uint32_t buf_of(uint32_t it) { return it & (kGroups - 1u); }
template <bool kFp8> __device__ __forceinline__ uint32_t phase_of(uint32_t it) { return (it / kGroups) & 1u; }
template <bool kFp8> constexpr uint32_t kBufReuse = kFp8 ? 1u : 2u;   // tiles between two uses of a score / P buffer
template <bool kFp8> __device__ __forceinline__ uint32_t s_col_of(uint32_t it) { return col_s<kFp8>() + (kFp8 ? 0u : (it & 1u) * 32u); }
template <bool kFp8> __device__ __forceinline__ uint32_t p_col_of(uint32_t it) { return col_p<kFp8>() + (kFp8 ? 0u : (it & 1u) * 16u); }

// ------------------------------------------------------------------ index translation
// Top-k slot value -> physical cache row, or -1 when the slot is padding / unusable.  Split in two so
// the loader warps can issue the block-table load of one tile and finish the arithmetic tiles later:
//   block_of(idx)        issues the block-table load (0 when there is nothing to load)
//   row_of(idx, phys)    the physical row from the loaded block number
__device__ __forceinline__ int block_of(int idx, int seq, const AttnParams& p) {
    if (idx < 0 || p.block_table == nullptr) return 0;
    const int blk = p.page_shift >= 0 ? (idx >> p.page_shift) : idx / p.page_block_size;
    if (blk >= p.block_table_stride) return -1;
    return __ldg(p.block_table + (size_t)seq * p.block_table_stride + blk);
}
__device__ __forceinline__ int row_of(int idx, int phys, int seq, const AttnParams& p) {
    if (idx < 0) return -1;
    long long row;
    if (p.block_table != nullptr) {
        if (phys < 0) return -1;
        const int in_page = p.page_shift >= 0 ? (idx & (p.page_block_size - 1)) : idx % p.page_block_size;
        row = (long long)phys * p.page_block_size + in_page;
    } else {
        row = (long long)seq * p.kv_batch_stride_rows + idx;
    }
    if (row < 0 || row >= p.num_kv_rows) return -1;
    return (int)row;
}
__device__ __forceinline__ int translate_row(int idx, int seq, const AttnParams& p) {
    return row_of(idx, block_of(idx, seq, p), seq, p);
}

__global__ void debug_rows_kernel(AttnParams p, int total_q, int32_t* rows_out) {
    const long long n = (long long)total_q * p.topk;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(i / p.topk);
        rows_out[i] = translate_row(__ldg(p.indices + i), q / p.s_q, p);
    }
}

// ------------------------------------------------------------------ tile row -> (query row, head)
// Tile row r of a work item is head head_block * 128 + r of query row q_row, or, for an item that stacks
// the query rows of one sequence that share an index list, head r % H of query row q_row + r / H.
struct RowMap {
    int q_row, head;
    bool live;
};
template <bool kExt>
__device__ __forceinline__ RowMap map_row(const dsa_v32_work_info& w, int row, int H) {
    RowMap m;
    if (w.stacked_rows > 1) {
        const int sub = row / H;
        m.q_row = w.q_row + sub;
        m.head = row - sub * H;
        m.live = sub < w.stacked_rows;
    } else {
        m.q_row = w.q_row;
        m.head = w.head_block * kHeadsPerBlock + row;
        m.live = m.head < H;
    }
    return m;
}

// ------------------------------------------------------------------ e4m3 -> bf16, exact, two at a time
// Input: the two e4m3 bytes in the high byte of each 16-bit half.  Moving the 7 magnitude bits down
// by 4 puts the 4 exponent bits and 3 mantissa bits where bf16 keeps them; read as bf16 that number
// is the e4m3 value times 2^-120 (normal and subnormal codes alike), so one exact multiply by 2^120
// finishes the conversion without going through the conversion unit.  (0x7F, the e4m3 NaN, becomes
// 480 instead of NaN; a cache row that is never selected is never converted.)
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t hi_bytes) {
    const uint32_t y = (hi_bytes & 0x80008000u) | ((hi_bytes >> 4) & 0x07F007F0u);
    uint32_t z;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(z) : "r"(y), "r"(0x7B807B80u));
    return z;
}

// ------------------------------------------------------------------ MMA issue (whole warp converged)
// S_c (+)= Q_c K_c^T for one 32-row tile: NKB blocks of 64 columns, four K=16 steps each.  With an fp8
// cache every scale group (two blocks) and the rope block get their own accumulator.
template <bool kFp8, int NKB>
__device__ __forceinline__ void issue_qk_mmas(uint32_t d0, uint64_t q_rope_desc, uint32_t q_tmem, uint64_t k_desc, uint32_t el) {
    constexpr uint32_t idesc = make_idesc_bf16(kHeadsPerBlock, kTileRows, false);
    const uint32_t k_lo = static_cast<uint32_t>(k_desc), k_hi = static_cast<uint32_t>(k_desc >> 32);
#pragma unroll
    for (int kb = 0; kb < NKB; ++kb) {
        const uint32_t b_lo = k_lo + static_cast<uint32_t>((kb * kKvBlockBytes) >> 4);
        if (!kFp8)   // A = Q from TMEM, one accumulator
            umma_ts_x4_el(d0, q_tmem + kb * 32, b_lo, k_hi, idesc, kb ? 1u : 0u, el);
        else if (kb < 4)   // one accumulator per scale group (two blocks)
            umma_ts_x4_el(d0 + (kb >> 1) * 32, q_tmem + kb * 32, b_lo, k_hi, idesc, (kb & 1) ? 1u : 0u, el);
        else   // rope block of an fp8 item: A from shared memory, its own accumulator
            umma_ss_x4_el(d0 + 64, static_cast<uint32_t>(q_rope_desc), static_cast<uint32_t>(q_rope_desc >> 32), b_lo, k_hi,
                          idesc, 0u, el);
    }
    if (!kFp8) {
        // bf16 cache: this CTA's half of the rope columns, the first two K steps of block 4 (A: TMEM columns 128-143 of the slice)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
            umma_ts_el(d0, q_tmem + 128 + ks * 8, k_desc + static_cast<uint64_t>(((4 * kKvBlockBytes) >> 4) + ks * 2), idesc, 1u, el);
    }
}

// O_c (+)= P V_c for one 32-row tile: two K=16 steps; V_c is the first 256 columns of the tile seen
// MN-major.  fp8 cache: two scaled copies of P, each for its own 128 output columns.
template <bool kFp8>
__device__ __forceinline__ void issue_pv_mmas(uint32_t o_tmem, uint32_t p_tmem, uint64_t v_desc, bool overwrite, uint32_t el) {
    constexpr uint32_t idesc256 = make_idesc_bf16(kHeadsPerBlock, kDvHalf, true);
    constexpr uint32_t idesc128 = make_idesc_bf16(kHeadsPerBlock, 128, true);
#pragma unroll
    for (int ks = 0; ks < kTileRows / 16; ++ks) {
        const uint32_t acc = (overwrite && ks == 0) ? 0u : 1u;
        if (kFp8) {
#pragma unroll
            for (int v2 = 0; v2 < 2; ++v2)
                umma_ts_el(o_tmem + v2 * 128, p_tmem + v2 * 16 + ks * 8,
                           v_desc + static_cast<uint64_t>((v2 * 2 * kKvBlockBytes + ks * 2048) >> 4), idesc128, acc, el);
        } else {
            umma_ts_el(o_tmem, p_tmem + ks * 8, v_desc + static_cast<uint64_t>((ks * 2048) >> 4), idesc256, acc, el);
        }
    }
}

// A warp's wait on a barrier of its own CTA.  bf16 cache: a non-blocking test first - most of these barriers
// have completed by the time they are looked at, and there the test returned sooner than try_wait (prefill
// +2 %; the fp8 kernel measured 1 % slower with it and keeps the plain form).
template <bool kFp8>
__device__ __forceinline__ bool tile_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (!kFp8 && __all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
    return warp_wait(bar, parity, abort_flag);
}

// ------------------------------------------------------------------ the kernel
// kExt: the instantiation that also handles stacked query rows, the attention sink and the second KV pool;
// the plain one keeps those branches out of the loaders and the epilogue.
template <bool kFp8, bool kExt>
__global__ void __launch_bounds__(Cfg<kFp8>::kThreads, 1)
sparse_mla_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_kv_tail, const AttnParams p) {
    using C = Cfg<kFp8>;
    constexpr int S = C::kKvStages;
    constexpr int R = kFp8 ? C::kRawStages : 1;
    extern __shared__ uint8_t smem_raw[];
    // Both CTAs of a cluster compute the same offsets (the dynamic shared window starts at the same
    // shared::cta address in every CTA of a launch), so a peer address is own address + mapa.
    // (offset arithmetic on the array itself, not through an integer, so that the compiler keeps every
    // access below in the shared address space instead of falling back to generic loads and stores)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = smem;
    uint8_t* sKV = smem + C::kOffKv;
    uint8_t* sRaw = smem + C::kOffRaw;
    uint8_t* sX = smem + C::kOffX;
    Ctl* ctl = reinterpret_cast<Ctl*>(smem + C::kOffCtl);
    volatile int* abort_flag = &ctl->abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int list = blockIdx.x >> 1;
    const int half = (int)cluster_ctarank();      // 0: columns [0,256); 1: columns [256,576)
    const int peer = half ^ 1;
    // The two MMA issuers sit on the schedulers (warp number mod 4) whose softmax warps only export and import
    // rows in this CTA - the light ones: quadrants 2, 3 in CTA 0 and 0, 1 in CTA 1; the gather issuers take the
    // other two of warps 16-19.  (TMEM is allocated and released by warp 16 in both.)
#ifndef DSA_ROLE_SWAP
#define DSA_ROLE_SWAP 0
#endif
    const int mma_warp = (half || !DSA_ROLE_SWAP) ? kMmaWarp : kMmaWarp + 2;
    const int pv_warp = mma_warp + 1;
    const int gather_warp0 = (half || !DSA_ROLE_SWAP) ? kGatherWarp0 : kMmaWarp;
    // Columns of the latent row this CTA works on: latent [256 half, 256 half + 256) (also its output columns) and
    //   bf16 cache: rope columns [32 half, 32 half + 32) - both CTAs get four and a half 64-column blocks, so
    //               neither waits for the other's partial scores;
    //   fp8 cache:  CTA 1 the whole rope (its raw row is one contiguous piece: latent half, scales, rope).
    const int col0 = half ? 256 : 0;              // first latent column of the slice
    const int rope0 = half ? 32 : 0;              // bf16 cache: first rope column of the slice
    const int w_begin = __ldg(p.list_indptr + list);
    const int w_end = __ldg(p.list_indptr + list + 1);

    // Barrier initialisation, spread over threads (about 120 barriers; one thread doing them all took
    // 2 000 cycles of every launch): thread i < 16 takes the i-th barrier of every 16-element family,
    // threads 32-39 the tile barriers, 64-67 the per-team ones, 96 the singles.
    if (tid < 16) {
        mbar_init(smem_u32(&ctl->raw_full[tid]), 1 + 32);   // the expect_tx arrival + one cp.async arrival per row
        mbar_init(smem_u32(&ctl->raw_empty[tid]), kConvertWarps);   // the eight converter warps that read it
        mbar_init(smem_u32(&ctl->m_bar[0][0]) + 8 * tid, 1);
        mbar_init(smem_u32(&ctl->x_full[tid]), 1);
        mbar_init(smem_u32(&ctl->x_free[tid]), 1);
        fence_mbar_init();
    } else if (tid >= 32 && tid < 40) {
        const int i = tid - 32;
        // fp8: the eight converter warps; bf16: every lane of the four loader warps of a group
        mbar_init(smem_u32(&ctl->kv_full[i]), kFp8 ? kConvertWarps : (kLoaderWarps / 2) * 32);
        mbar_init(smem_u32(&ctl->kv_empty[i]), 1);
        fence_mbar_init();
    } else if (tid >= 64 && tid < 64 + kGroups) {
        const int i = tid - 64;
        mbar_init(smem_u32(&ctl->s_full[i]), 1);
        mbar_init(smem_u32(&ctl->s_empty[i]), kSoftmaxWarps / kGroups);   // one team
        mbar_init(smem_u32(&ctl->p_full[i]), kSoftmaxWarps / kGroups);
        mbar_init(smem_u32(&ctl->pv_done[i]), 1);
        fence_mbar_init();
    } else if (tid == 96) {
        mbar_init(smem_u32(&ctl->q_full), kSoftmaxWarps + ((kFp8 && half) ? 1 : 0));   // + the rope block's TMA
        mbar_init(smem_u32(&ctl->q_empty), kFp8 ? 1 : 2);   // bf16 cache: two score issuers
        mbar_init(smem_u32(&ctl->o_free), kSoftmaxWarps);
        mbar_init(smem_u32(&ctl->l_bar), kSoftmaxWarps);
        mbar_init(smem_u32(&ctl->e_bar), kSoftmaxWarps);
        mbar_init(smem_u32(&ctl->o_full), 1);
        ctl->abort_flag = 0;
        fence_mbar_init();
    }
    if (kFp8 && p.H < kHeadsPerBlock) {   // rows of the rope block of Q that no load covers (heads >= H) must read as zero
        for (int i = tid * 16; i < kQBlockBytes; i += C::kThreads * 16) *reinterpret_cast<uint4*>(sQ + i) = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async_smem();         // the MMAs read the block through the async proxy
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    if (kFp8 && warp == kLoaderWarp0 && lane == 0) {   // a bf16 cache is read with plain loads: its maps are unused
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_kv);
        prefetch_tensormap(&tm_kv_tail);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything is sent to it
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;
    // Launched with programmatic stream serialization: everything above (barriers, tensor memory, descriptor
    // prefetch) may overlap the tail of the kernel before it in the stream; its results are needed from here on.
    grid_dependency_wait();
    const uint32_t peer_abort = map_to_cta(smem_u32(&ctl->abort_flag), peer);

    if (warp < kSoftmaxWarps) {
        // the four softmax warpgroups take the registers the light warpgroups give up (setmaxnreg is
        // per warpgroup; each class of warpgroups executes one instruction at the top of its branch)
        setmaxnreg_inc<kRegsSoftmax<kFp8>>();
        // ============================================================ softmax + epilogue
        // Four teams of four warps (one warp per TMEM lane quadrant) take the 32-slot tiles round robin (team =
        // tile number mod 4), so four tiles are in flight.  Thread = head row: it holds its row's 32 scores of
        // the tile, so the row maximum and sum need no other thread.  The two CTAs split the softmax by head
        // rows: CTA c computes it for rows [64 c, 64 c + 64) ("own" rows, two of a team's four warps).  For the
        // other 64 rows a warp only exports this CTA's partial scores to the peer and later imports the
        // finished P of those rows from it.  Per tile and direction 4.3 KB of partial scores and 4.3 KB of P
        // cross the SM-to-SM link (it carries ~11-17 bytes per clock): the partials as 16-bit fixed point with
        // one power-of-two-ish step per row and tile (step = 2^-15 of the row's largest partial: <= 1.5e-4 in
        // the exponent for scores up to 128), P as the bf16 the MMA consumes anyway.
        // Only the short commit of a tile is ordered after the commit of the tile before: there the shared
        // reference maximum of the row is read and moved when the tile's maximum exceeds it by more than the
        // lazy margin of 8 (the reference's threshold); O is rescaled in that rare case, in both CTAs (the
        // factor travels with P).
        constexpr int G = kGroups, CPT = kTileRows, NP = CPT / 2, OCOLS = kDvHalf / G;
        static_assert(kGroups == 4 && kTileRows == 32, "four teams, one thread per row and tile");
        const int cg = warp >> 2;            // warpgroup
        const int team = cg;                 // tiles this warp works on: it % 4 == team
        const int quad = warp & 3;           // TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;    // head row inside the block == TMEM lane
        // kRowSplit: the pair splits the softmax by head rows as described above.  Otherwise (fp8 cache, where
        // the single score buffer in TMEM and the four tile stages make the latency of a tile's chain the
        // bound, not the work in it) both CTAs run the softmax of all 128 rows on the same numbers: every warp
        // sends its partial scores and adds the peer's - both sides add the two *quantised* partials, so they
        // hold the same scores bit for bit - and no P crosses the link.
        constexpr bool kRowSplit = kFp8 ? (DSA_ROWSPLIT_FP8 != 0) : (DSA_ROWSPLIT_BF16 != 0);
        const bool own = !kRowSplit || (quad >> 1) == half;   // this CTA computes the softmax of the warp's rows
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        // Incoming buffer of this warp, written by the peer CTA's warp of the same number (it handles the same
        // rows): [4 chunks of 16 bytes][32 lanes] + one word per lane.  An own-row warp receives partial scores
        // there and sends P; the other warps send partial scores and receive P.
        const uint32_t xin = smem_u32(sX) + static_cast<uint32_t>(warp) * kXWarpBytes;
        const uint8_t* xin_p = sX + warp * kXWarpBytes;
        const uint32_t xout = map_to_cta(xin, peer);
        // one byte-counting barrier per warp for arrival, one per warp for the credit "the peer has read the last one"
        const uint32_t my_xfull = smem_u32(&ctl->x_full[warp]);
        const uint32_t my_xfree = smem_u32(&ctl->x_free[warp]);
        const uint32_t peer_xfull = map_to_cta(my_xfull, peer);
        const uint32_t peer_xfree = map_to_cta(my_xfree, peer);
        const uint32_t peer_xsink = map_to_cta(smem_u32(&ctl->x_sink[warp]), peer);
        uint32_t it_base = 0;   // global tile counter at the start of the item
        uint32_t n_sent = 0;    // tiles this warp has sent to the peer
        int item_n = 0;

        // this thread's share of an item's Q slice (its head row, a quarter of the slice's columns), read from
        // global memory one item ahead and stored into TMEM when the item starts.
        // The slice in TMEM: [latent 128 columns (256 bf16) | bf16 cache: this CTA's half of the rope, 16 columns].
        // A team stores a quarter of each part: 32 latent columns and (bf16 cache) 4 rope columns.
        constexpr int kQRegs = kFp8 ? 32 : 36;
        uint32_t qreg[kQRegs];
        auto q_fetch = [&](const dsa_v32_work_info& wq) {
            const RowMap rm = map_row<kExt>(wq, row, p.H);
            const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)rm.q_row * p.stride_q_row +
                                        (size_t)rm.head * p.stride_q_head;
            const __nv_bfloat16* src = base + col0 + 64 * cg;
            const bool live = rm.live;
            // thread = row: a warp's load touches 32 different lines, so the number of load instructions is what the
            // L1 pays for (all sixteen warps do this at once in the epilogue): 32-byte loads, four per thread
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                if (live) ldg_nc_256(reinterpret_cast<const char*>(src) + 32 * j, v);
#pragma unroll
                for (int k = 0; k < 8; ++k) qreg[8 * j + k] = v[k];
            }
            if (!kFp8) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (live) v = __ldg(reinterpret_cast<const uint4*>(base + kDV + rope0 + 8 * cg));
                qreg[32] = v.x;
                qreg[33] = v.y;
                qreg[34] = v.z;
                qreg[35] = v.w;
            }
        };
        auto q_prefetch_l2 = [&](const dsa_v32_work_info& wq) {
            const RowMap rm = map_row<kExt>(wq, row, p.H);
            if (rm.live) {
                const char* base = reinterpret_cast<const char*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)rm.q_row * p.stride_q_row +
                                                                (size_t)rm.head * p.stride_q_head);
                asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (col0 + 64 * cg) * 2));
                if (!kFp8) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (kDV + rope0 + 8 * cg) * 2));
            }
        };

        for (int w = w_begin; w < w_end; ++w, ++item_n) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            const uint32_t it_end = it_base + n_tiles;
            // Q of item n goes into TMEM once the score MMAs of item n - 1 have all read theirs: for the
            // list's first item here, for every later item during the epilogue of the item before it (so
            // the next item's scores start while this item's output is still being written).
            auto q_store = [&](const dsa_v32_work_info& wq, int n) -> bool {
                q_fetch(wq);
                if (!tile_wait<kFp8>(smem_u32(&ctl->q_empty), (n & 1) ^ 1, abort_flag)) return false;
                tc_fence_after();
                const uint32_t qcol = lane_base + kColQ + cg * 32;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t v[8] = {qreg[8 * j + 0], qreg[8 * j + 1], qreg[8 * j + 2], qreg[8 * j + 3],
                                           qreg[8 * j + 4], qreg[8 * j + 5], qreg[8 * j + 6], qreg[8 * j + 7]};
                    tmem_st_n<8>(qcol + 8 * j, v);
                }
                if (!kFp8) {
                    const uint32_t v[4] = {qreg[32], qreg[33], qreg[34], qreg[35]};
                    tmem_st_n<4>(lane_base + kColQ + 128 + cg * 4, v);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->q_full));
                return true;
            };
            if (item_n == 0) {
                if (!q_store(wi, 0)) goto done;
            }
            if (kFp8 && w + 1 < w_end) q_prefetch_l2(p.works[w + 1]);   // on its way to L2 while this item runs (bf16 cache: the Q prefetcher warp asks later)
            float l_part = 0.0f;        // this thread's share of the row sum, expressed against l_ref
            float l_ref = 0.0f;
            for (uint32_t it = it_base + ((team - it_base) & (G - 1u)); it < it_end; it += G) {
                const uint32_t tb = buf_of<kFp8>(it);         // barrier index (= team) and phase of this tile
                const uint32_t tph = phase_of<kFp8>(it);
                const bool first = (it == it_base);
                const uint32_t xph = (it / G) & 1u;           // the warp's own exchange barriers advance once per tile of its team
                // The tile's values live in pairs (64-bit registers) so that the fp32 arithmetic on them uses the
                // two-wide forms (fma/mul/add .f32x2): half the instructions of the scalar forms.
                uint64_t tv2[NP];
                if (lane == 0) mbar_arrive_expect_tx(my_xfull, kXWarpBytes);
                // ---- this CTA's partial scores of the warp's 32 rows, out of TMEM
                if (kFp8)
                    if (!tile_wait<kFp8>(smem_u32(&ctl->kv_full[it % S]), (it / S) & 1, abort_flag)) goto done;
                if (!tile_wait<kFp8>(smem_u32(&ctl->s_full[tb]), tph, abort_flag)) goto done;
                tc_fence_after();
                {
                    const uint32_t s0 = lane_base + s_col_of<kFp8>(it);
                    if (kFp8) {
                        // 16 columns at a time: the accumulators of scale group a, scale group b and (in the CTA
                        // that has them) the rope columns, all loads of a round in flight together.  The score
                        // buffer is single, so it is handed back to the MMA warp the moment the last load has returned.
#pragma unroll
                        for (int hc = 0; hc < 2; ++hc) {
                            uint32_t sr[16], sr2[16], sr3[16];
                            tmem_ld_n<16>(s0 + 16 * hc, sr);
                            tmem_ld_n<16>(s0 + 32 + 16 * hc, sr2);
                            if (half) tmem_ld_n<16>(s0 + 64 + 16 * hc, sr3);
                            const float4* sa = reinterpret_cast<const float4*>(ctl->row_scale[it % kScaleSlots][0] + 16 * hc);
                            const float4* sb4 = reinterpret_cast<const float4*>(ctl->row_scale[it % kScaleSlots][1] + 16 * hc);
                            tmem_wait_ld();
                            if (hc == 1) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[tb]));
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float4 wa = sa[j], wb = sb4[j];
                                uint64_t r0 = mul2(pack2(wa.x, wa.y), pack2u(sr[4 * j], sr[4 * j + 1]));
                                uint64_t r1 = mul2(pack2(wa.z, wa.w), pack2u(sr[4 * j + 2], sr[4 * j + 3]));
                                if (half) {
                                    r0 = add2(r0, pack2u(sr3[4 * j], sr3[4 * j + 1]));
                                    r1 = add2(r1, pack2u(sr3[4 * j + 2], sr3[4 * j + 3]));
                                }
                                tv2[8 * hc + 2 * j] = fma2(pack2(wb.x, wb.y), pack2u(sr2[4 * j], sr2[4 * j + 1]), r0);
                                tv2[8 * hc + 2 * j + 1] = fma2(pack2(wb.z, wb.w), pack2u(sr2[4 * j + 2], sr2[4 * j + 3]), r1);
                            }
                        }
                    } else {
                        uint32_t sr[CPT];
                        tmem_ld_n<CPT>(s0, sr);
                        tmem_wait_ld();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[tb]));   // the MMA warp may overwrite the scores
#pragma unroll
                        for (int j = 0; j < NP; ++j) tv2[j] = pack2u(sr[2 * j], sr[2 * j + 1]);
                    }
                }
                constexpr int kPVariants = kFp8 ? 2 : 1;
                uint32_t pk[kPVariants][NP];   // P as the MMA wants it: bf16 pairs; fp8 cache: one copy per scale group
                float f2 = 1.0f;               // factor that brings O so far to this tile's reference maximum
                if (!own) {
                    // ================================ rows whose softmax the peer computes
                    // ---- export this CTA's partial scores as 16-bit fixed point
                    {
                        float amax = 0.0f;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            float v0, v1;
                            unpack2(tv2[j], v0, v1);
                            amax = fmaxf(amax, fmaxf(fabsf(v0), fabsf(v1)));
                        }
                        // e = biased exponent of the largest partial (NaN/Inf -> the step becomes NaN and so do the scores)
                        uint32_t e = __float_as_uint(amax) >> 23;
                        e = e < 20u ? 20u : e;
                        const float q_scale = __uint_as_float((268u - e) << 23) * 0.99996948f;   // largest partial -> < 32767.5
                        const uint32_t inv_bits = e >= 255u ? 0x7FC00000u : __float_as_uint(__uint_as_float((e - 14u) << 23) * 1.0000305f);
                        const uint64_t qs2 = pack2(q_scale, q_scale), qc2 = pack2(kQuantBias, kQuantBias);
#pragma unroll
                        for (int j = 0; j < NP; ++j) tv2[j] = fma2(tv2[j], qs2, qc2);   // 2^23 + 32768 + n: n in the low 16 bits
                        if (n_sent > 0)   // the peer has read what this warp sent last (its credit has arrived)
                            if (!warp_wait_cluster(my_xfree, (n_sent & 1u) ^ 1u, abort_flag)) goto done;
                        if (lane == 0) mbar_arrive_expect_tx(my_xfree, 4);   // the credit for this send
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t wq[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                wq[k] = __byte_perm(static_cast<uint32_t>(tv2[4 * c + k]), static_cast<uint32_t>(tv2[4 * c + k] >> 32), 0x5410u);
                            st_async_b32x4(xout + c * 512 + lane * 16, wq[0], wq[1], wq[2], wq[3], peer_xfull);
                        }
                        st_async_u32(xout + 2048 + lane * 4, inv_bits, peer_xfull);
                        ++n_sent;
                    }
                    // ---- import the finished P of these rows (bf16 pairs) and the rescale factor
                    if (!warp_wait_cluster(my_xfull, xph, abort_flag)) goto done;
                    {
                        uint32_t pw[NP];
                        uint32_t dep;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint4 o = *reinterpret_cast<const uint4*>(xin_p + c * 512 + lane * 16);
                            pw[4 * c + 0] = o.x;
                            pw[4 * c + 1] = o.y;
                            pw[4 * c + 2] = o.z;
                            pw[4 * c + 3] = o.w;
                        }
                        f2 = *reinterpret_cast<const float*>(xin_p + 2048 + lane * 4);
                        // credit: the peer may overwrite the buffer.  The credit word is computed from every lane's
                        // loaded values, so it cannot leave before all of the warp's reads have returned.
                        dep = pw[0] | pw[4] | pw[8] | pw[12] | __float_as_uint(f2);
                        dep = __reduce_or_sync(0xffffffffu, dep);
                        if (lane == 0) st_async_u32(peer_xsink, dep, peer_xfree);
                        if (kFp8) {
#pragma unroll
                            for (int v = 0; v < kPVariants; ++v) {
                                const float4* sc = reinterpret_cast<const float4*>(ctl->row_scale[it % kScaleSlots][v]);
#pragma unroll
                                for (int j = 0; j < CPT / 4; ++j) {
                                    const float4 w4 = sc[j];
                                    const uint64_t a2 = pack2u(pw[2 * j] << 16, pw[2 * j] & 0xFFFF0000u);
                                    const uint64_t b2 = pack2u(pw[2 * j + 1] << 16, pw[2 * j + 1] & 0xFFFF0000u);
                                    pk[v][2 * j] = pack_bf16x2_from2(mul2(a2, pack2(w4.x, w4.y)));
                                    pk[v][2 * j + 1] = pack_bf16x2_from2(mul2(b2, pack2(w4.z, w4.w)));
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < NP; ++j) pk[0][j] = pw[j];
                        }
                    }
                } else {
                    // ================================ rows whose softmax this CTA computes
                    if (!kRowSplit) {
                        // ---- both CTAs compute these rows: send this CTA's partial scores (16-bit fixed point) ...
                        float amax = 0.0f;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            float v0, v1;
                            unpack2(tv2[j], v0, v1);
                            amax = fmaxf(amax, fmaxf(fabsf(v0), fabsf(v1)));
                        }
                        uint32_t e = __float_as_uint(amax) >> 23;
                        e = e < 20u ? 20u : e;
                        const float q_scale = __uint_as_float((268u - e) << 23) * 0.99996948f;
                        const uint32_t inv_bits = e >= 255u ? 0x7FC00000u : __float_as_uint(__uint_as_float((e - 14u) << 23) * 1.0000305f);
                        const uint64_t qs2 = pack2(q_scale, q_scale), qc2 = pack2(kQuantBias, kQuantBias);
#pragma unroll
                        for (int j = 0; j < NP; ++j) tv2[j] = fma2(tv2[j], qs2, qc2);
                        if (n_sent > 0)
                            if (!warp_wait_cluster(my_xfree, (n_sent & 1u) ^ 1u, abort_flag)) goto done;
                        if (lane == 0) mbar_arrive_expect_tx(my_xfree, 4);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t wq[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                wq[k] = __byte_perm(static_cast<uint32_t>(tv2[4 * c + k]), static_cast<uint32_t>(tv2[4 * c + k] >> 32), 0x5410u);
                            st_async_b32x4(xout + c * 512 + lane * 16, wq[0], wq[1], wq[2], wq[3], peer_xfull);
                        }
                        st_async_u32(xout + 2048 + lane * 4, inv_bits, peer_xfull);
                        ++n_sent;
                        // ... and take them back from the quantised form while the peer's are on their way
                        const float own_inv = __uint_as_float(inv_bits);
                        const uint64_t oi2 = pack2(own_inv, own_inv), nb2 = pack2(-kQuantBias, -kQuantBias);
#pragma unroll
                        for (int j = 0; j < NP; ++j) tv2[j] = mul2(add2(tv2[j], nb2), oi2);
                    }
                    // ---- add the peer's partial scores
                    if (!warp_wait_cluster(my_xfull, xph, abort_flag)) goto done;
                    {
                        const float peer_inv = *reinterpret_cast<const float*>(xin_p + 2048 + lane * 4);
                        const uint64_t pi2 = pack2(peer_inv, peer_inv), nb2 = pack2(-kQuantBias, -kQuantBias);
                        uint32_t dep = __float_as_uint(peer_inv);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint4 o = *reinterpret_cast<const uint4*>(xin_p + c * 512 + lane * 16);
                            const uint32_t wq[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint64_t b2 = pack2u(__byte_perm(wq[k], 0x4B00u, 0x5410u), __byte_perm(wq[k], 0x4B00u, 0x5432u));
                                tv2[4 * c + k] = fma2(add2(b2, nb2), pi2, tv2[4 * c + k]);
                            }
                            dep |= o.x;
                        }
                        dep = __reduce_or_sync(0xffffffffu, dep);
                        if (lane == 0) st_async_u32(peer_xsink, dep, peer_xfree);
                    }
                    if (!kFp8)
                        if (!tile_wait<kFp8>(smem_u32(&ctl->kv_full[it % S]), (it / S) & 1, abort_flag)) goto done;
                    // ---- mask (padding slots; the mask is the same for every row, so a full tile skips this)
                    const uint32_t mask = ctl->tile_mask[it % kMaskSlots];
                    if (mask != 0xFFFFFFFFu) {
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            float v0, v1;
                            unpack2(tv2[j], v0, v1);
                            if (!((mask >> (2 * j)) & 1u)) v0 = -INFINITY;
                            if (!((mask >> (2 * j + 1)) & 1u)) v1 = -INFINITY;
                            tv2[j] = pack2(v0, v1);
                        }
                    }
                    // ---- row maximum over the tile's 32 columns, in the log2 domain; the scale is positive, so
                    // the maximum is taken on the raw scores and scaled once
                    float mt;
                    {
                        float t[NP];
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            float v0, v1;
                            unpack2(tv2[j], v0, v1);
                            t[j] = fmaxf(v0, v1);
                        }
                        const float u0 = max3(t[0], t[1], t[2]), u1 = max3(t[3], t[4], t[5]), u2 = max3(t[6], t[7], t[8]);
                        const float u3 = max3(t[9], t[10], t[11]), u4 = max3(t[12], t[13], t[14]);
                        mt = fmaxf(max3(u0, u1, t[15]), max3(u2, u3, u4)) * p.scale_log2;
                    }
                    // ---- the row's reference maximum, moved in tile order.  This is the only step that waits
                    // for the tile before (per lane quadrant: the warp of the previous team with the same rows),
                    // and it is a handful of instructions: read the reference, move it if the tile's maximum
                    // exceeds it by more than the lazy margin of 8, publish.
                    if (!first)
                        if (!tile_wait<kFp8>(smem_u32(&ctl->m_bar[buf_of<kFp8>(it - 1)][quad]), phase_of<kFp8>(it - 1), abort_flag)) goto done;
                    const float m_cur = first ? -INFINITY : ctl->m_shared[row];
                    const bool raise = mt > m_cur + 8.0f;
                    const float m_fin = raise ? mt : m_cur;
                    if (raise || first) ctl->m_shared[row] = m_fin;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl->m_bar[tb][quad]));
                    if (raise && !first) f2 = (m_cur == -INFINITY) ? 0.0f : ex2_approx(m_cur - m_fin);
                    // ---- P = 2^(score - reference): at most 2^8; a masked slot gives 0
                    const float m_fin_use = (m_fin == -INFINITY) ? 0.0f : m_fin;
                    float lsum;
                    {
                        const uint64_t c2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(-m_fin_use, -m_fin_use);
                        uint64_t ls2 = pack2(0.0f, 0.0f);
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            float v0, v1;
                            unpack2(fma2(tv2[j], c2, nm2), v0, v1);
                            tv2[j] = pack2(ex2_approx(v0), ex2_approx(v1));
                            ls2 = add2(ls2, tv2[j]);
                        }
                        float l0, l1;
                        unpack2(ls2, l0, l1);
                        lsum = l0 + l1;
                    }
                    if (l_part != 0.0f && l_ref != m_fin) l_part *= ex2_approx(l_ref - m_fin);
                    l_part += lsum;
                    l_ref = m_fin;
                    // ---- P to the peer (bf16 pairs) with the rescale factor, once it has read the last one
                    {
                        uint32_t ps[NP];
#pragma unroll
                        for (int j = 0; j < NP; ++j) ps[j] = pack_bf16x2_from2(tv2[j]);
                        if (kRowSplit) {
                            if (n_sent > 0)
                                if (!warp_wait_cluster(my_xfree, (n_sent & 1u) ^ 1u, abort_flag)) goto done;
                            if (lane == 0) mbar_arrive_expect_tx(my_xfree, 4);   // the credit for this send
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                st_async_b32x4(xout + c * 512 + lane * 16, ps[4 * c], ps[4 * c + 1], ps[4 * c + 2], ps[4 * c + 3], peer_xfull);
                            st_async_u32(xout + 2048 + lane * 4, __float_as_uint(f2), peer_xfull);
                            ++n_sent;
                        }
                        if (!kFp8) {
#pragma unroll
                            for (int j = 0; j < NP; ++j) pk[0][j] = ps[j];
                        }
                    }
                    if (kFp8) {
                        // two copies, each pre-multiplied by one scale group's row scales
#pragma unroll
                        for (int v = 0; v < kPVariants; ++v) {
                            const float4* sc = reinterpret_cast<const float4*>(ctl->row_scale[it % kScaleSlots][v]);
#pragma unroll
                            for (int j = 0; j < CPT / 4; ++j) {
                                const float4 w4 = sc[j];
                                pk[v][2 * j] = pack_bf16x2_from2(mul2(tv2[2 * j], pack2(w4.x, w4.y)));
                                pk[v][2 * j + 1] = pack_bf16x2_from2(mul2(tv2[2 * j + 1], pack2(w4.z, w4.w)));
                            }
                        }
                    }
                }
                // ---- hand P to the MMA warp: after the P V product that last read this tile's P buffer
                if (it >= kBufReuse<kFp8>)
                    if (!tile_wait<kFp8>(smem_u32(&ctl->pv_done[buf_of<kFp8>(it - kBufReuse<kFp8>)]), phase_of<kFp8>(it - kBufReuse<kFp8>), abort_flag))
                        goto done;
                if (__any_sync(0xffffffffu, f2 != 1.0f) && !first) {
                    // the reference moved: O so far (complete once the previous tile's P V product has finished)
                    // is brought to the new reference before this tile's product is added
                    if (!tile_wait<kFp8>(smem_u32(&ctl->pv_done[buf_of<kFp8>(it - 1)]), phase_of<kFp8>(it - 1), abort_flag)) goto done;
                    tc_fence_after();
#pragma unroll 1
                    for (int oc = 0; oc < kDvHalf; oc += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + oc, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f2);
                        tmem_st32(lane_base + kColO + oc, o);
                    }
                    tmem_wait_st();
                }
                {
                    const uint32_t p0col = lane_base + p_col_of<kFp8>(it);
#pragma unroll
                    for (int v = 0; v < kPVariants; ++v) tmem_st_n<NP>(p0col + 16 * v, pk[v]);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[tb]));
            }
            // ---- epilogue of the item (all sixteen warps)
            {
                const int lp = item_n & 1;   // the row sums are kept per item parity: the next item's may arrive early
                // Every warp arrives when its own tiles of the item are committed; once all sixteen have, every
                // row's reference maximum is final.  (A per-item barrier and not the last tile's p_full: a parity
                // wait is only safe when the barrier's previous phase has already completed, which a warp that
                // finished early cannot know of another team's barrier.)
                // the next work item is read before the barrier: its Q is fetched right after the row sums below, and
                // the addresses of those loads should not wait for this one
                const dsa_v32_work_info wnext = p.works[w + 1 < w_end ? w + 1 : w];
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->e_bar));
                if (!tile_wait<kFp8>(smem_u32(&ctl->e_bar), item_n & 1, abort_flag)) goto done;
                float m_ref = 0.0f;
                if (own) {
                    // this team's share of the row sums, for this CTA and for the peer (it holds the other half of
                    // the rows' output columns)
                    m_ref = ctl->m_shared[row];
                    float lv = (l_part != 0.0f && l_ref != m_ref) ? l_part * ex2_approx(l_ref - m_ref) : l_part;
                    if (kExt && p.attn_sink != nullptr) {
                        // attention sink (opus_attn/dsa_v4/common/mla_v4_host.cc:469-472): one more term exp(sink - m) in the
                        // denominator, counted once per query row and head: by team 0, in the piece that starts the list
                        const RowMap rs = map_row<kExt>(wi, row, p.H);
                        const float sink2 = rs.live ? __ldg(p.attn_sink + rs.head) * 1.4426950408889634f : -INFINITY;
                        if (m_ref == -INFINITY) m_ref = sink2;                      // no valid score in this piece: the sink is the reference
                        if (cg == 0 && wi.k_begin == 0 && sink2 > -INFINITY) lv += ex2_approx(sink2 - m_ref);
                    }
                    ctl->l_part[lp][cg][row] = lv;
                    if (kRowSplit) st_cluster_u32(map_to_cta(smem_u32(&ctl->l_part[lp][cg][row]), peer), __float_as_uint(lv));
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(smem_u32(&ctl->l_bar));
                        if (kRowSplit) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->l_bar), peer));
                    }
                }
                if (w + 1 < w_end)
                    if (!q_store(wnext, item_n + 1)) goto done;
                if (!warp_wait_cluster(smem_u32(&ctl->l_bar), item_n & 1, abort_flag)) goto done;
                float l = 0.0f;
#pragma unroll
                for (int g = 0; g < G; ++g) l += ctl->l_part[lp][g][row];
                if (!tile_wait<kFp8>(smem_u32(&ctl->o_full), item_n & 1, abort_flag)) goto done;
                tc_fence_after();
                const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
                const RowMap rm = map_row<kExt>(wi, row, p.H);
                const int head = rm.head;
                const bool live = rm.live;
                const float lse_nat = (l > 0.0f) ? (m_ref + __log2f(l)) * 0.69314718055994531f : INFINITY;
                if (wi.partial_slot < 0 && kExt && p.n_peers > 0) {
                    // element offset of the row's 256 columns of this CTA; the same in out and in every peer's
                    // gathered buffer (fused all-gather: plain stores through the peer-mapped pointers)
                    const size_t o_off = (size_t)rm.q_row * p.stride_o_row + (size_t)head * p.stride_o_head + half * kDvHalf;
                    const int n_dst = p.n_peers > 0 ? p.n_peers : 1;
#pragma unroll 1
                    for (int oc = cg * OCOLS; oc < (cg + 1) * OCOLS; oc += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + oc, o);
                        tmem_wait_ld();
                        if (live) {
                            uint4 u[4];
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                u[v].x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                                u[v].y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                                u[v].z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                                u[v].w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                            }
#pragma unroll 1
                            for (int d = 0; d < n_dst; ++d) {
                                __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.n_peers > 0 ? p.out_peers[d] : p.out);
                                stg_256(base + o_off + oc, u[0].x, u[0].y, u[0].z, u[0].w, u[1].x, u[1].y, u[1].z, u[1].w);
                                stg_256(base + o_off + oc + 16, u[2].x, u[2].y, u[2].z, u[2].w, u[3].x, u[3].y, u[3].z, u[3].w);
                            }
                        }
                    }
                    if (live && (kRowSplit ? own : half == 0) && cg == 0) {
                        const size_t l_off = (size_t)rm.q_row * p.lse_stride_row + head;
                        if (p.n_peers > 0) {
                            for (int d = 0; d < p.n_peers; ++d)
                                if (p.lse_peers[d] != nullptr) p.lse_peers[d][l_off] = lse_nat;
                        } else if (p.lse != nullptr) {
                            p.lse[l_off] = lse_nat;
                        }
                    }
                } else if (wi.partial_slot < 0) {
                    __nv_bfloat16* o_dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)rm.q_row * p.stride_o_row +
                                           (size_t)head * p.stride_o_head + half * kDvHalf;
#pragma unroll 1
                    for (int oc = cg * OCOLS; oc < (cg + 1) * OCOLS; oc += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + oc, o);
                        tmem_wait_ld();
                        if (live) {
                            // thread = row, so a store touches 32 lines whatever its width: 32-byte stores, two per round
                            uint32_t u[16];
#pragma unroll
                            for (int v = 0; v < 16; ++v) u[v] = pack_bf16x2(__uint_as_float(o[2 * v]) * inv, __uint_as_float(o[2 * v + 1]) * inv);
                            stg_256(o_dst + oc, u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7]);
                            stg_256(o_dst + oc + 16, u[8], u[9], u[10], u[11], u[12], u[13], u[14], u[15]);
                        }
                    }
                    if (live && (kRowSplit ? own : half == 0) && cg == 0 && p.lse != nullptr) p.lse[(size_t)rm.q_row * p.H + head] = lse_nat;
                } else {
                    float* o_dst = p.o_accum + ((size_t)wi.partial_slot * kHeadsPerBlock + row) * kDV + half * kDvHalf;
#pragma unroll 1
                    for (int oc = cg * OCOLS; oc < (cg + 1) * OCOLS; oc += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + oc, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            stg_256(o_dst + oc + 8 * v, __float_as_uint(__uint_as_float(o[8 * v + 0]) * inv), __float_as_uint(__uint_as_float(o[8 * v + 1]) * inv),
                                    __float_as_uint(__uint_as_float(o[8 * v + 2]) * inv), __float_as_uint(__uint_as_float(o[8 * v + 3]) * inv),
                                    __float_as_uint(__uint_as_float(o[8 * v + 4]) * inv), __float_as_uint(__uint_as_float(o[8 * v + 5]) * inv),
                                    __float_as_uint(__uint_as_float(o[8 * v + 6]) * inv), __float_as_uint(__uint_as_float(o[8 * v + 7]) * inv));
                    }
                    if ((kRowSplit ? own : half == 0) && cg == 0)
                        p.lse_accum[(size_t)wi.partial_slot * kHeadsPerBlock + row] = (l > 0.0f) ? lse_nat : -FLT_MAX;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->o_free));
            }
            it_base = it_end;
        }
        // nothing this warp sent may still be on its way when the CTA exits: wait for the credit of the last send
        if (n_sent > 0)
            if (!warp_wait_cluster(my_xfree, (n_sent & 1u) ^ 1u, abort_flag)) goto done;
    } else {
    setmaxnreg_dec<kRegsOther<kFp8>>();
    if (warp == mma_warp || (!kFp8 && warp == gather_warp0)) {
        // ============================================================ score MMA issuer(s)
        // The whole warp runs the loop converged (descriptors stay warp-uniform); one elected lane issues.
        // Scores and P V products are issued by different warps, each blocking on its own inputs, so
        // neither waits behind the other's barrier round trips; the tensor pipe runs them in issue order.
        // bf16 cache: two score issuers on alternate tiles (warp 18 has no gathers to issue there).  An issuer's
        // turn per tile - tile barrier, proxy fence, score-buffer barrier, tcgen05 fence, 18 instructions, commit -
        // takes about as long as the whole pipeline's period, so one issuer alone was the bound.  Even tiles use
        // score buffer 0 and teams 0, 2, odd tiles buffer 1 and teams 1, 3, so the two never share a buffer or a
        // team barrier; both wait on every tile's landing barrier, in order, so that neither ever waits on a
        // phase whose predecessor it has not seen complete.
        const uint32_t par = (!kFp8 && warp != mma_warp) ? 1u : 0u;
        const uint32_t el = elect_one() ? 1u : 0u;
        const uint64_t q_desc = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);            // K-major view
        uint32_t it = 0;
        int item_n = 0;
        for (int w = w_begin; w < w_end; ++w, ++item_n) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            if (!tile_wait<kFp8>(smem_u32(&ctl->q_full), item_n & 1, abort_flag)) goto done;
            for (int t = 0; t < n_tiles; ++t, ++it) {
                const int s = it % S;
                const uint32_t sb = buf_of<kFp8>(it);
                if (!tile_wait<kFp8>(smem_u32(&ctl->kv_full[s]), (it / S) & 1, abort_flag)) goto done;
                if (!kFp8 && (it & 1u) != par) continue;   // the other issuer's tile
                if (!kFp8) fence_proxy_async_smem();   // the tile was written by cp.async (generic proxy)
                // the softmax warps have drained the tile that used this score buffer last
                if (it >= kBufReuse<kFp8>)
                    if (!tile_wait<kFp8>(smem_u32(&ctl->s_empty[buf_of<kFp8>(it - kBufReuse<kFp8>)]), phase_of<kFp8>(it - kBufReuse<kFp8>), abort_flag))
                        goto done;
                tc_fence_after();
                const uint64_t k_desc = k_desc0 + static_cast<uint64_t>((s * kKvTileBytes) >> 4);
                const uint32_t d0 = tmem + s_col_of<kFp8>(it);
                if (kFp8 && half) issue_qk_mmas<kFp8, 5>(d0, q_desc, tmem + kColQ, k_desc, el);
                else issue_qk_mmas<kFp8, 4>(d0, q_desc, tmem + kColQ, k_desc, el);   // bf16 cache: four blocks + half a block
                tc_commit_el(smem_u32(&ctl->s_full[sb]), el);
            }
            // the item's Q may be replaced once this issuer's products of the item are complete (bf16 cache: and the other's)
            tc_commit_el(smem_u32(&ctl->q_empty), el);
        }
    } else if (warp == pv_warp) {
        // ============================================================ P V MMA issuer
        const uint32_t el = elect_one() ? 1u : 0u;
        const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(sKV), kKvBlockBytes, 1024); // MN-major view
        uint32_t it = 0;
        int item_n = 0;
        for (int w = w_begin; w < w_end; ++w, ++item_n) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            for (int t = 0; t < n_tiles; ++t, ++it) {
                const int s = it % S;
                const uint32_t sb = buf_of<kFp8>(it);
                if (!tile_wait<kFp8>(smem_u32(&ctl->p_full[sb]), phase_of<kFp8>(it), abort_flag)) goto done;
                if (!kFp8) {   // the tile was written by cp.async (generic proxy): observe its barrier, then fence
                    if (!tile_wait<kFp8>(smem_u32(&ctl->kv_full[s]), (it / S) & 1, abort_flag)) goto done;
                    fence_proxy_async_smem();
                }
                if (t == 0 && item_n > 0)   // the previous item's O has been read out
                    if (!tile_wait<kFp8>(smem_u32(&ctl->o_free), (item_n - 1) & 1, abort_flag)) goto done;
                tc_fence_after();
                issue_pv_mmas<kFp8>(tmem + kColO, tmem + p_col_of<kFp8>(it),
                                    v_desc0 + static_cast<uint64_t>((s * kKvTileBytes) >> 4), t == 0, el);
                tc_commit_el(smem_u32(&ctl->kv_empty[s]), el);
                tc_commit_el(smem_u32(&ctl->pv_done[sb]), el);
                if (t + 1 == n_tiles) tc_commit_el(smem_u32(&ctl->o_full), el);
            }
        }
    } else if (!kFp8) {
        // ============================================================ loaders (bf16 cache)
        // Eight warps in two groups that take alternate tiles; in a group, warp l4 owns rows [8 l4, 8 l4 + 8)
        // of the tile, four lanes per row: top-k slot -> block table -> physical row, then the row's 512
        // or 640 bytes of this CTA's slice go straight into the 128-byte swizzled MMA tile as 16-byte
        // cp.async copies (8-10 per lane), completion counted on the tile's barrier.  A TMA tile::gather4
        // here moves one 128-byte block of four rows per request, 40 requests per tile, and the TMA unit
        // takes a request only every ~25-37 cycles whatever the number of issuing warps (measured): that
        // was the period of the whole bf16 pipeline.  (The fp8 path, 8 requests per tile, keeps gather4.)
        const int lw = warp - kLoaderWarp0;
        if (warp == kGatherWarp0 + 1) {
            // ======================================================== Q prefetcher (the warp left over for a bf16 cache)
            // The softmax warps load the next item's Q in their epilogue, and the score MMAs of that item wait
            // for it.  This warp follows the tiles (it waits on every tile's landing barrier, in order) and asks
            // for this CTA's slice of the next item's Q eight tiles before the item ends: late enough that the
            // lines are still in L2 when they are loaded, early enough to be there.
            uint32_t it = 0;
            for (int w = w_begin; w < w_end; ++w) {
                const dsa_v32_work_info wi = p.works[w];
                const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
                const int t_ask = n_tiles > 8 ? n_tiles - 8 : 0;
                for (int t = 0; t < n_tiles; ++t, ++it) {
                    if (t == t_ask && w + 1 < w_end) {
                        const dsa_v32_work_info wn = p.works[w + 1];
#pragma unroll 1
                        for (int r = lane; r < kHeadsPerBlock; r += 32) {
                            const RowMap rn = map_row<kExt>(wn, r, p.H);
                            if (rn.live) {
                                const char* qb = reinterpret_cast<const char*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                                                                               (size_t)rn.q_row * p.stride_q_row + (size_t)rn.head * p.stride_q_head);
#pragma unroll
                                for (int c = 0; c < 4; ++c) asm volatile("prefetch.global.L2 [%0];" ::"l"(qb + col0 * 2 + 128 * c));
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(qb + (kDV + rope0) * 2));
                            }
                        }
                    }
                    if (!tile_wait<kFp8>(smem_u32(&ctl->kv_full[it % S]), (it / S) & 1, abort_flag)) goto done;
                }
            }
        } else if (lw >= 0 && lw < kLoaderWarps) {
            const int grp = lw >> 2;                 // tiles this warp loads: it % 2 == grp
            const int l4 = lw & 3;
            const int rloc = lane >> 2;              // row of the warp's eight this lane copies
            const int r = 8 * l4 + rloc;             // tile row
            const int c4 = lane & 3;                 // its 16-byte chunks: c4, c4 + 4, ...
            uint8_t* mask_bytes = reinterpret_cast<uint8_t*>(ctl->tile_mask);
            const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
            uint32_t it_base = 0;
            for (int w = w_begin; w < w_end; ++w) {
                const dsa_v32_work_info wi = p.works[w];
                const int seq = wi.q_row / p.s_q;
                const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
                const int32_t* idx_row = p.indices + (size_t)wi.q_row * p.topk;
                const int pool_split = (kExt && p.pool_split != nullptr) ? __ldg(p.pool_split + wi.q_row) : 0x7FFFFFFF;
                auto load_slot = [&](int k0) -> int {
                    const int k = k0 + r;
                    return (k < wi.k_end) ? __ldg(idx_row + k) : -1;
                };
                // this warp's tiles of the item: u0, u0 + 2, ...; two-deep software pipeline over them so no
                // load is consumed in the step that issues it
                const int u0 = (grp - (int)it_base) & 1;
                const int kb0 = wi.k_begin + u0 * kTileRows;
                int idx_a = load_slot(kb0), idx_b = load_slot(kb0 + 2 * kTileRows);
                int idx_c = load_slot(kb0 + 4 * kTileRows), idx_d = load_slot(kb0 + 6 * kTileRows);
                int phys_a = block_of(idx_a, seq, p), phys_b = block_of(idx_b, seq, p);
                for (int u = u0; u < n_tiles; u += 2) {
                    const uint32_t it = it_base + u;
                    const int k0 = wi.k_begin + u * kTileRows;
                    int row = row_of(idx_a, phys_a, seq, p);
                    const uint8_t* pool = kv_bytes;
                    if (kExt && p.kv2 != nullptr && k0 + r >= pool_split) {   // "extend" slots: physical rows of the second pool
                        row = (idx_a >= 0 && idx_a < p.num_kv2_rows) ? idx_a : -1;
                        pool = reinterpret_cast<const uint8_t*>(p.kv2);
                    }
                    {
                        const int phys_n = block_of(idx_c, seq, p);
                        const int idx_n = load_slot(k0 + 8 * kTileRows);
                        idx_a = idx_b; phys_a = phys_b;
                        idx_b = idx_c; phys_b = phys_n;
                        idx_c = idx_d; idx_d = idx_n;
                    }
                    // one mask bit per row (lanes 0, 4, 8, ... hold the eight rows)
                    const int row_of_lane8 = __shfl_sync(0xffffffffu, row, (lane & 7) * 4);
                    const uint32_t mask8 = __ballot_sync(0xffffffffu, row_of_lane8 >= 0) & 0xFFu;
                    const int s = it % S;
                    if (!tile_wait<kFp8>(smem_u32(&ctl->kv_empty[s]), ((it / S) & 1) ^ 1, abort_flag)) goto done;
                    const uint32_t bar = smem_u32(&ctl->kv_full[s]);
                    if (lane == 0) mask_bytes[(it % kMaskSlots) * 4 + l4] = static_cast<uint8_t>(mask8);
                    // padding / out-of-range rows: nothing is read, the row is filled with zeros
                    const uint8_t* src_row = pool + (size_t)(row >= 0 ? row : 0) * (kDQK * 2);
                    const uint8_t* src = src_row + col0 * 2;
                    const uint32_t nbytes = row >= 0 ? 16u : 0u;
                    const uint32_t dst_row = smem_u32(sKV + s * kKvTileBytes) + r * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int cc = c4 + 4 * j;           // latent chunk of the slice: block cc / 8, chunk cc % 8 of its row
                        cp_async_16(dst_row + (cc >> 3) * kKvBlockBytes + (((cc & 7) ^ (r & 7)) << 4), src + cc * 16, nbytes);
                    }
                    // this CTA's half of the rope columns: chunks 0-3 of block 4 (the score MMAs take two K steps of it)
                    cp_async_16(dst_row + 4 * kKvBlockBytes + ((c4 ^ (r & 7)) << 4), src_row + (kDV + rope0) * 2 + c4 * 16, nbytes);
                    cp_async_mbar_arrive_noinc(bar);
                }
                it_base += n_tiles;
            }
        }
    } else if (warp < kGatherWarp0 + kGatherWarps) {
        // ============================================================ gather issuers (fp8 cache)
        // Two warps that take alternate tiles (an issue is a chain of latencies: slot and block-table loads,
        // shuffles, the gather4 instructions themselves at ~70 cycles each; two tiles in flight hide it).
        // Lane = row of the tile: top-k slot -> physical row; lanes 0-7 each issue ONE TMA tile::gather4 for a
        // group of four rows (the row's bytes of this CTA's slice in one request: the cache is described as
        // 32-bit elements so that a request may be wider than 256 bytes); every lane fetches its row's two
        // scales by cp.async straight into the scale table.  The issuers run ahead of the converters by the
        // raw ring (kRawStages tiles), across items.
        const int iw = warp - gather_warp0;
        const int gl = lane & 7;
        const int oob_row = (int)p.num_kv_rows;
        const uint32_t row_bytes = half ? 400u : 256u;   // latent half (+ scales + rope)
        const CUtensorMap* tmap = half ? &tm_kv_tail : &tm_kv;
        const int tcol = half ? 64 : 0;                  // first 32-bit element of the slice
        const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
        uint32_t it_base = 0;
        for (int w = w_begin; w < w_end; ++w) {
            const dsa_v32_work_info wi = p.works[w];
            const int seq = wi.q_row / p.s_q;
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            const int32_t* idx_row = p.indices + (size_t)wi.q_row * p.topk;
            auto load_slot = [&](int k0) -> int {
                const int k = k0 + lane;
                return (k < wi.k_end) ? __ldg(idx_row + k) : -1;
            };
            // this warp's tiles of the item: u0, u0 + 2, ...; two-deep software pipeline over them
            const int u0 = (iw - (int)it_base) & 1;
            const int kb0 = wi.k_begin + u0 * kTileRows;
            int idx_a = load_slot(kb0), idx_b = load_slot(kb0 + 2 * kTileRows);
            int idx_c = load_slot(kb0 + 4 * kTileRows), idx_d = load_slot(kb0 + 6 * kTileRows);
            int phys_a = block_of(idx_a, seq, p), phys_b = block_of(idx_b, seq, p);
            for (int u = u0; u < n_tiles; u += 2) {
                const uint32_t it = it_base + u;
                const int k0 = wi.k_begin + u * kTileRows;
                const int row = row_of(idx_a, phys_a, seq, p);
                {
                    const int phys_n = block_of(idx_c, seq, p);
                    const int idx_n = load_slot(k0 + 8 * kTileRows);
                    idx_a = idx_b; phys_a = phys_b;
                    idx_b = idx_c; phys_b = phys_n;
                    idx_c = idx_d; idx_d = idx_n;
                }
                const uint32_t mask = __ballot_sync(0xffffffffu, row >= 0);
                const int coord = row >= 0 ? row : oob_row;
                const int r0 = __shfl_sync(0xffffffffu, coord, 4 * gl + 0);
                const int r1 = __shfl_sync(0xffffffffu, coord, 4 * gl + 1);
                const int r2 = __shfl_sync(0xffffffffu, coord, 4 * gl + 2);
                const int r3 = __shfl_sync(0xffffffffu, coord, 4 * gl + 3);
                const int rs = it % R;
                if (!tile_wait<kFp8>(smem_u32(&ctl->raw_empty[rs]), ((it / R) & 1) ^ 1, abort_flag)) goto done;
                const uint32_t bar = smem_u32(&ctl->raw_full[rs]);
                if (lane == 0) {
                    ctl->tile_mask[it % kMaskSlots] = mask;
                    mbar_arrive_expect_tx(bar, kTileRows * row_bytes);
                }
                __syncwarp();
                {
                    // the two fp32 scales of this CTA's groups: bytes 512 + 8 half of the row (zeros for padding)
                    const uint8_t* src = kv_bytes + (size_t)(row >= 0 ? row : 0) * kFp8RowBytes + 512 + 8 * half;
                    const uint32_t n = row >= 0 ? 4u : 0u;
                    float* sc = &ctl->row_scale[it % kScaleSlots][0][lane];
                    cp_async_4(smem_u32(sc), src, n);
                    cp_async_4(smem_u32(sc + kTileRows), src + 4, n);
                    cp_async_mbar_arrive_noinc(bar);
                }
                if (lane < 8) {
                    const uint32_t dst = smem_u32(sRaw + rs * kRawTileBytes + lane * kRawGroupBytes);
                    tma_gather4(dst, tmap, bar, tcol, r0, r1, r2, r3);
                }
            }
            it_base += n_tiles;
        }
    } else {
        // ============================================================ converters (fp8 cache)
        // Eight warps in two groups that take alternate tiles (a tile's conversion is a chain of latencies:
        // raw bytes in, arithmetic, tile bytes out, proxy fence; two tiles in flight hide it).  In a group,
        // warp c4 turns rows [8 c4, 8 c4 + 8) of the raw tile into the bf16 MMA tile:
        // e4m3 -> bf16 exactly (e4m3 has 4 significant bits; the reference's LDS round trip is
        // ..mxfp8_16mx8_32nx1_template.hpp:852-864), and copies the rope columns.  The per-128 fp32
        // scales never touch the operands (see the softmax warps).
        const int cw = warp - kConvertWarp0;
        const int r = 4 * cw + (lane >> 3);      // tile row: all eight warps work on every tile, four rows each
        const int oc = lane & 7;                 // this lane converts the 16-byte raw chunks oc and oc + 8 of the row's 256 latent bytes
        const uint32_t row_bytes = half ? 400u : 256u;
        uint32_t it = 0;
        int item_n = 0;
        for (int w = w_begin; w < w_end; ++w, ++item_n) {
            const dsa_v32_work_info wi = p.works[w];
            const int n_tiles = (wi.k_end - wi.k_begin + kTileRows - 1) / kTileRows;
            if (half && cw == 0) {
                // rope block of the item's Q (the latent part goes to TMEM through the softmax warps)
                if (!tile_wait<kFp8>(smem_u32(&ctl->q_empty), (item_n & 1) ^ 1, abort_flag)) goto done;
                if (lane == 0) {
                    // the box holds min(H, 128) heads of one query row; a stacked item loads one box per query
                    // row, H heads apart (rows of the block that no box covers were zeroed at kernel start)
                    const uint32_t bar = smem_u32(&ctl->q_full);
                    const int hbox = p.H < kHeadsPerBlock ? p.H : kHeadsPerBlock;
                    const int n_box = (kExt && wi.stacked_rows > 1) ? wi.stacked_rows : 1;
                    mbar_arrive_expect_tx(bar, static_cast<uint32_t>(n_box * hbox * 128));
                    for (int b = 0; b < n_box; ++b)
                        tma_load_3d(smem_u32(sQ) + static_cast<uint32_t>(b * hbox * 128), &tm_q, bar, kDV,
                                    wi.head_block * kHeadsPerBlock, wi.q_row + b);
                }
            }
            for (int t = 0; t < n_tiles; ++t, ++it) {
                const int rs = it % R, s = it % S;
                if (!tile_wait<kFp8>(smem_u32(&ctl->raw_full[rs]), (it / R) & 1, abort_flag)) goto done;
                // the raw bytes are read before the wait for a free tile stage: a stage is the scarce resource (the
                // period of the pipeline is the time a tile occupies one), so as little as possible happens after it
                const uint8_t* row_raw = sRaw + rs * kRawTileBytes + (r >> 2) * kRawGroupBytes + (r & 3) * row_bytes;
                uint4 raw[2], rope = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int k = 0; k < 2; ++k) raw[k] = *reinterpret_cast<const uint4*>(row_raw + (oc + 8 * k) * 16);
                // rope: 64 bf16 = 8 chunks (after the 256 latent bytes and the 16 scale bytes of the raw row), one per lane
                if (half) rope = *reinterpret_cast<const uint4*>(row_raw + 272 + oc * 16);
                if (!tile_wait<kFp8>(smem_u32(&ctl->kv_empty[s]), ((it / S) & 1) ^ 1, abort_flag)) goto done;
                uint8_t* tile = sKV + s * kKvTileBytes + r * 128;
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int j = oc + 8 * k;    // raw chunk -> 64-column block j / 4, its 16-byte chunks 2 c and 2 c + 1
                    const int c = j & 3;
                    const uint32_t wv[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
                    uint32_t o[8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        o[2 * q + 0] = e4m3x2_to_bf16x2(__byte_perm(wv[q], 0u, 0x1404u));
                        o[2 * q + 1] = e4m3x2_to_bf16x2(__byte_perm(wv[q], 0u, 0x3424u));
                    }
                    uint8_t* dst_row = tile + (j >> 2) * kKvBlockBytes;
                    // lanes 4-7 of a row store their two chunks in the other order: the eight lanes then hit eight different banks groups
                    const int h0 = (oc >> 2) & 1;
                    *reinterpret_cast<uint4*>(dst_row + (((2 * c + h0) ^ (r & 7)) * 16)) =
                        h0 ? make_uint4(o[4], o[5], o[6], o[7]) : make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(dst_row + (((2 * c + (h0 ^ 1)) ^ (r & 7)) * 16)) =
                        h0 ? make_uint4(o[0], o[1], o[2], o[3]) : make_uint4(o[4], o[5], o[6], o[7]);
                }
                if (half) *reinterpret_cast<uint4*>(tile + 4 * kKvBlockBytes + ((oc ^ (r & 7)) * 16)) = rope;
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&ctl->kv_full[s]));
                    mbar_arrive(smem_u32(&ctl->raw_empty[rs]));
                }
            }
        }
    }
    }

done:
    if (ctl->abort_flag) st_cluster_u32(peer_abort, 1u);   // let the peer stop waiting for us
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ctl->abort_flag) atomicExch(p.status, DSA_V32_ERR_DEVICE_WAIT);
    cluster_sync_all();
    if (warp == kMmaWarp) {
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
                                                      const ReduceDst* __restrict__ reduce_dst, const OutTargets tgt,
                                                      int64_t stride_o_row, int64_t stride_o_head, int H) {
    const int rr = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hrow = blockIdx.y * 8 + warp;  // head inside the 128-head block
    grid_dependency_wait();   // launched ahead of the attention kernel's end (programmatic stream serialization)
    const ReduceDst dst = reduce_dst[rr];
    int head = dst.head_block * kHeadsPerBlock + hrow, q_row = dst.q_row;
    if (dst.head_block < 0) {   // stacked unit: -head_block query rows of H heads each
        const int sub = hrow / H;
        if (sub >= -dst.head_block) return;
        head = hrow - sub * H;
        q_row += sub;
    }
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
    const float lse_val = denom > 0.0f ? m + log2f(denom) * 0.69314718055994531f : INFINITY;
    for (int d = 0; d < tgt.n_peers; ++d) {   // one destination, or every peer's gathered buffer
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(tgt.out[d]) + (size_t)q_row * stride_o_row + (size_t)head * stride_o_head;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint2 u;
            u.x = pack_bf16x2(acc[4 * v + 0] * inv, acc[4 * v + 1] * inv);
            u.y = pack_bf16x2(acc[4 * v + 2] * inv, acc[4 * v + 3] * inv);
            *reinterpret_cast<uint2*>(o + (v * 32 + lane) * 4) = u;
        }
        if (lane == 0 && tgt.lse[d] != nullptr) tgt.lse[d][(size_t)q_row * tgt.lse_stride_row + head] = lse_val;
    }
}

// ------------------------------------------------------------------ arrival flags of the fused all-gather
// After the kernels that stored this rank's rows into the peers' buffers: publish the step in every peer's
// flag array (system-scope release after a system-scope fence, so the rows are visible before the flag),
// then wait until every peer has published the same step here.  The wait is bounded (one second); on expiry
// the status word gets DSA_V32_ERR_DEVICE_WAIT and the kernel returns.
__global__ void __launch_bounds__(32) peer_signal_wait_kernel(const PeerSync s) {
    const int lane = threadIdx.x;
    __threadfence_system();
    if (lane < s.n_peers) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(s.flags[lane] + s.my_rank), "r"(s.step) : "memory");
        const uint32_t* mine = s.flags[s.my_rank] + lane;
        const uint64_t t0 = global_ns();
        bool ok = false;
        for (uint32_t it = 0; it < DSA_WAIT_LIMIT; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int32_t>(v - s.step) >= 0) {
                ok = true;
                break;
            }
            if (global_ns() - t0 > 1000000000ull) break;
            __nanosleep(200);
        }
        if (!ok) atomicExch(s.status, DSA_V32_ERR_DEVICE_WAIT);
    }
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

// ------------------------------------------------------------------ self-test of the bounded wait
// One warp waits, with a short budget, on an initialised barrier that nothing ever arrives at: the wait
// must give up, raise the CTA's abort flag and record DSA_V32_ERR_DEVICE_WAIT in the status word - the
// path every wait of the attention kernel takes when its peer never answers - and the kernel must exit
// normally.  result[0] = 1 when the wait returned false, result[1] = the abort flag it left.
__global__ void __launch_bounds__(32) wait_expiry_selftest_kernel(int32_t* status, int32_t* result, unsigned long long budget_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncwarp();
    const bool ok = __all_sync(0xffffffffu, mbar_wait_budget(smem_u32(&bar), 0, &abort_flag, budget_ns));
    __syncwarp();
    if (threadIdx.x == 0) {
        if (abort_flag) atomicExch(status, DSA_V32_ERR_DEVICE_WAIT);
        result[0] = ok ? 0 : 1;
        result[1] = abort_flag;
    }
}

// ------------------------------------------------------------------ launch helpers (called from capi.cu)
// The opt-in for more than 48 KB of dynamic shared memory is a per-device attribute of the kernel: it is
// set once for every device this process launches on (the current device at the time of the call).
template <bool kFp8, bool kExt>
static cudaError_t configure() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> guard(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(sparse_mla_kernel<kFp8, kExt>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<kFp8>::kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[dev] = true;
    return cudaSuccess;
}

template <bool kFp8>
static void fill_launch(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int num_lists, cudaStream_t stream) {
    cfg->gridDim = dim3(2 * num_lists, 1, 1);
    cfg->blockDim = dim3(Cfg<kFp8>::kThreads, 1, 1);
    cfg->dynamicSmemBytes = Cfg<kFp8>::kSmemBytes;
    cfg->stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 2;
}

// How many CTA pairs the device can keep resident at once (one work list per pair).
int max_resident_pairs(bool fp8, int* out) {
    cudaError_t e = fp8 ? configure<true, false>() : configure<false, false>();
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (fp8) {
        fill_launch<true>(&cfg, attr, 1, nullptr);
        e = cudaOccupancyMaxActiveClusters(&n, sparse_mla_kernel<true, false>, &cfg);
    } else {
        fill_launch<false>(&cfg, attr, 1, nullptr);
        e = cudaOccupancyMaxActiveClusters(&n, sparse_mla_kernel<false, false>, &cfg);
    }
    if (e != cudaSuccess) return (int)e;
    *out = n;
    return 0;
}

template <bool kFp8, bool kExt>
static cudaError_t launch_attn_t(int num_lists, const CUtensorMap& tq, const CUtensorMap& tkv, const CUtensorMap& ttail,
                                 const AttnParams& p, cudaStream_t stream) {
    cudaError_t e = configure<kFp8, kExt>();
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    fill_launch<kFp8>(&cfg, attr, num_lists, stream);
    return cudaLaunchKernelEx(&cfg, sparse_mla_kernel<kFp8, kExt>, tq, tkv, ttail, p);
}

// ext: the plan holds stacked items, or a sink / second pool is given
cudaError_t launch_attn(bool fp8, bool ext, int num_lists, const CUtensorMap& tq, const CUtensorMap& tkv, const CUtensorMap& ttail,
                        const AttnParams& p, cudaStream_t stream) {
    if (fp8) return ext ? launch_attn_t<true, true>(num_lists, tq, tkv, ttail, p, stream) : launch_attn_t<true, false>(num_lists, tq, tkv, ttail, p, stream);
    return ext ? launch_attn_t<false, true>(num_lists, tq, tkv, ttail, p, stream) : launch_attn_t<false, false>(num_lists, tq, tkv, ttail, p, stream);
}

cudaError_t launch_combine(const float* o_accum, const float* lse_accum, const int32_t* reduce_indptr,
                           const int32_t* reduce_slots, const ReduceDst* reduce_dst, int num_reduce_rows, const OutTargets& tgt,
                           int64_t stride_o_row, int64_t stride_o_head, int H, cudaStream_t stream) {
    if (num_reduce_rows <= 0) return cudaSuccess;
    dim3 grid(num_reduce_rows, kHeadsPerBlock / 8);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, combine_kernel, o_accum, lse_accum, reduce_indptr, reduce_slots, reduce_dst, tgt, stride_o_row,
                              stride_o_head, H);
}

// Pushes a contiguous block of this GPU's gathered buffer to the same place in every peer's (plain 16-byte
// stores through the peer mappings, all SMs): the sequence-sharded form of the fused all-gather.
struct PeerPush {
    int32_t n_peers, my_rank;
    const uint4* src;
    uint4* dst[DSA_V32_MAX_PEERS];
    int64_t n16;   // 16-byte words
};
__global__ void __launch_bounds__(512) peer_push_kernel(const PeerPush s) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < s.n16; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 v = s.src[i];
        for (int r = 0; r < s.n_peers; ++r)
            if (r != s.my_rank) s.dst[r][i] = v;
    }
}
cudaError_t launch_peer_push(int n_peers, int my_rank, const void* src, void* const* dst, int64_t bytes, cudaStream_t stream) {
    if (bytes <= 0 || n_peers <= 1) return cudaSuccess;
    PeerPush s;
    s.n_peers = n_peers;
    s.my_rank = my_rank;
    s.src = reinterpret_cast<const uint4*>(src);
    for (int r = 0; r < DSA_V32_MAX_PEERS; ++r) s.dst[r] = r < n_peers ? reinterpret_cast<uint4*>(dst[r]) : nullptr;
    s.n16 = bytes / 16;
    peer_push_kernel<<<148 * 2, 512, 0, stream>>>(s);
    return cudaGetLastError();
}

cudaError_t launch_peer_sync(const PeerSync& s, cudaStream_t stream) {
    peer_signal_wait_kernel<<<1, 32, 0, stream>>>(s);
    return cudaGetLastError();
}

cudaError_t launch_wait_selftest(int32_t* status, int32_t* result, unsigned long long budget_ns, cudaStream_t stream) {
    wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(status, result, budget_ns);
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
