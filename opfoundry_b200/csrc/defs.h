// Internal definitions shared by the host launcher, the planner and the kernels.
#pragma once
#include <cstdint>
#include "../../include/dsa_v32.h"

namespace dsa {

constexpr int kDQK = DSA_V32_D_QK;      // 576
constexpr int kDV = DSA_V32_D_V;        // 512
constexpr int kDRope = DSA_V32_D_ROPE;  // 64
constexpr int kHeadsPerBlock = 128;     // MMA M: one head per TMEM lane
constexpr int kDvHalf = 256;            // output columns accumulated by one CTA of a pair
constexpr int kTileRows = 32;           // top-k slots per pipeline step
constexpr int kFp8RowBytes = DSA_V32_FP8_ROW_BYTES;

constexpr uint32_t kWorkspaceMagic = 0x44534133u;  // "DSA3"

// First 256 bytes of the caller's workspace (device memory); everything else is addressed by
// the byte offsets stored here.
struct WorkspaceHeader {
    uint32_t magic;
    int32_t total_q, H, topk, s_q;
    int32_t num_lists, num_works, num_partials, num_reduce_rows, num_head_blocks;
    int32_t status;  // device status word, 0 = ok
    int32_t has_stacked;  // 1 when some work item stacks several query rows
    int64_t off_list_indptr, off_works, off_reduce_indptr, off_reduce_slots, off_reduce_dst;
    int64_t off_o_accum, off_lse_accum, total_bytes;
};
static_assert(sizeof(WorkspaceHeader) <= 256, "header must fit its slot");

// Where a merged row goes: query row and head block of a split unit.
struct ReduceDst {
    int32_t q_row;
    int32_t head_block;   // >= 0: head block; < 0: minus the number of stacked query rows of the unit (head block 0)
};

// Kernel parameters (passed by value next to the tensor maps).
struct AttnParams {
    const void* kv;    // the cache (read directly for the row scales of an fp8 cache)
    const void* q;     // bf16 [total_q][H][576] with the element strides below (read directly for a bf16 cache)
    int64_t stride_q_row, stride_q_head;
    const int32_t* indices;
    const int32_t* block_table;
    void* out;     // bf16
    float* lse;
    float* o_accum;    // [num_partials][128][512] fp32, normalised partial outputs
    float* lse_accum;  // [num_partials][128]      fp32, natural-log lse or -FLT_MAX when empty
    const int32_t* list_indptr;
    const dsa_v32_work_info* works;
    int32_t* status;
    int64_t stride_o_row, stride_o_head;
    int64_t kv_batch_stride_rows;
    int64_t num_kv_rows;
    int32_t H, topk, s_q, block_table_stride, page_block_size;
    int32_t page_shift;  // log2(page_block_size) when that is a power of two, else -1
    float scale_log2;  // sm_scale * log2(e)
    // fused all-gather: when n_peers > 0 finished rows go to every peer's gathered buffer instead of out / lse
    int32_t n_peers;
    int64_t lse_stride_row;   // elements between query rows of lse (H without peers)
    void* out_peers[DSA_V32_MAX_PEERS];
    float* lse_peers[DSA_V32_MAX_PEERS];
    // v4-style extensions (NULL = off): attention sink per head; second pool of bf16 rows for the slots at or
    // beyond pool_split[query row], indexed by physical row
    const float* attn_sink;
    const void* kv2;
    const int32_t* pool_split;
    int64_t num_kv2_rows;
};

// Destinations of the merge kernel (same convention as AttnParams).
struct OutTargets {
    int32_t n_peers;
    int64_t lse_stride_row;
    void* out[DSA_V32_MAX_PEERS];
    float* lse[DSA_V32_MAX_PEERS];
};

// Arrival flags of the fused all-gather: flags[r] = peer r's array, one word per sending rank.
struct PeerSync {
    int32_t n_peers, my_rank;
    uint32_t step;
    uint32_t* flags[DSA_V32_MAX_PEERS];
    int32_t* status;
};

}  // namespace dsa
