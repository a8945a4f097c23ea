// Top-k selection of the sparse-attention index lists: for every query row, the positions of the k largest
// indexer scores among the row's valid positions, as the int32 list the attention kernels consume (-1 padding).
// This is the output stage of the DSA indexer that produces `indices` upstream of the attention; the
// reference lab has no counterpart (its harness draws the lists at random, common/host.cc:239-261).
//
// One CTA per query row, exact radix select on order-preserving 32-bit keys: four passes of 8 bits narrow the
// k-th largest key down (256-bin histograms in shared memory over the candidates that match the prefix found
// so far), then one ordered pass writes every position whose key is above the threshold and the lowest
// positions among those equal to it, in ascending position order - the list is deterministic.  The row is
// read five times; at 128-512 KB it stays in L2, so the kernel is bound by L2 bandwidth and launch latency.
#include <cstdint>
#include <cuda_runtime.h>
#include "defs.h"

namespace dsa {

constexpr int kSelThreads = 512;

// float -> key with the same order as the values (NaN sorts lowest: it is never preferred)
__device__ __forceinline__ uint32_t order_key(float x) {
    if (x != x) return 0u;
    const uint32_t b = __float_as_uint(x);
    if (b == 0x80000000u) return 0x80000000u;   // -0.0 ties with +0.0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// exclusive prefix sum of one flag per thread over the block, in thread order; returns the block total too
__device__ __forceinline__ int block_scan_flag(bool flag, int* warp_sums, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t bal = __ballot_sync(0xffffffffu, flag);
    const int in_warp = __popc(bal & ((1u << lane) - 1u));
    if (lane == 0) warp_sums[warp] = __popc(bal);
    __syncthreads();
    int base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kSelThreads / 32; ++w) {
        const int c = warp_sums[w];
        if (w < warp) base += c;
        tot += c;
    }
    __syncthreads();
    total = tot;
    return base + in_warp;
}

__global__ void __launch_bounds__(kSelThreads) topk_select_kernel(const float* __restrict__ scores, int64_t stride_row,
                                                                   const int32_t* __restrict__ valid_len, int kv_len, int topk,
                                                                   int32_t* __restrict__ indices_out) {
    __shared__ int hist[256];
    __shared__ int warp_sums[kSelThreads / 32];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    const int q = blockIdx.x, tid = threadIdx.x;
    const float* row = scores + (size_t)q * stride_row;
    int32_t* out = indices_out + (size_t)q * topk;
    int n = valid_len ? valid_len[q] : kv_len;
    n = n < 0 ? 0 : (n > kv_len ? kv_len : n);
    const int k = topk < n ? topk : n;
    if (k == n) {   // everything valid is selected
        for (int i = tid; i < topk; i += kSelThreads) out[i] = i < n ? i : -1;
        return;
    }
    // ---- the k-th largest key, 8 bits at a time from the top
    uint32_t prefix = 0, mask = 0;
    int need = k;   // how many more to take among the candidates that match the prefix
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += kSelThreads) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kSelThreads) {
            const uint32_t key = order_key(row[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFFu], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int left = need, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= left) break;
                left -= hist[b];
            }
            s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
            s_need = left;
        }
        __syncthreads();
        prefix = s_prefix;
        need = s_need;
        mask |= 0xFFu << shift;
        __syncthreads();
    }
    // prefix = the threshold key; take every key above it and the `need` lowest positions equal to it
    int eq_base = 0, out_base = 0;
    for (int i0 = 0; i0 < n; i0 += kSelThreads) {
        const int i = i0 + tid;
        const uint32_t key = i < n ? order_key(row[i]) : 0u;
        const bool eq = i < n && key == prefix;
        int eq_total, take_total;
        const int eq_rank = block_scan_flag(eq, warp_sums, eq_total);
        const bool take = i < n && (key > prefix || (eq && eq_base + eq_rank < need));
        const int slot = block_scan_flag(take, warp_sums, take_total);
        if (take) out[out_base + slot] = i;
        eq_base += eq_total;
        out_base += take_total;
    }
    for (int i = k + tid; i < topk; i += kSelThreads) out[i] = -1;
}

cudaError_t launch_topk_select(const float* scores, int64_t stride_row, const int32_t* valid_len, int total_q, int kv_len, int topk,
                               int32_t* indices_out, cudaStream_t stream) {
    if (total_q <= 0) return cudaSuccess;
    topk_select_kernel<<<total_q, kSelThreads, 0, stream>>>(scores, stride_row, valid_len, kv_len, topk, indices_out);
    return cudaGetLastError();
}

}  // namespace dsa
