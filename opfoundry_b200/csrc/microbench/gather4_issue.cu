// Micro-benchmark behind a design choice of the bf16 loaders: how fast one SM can get TMA tile::gather4 requests
// out, by issue pattern (every request moves one 128-byte block of four rows; a 32-row x 640-byte tile is 40
// requests).  Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o gather4_issue gather4_issue.cu -lcuda
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include "../ptx.cuh"
#include "../tmap.h"
using namespace dsa;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)
constexpr int kStages = 8, kRows = 32, kNB = 5, kTile = kNB * kRows * 128;

__device__ __forceinline__ int rnd_row(int cta, int tile, int r, int nrows) {
    uint32_t x = (uint32_t)cta * 2654435761u ^ (uint32_t)tile * 40503u ^ (uint32_t)r * 2246822519u;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    return (int)(x % (uint32_t)nrows);
}
// MODE 0: warp 0, lanes 0-7, 5 requests each.  MODE 1: warp 0, 32 lanes (8 row groups x 4 lane groups), blocks lg, lg+4.
// MODE 2: warps 0-3, lanes 0-1 of each: 2 row groups x 5 blocks.  MODE 3: warp 0 lane 0 issues all 40.
// MODE 4: warps 0-3, 8 lanes each, warp w issues blocks {w, w+4} for all 8 row groups.
template <int MODE>
__global__ void __launch_bounds__(320, 1) k(const __grid_constant__ CUtensorMap tm, int nrows, int tiles, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t full[kStages], empty[kStages];
    __shared__ int abortf;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kIssuers = (MODE == 2 || MODE == 4 || MODE == 7) ? 4 : (MODE == 5 ? 8 : (MODE == 6 ? 2 : 1));
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(smem_u32(&full[i]), kIssuers); mbar_init(smem_u32(&empty[i]), 1); }
        abortf = 0; fence_mbar_init();
    }
    __syncthreads();
    long long t0 = clock64();
    if (warp < kIssuers) {
        for (int t = 0; t < tiles; ++t) {
            const int s = t % kStages;
            if (!warp_wait(smem_u32(&empty[s]), ((t / kStages) & 1) ^ 1, &abortf)) break;
            const uint32_t bar = smem_u32(&full[s]);
            const uint32_t dst0 = smem_u32(smem + s * kTile);
            auto req = [&](int g, int kb) {
                tma_gather4(dst0 + kb * 4096 + g * 512, &tm, bar, kb * 64, rnd_row(blockIdx.x, t, 4 * g, nrows), rnd_row(blockIdx.x, t, 4 * g + 1, nrows),
                            rnd_row(blockIdx.x, t, 4 * g + 2, nrows), rnd_row(blockIdx.x, t, 4 * g + 3, nrows));
            };
            if (MODE == 0) {
                if (lane == 0) mbar_arrive_expect_tx(bar, kTile);
                __syncwarp();
                if (lane < 8) for (int kb = 0; kb < kNB; ++kb) req(lane, kb);
            } else if (MODE == 1) {
                if (lane == 0) mbar_arrive_expect_tx(bar, kTile);
                __syncwarp();
                const int g = lane & 7, lg = lane >> 3;
                req(g, lg);
                if (lg == 0) req(g, 4);
            } else if (MODE == 2) {
                if (lane == 0) mbar_arrive_expect_tx(bar, kTile / 4);
                __syncwarp();
                if (lane < 2) for (int kb = 0; kb < kNB; ++kb) req(2 * warp + lane, kb);
            } else if (MODE == 3) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar, kTile);
                    for (int g = 0; g < 8; ++g) for (int kb = 0; kb < kNB; ++kb) req(g, kb);
                }
            } else if (MODE == 5) {
                if (lane == 0) { mbar_arrive_expect_tx(bar, kTile / 8); for (int kb = 0; kb < kNB; ++kb) req(warp, kb); }
            } else if (MODE == 6) {
                if (lane == 0) mbar_arrive_expect_tx(bar, kTile / 2);
                __syncwarp();
                if (lane < 4) for (int kb = 0; kb < kNB; ++kb) req(4 * warp + lane, kb);
            } else if (MODE == 7) {
                if (lane == 0) { mbar_arrive_expect_tx(bar, kTile / 4); for (int g = 0; g < 2; ++g) for (int kb = 0; kb < kNB; ++kb) req(2 * warp + g, kb); }
            } else {
                const int nreq = (warp == 0) ? 2 : 1;
                if (lane == 0) mbar_arrive_expect_tx(bar, 8 * 512 * nreq);
                __syncwarp();
                if (lane < 8) { req(lane, warp); if (warp == 0) req(lane, 4); }
            }
        }
    } else if (warp == 8) {
        for (int t = 0; t < tiles; ++t) {
            const int s = t % kStages;
            if (!warp_wait(smem_u32(&full[s]), (t / kStages) & 1, &abortf)) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
        }
        if (lane == 0 && blockIdx.x == 0) out[0] = clock64() - t0;
    }
}
template <int MODE>
int run(const char* name, const CUtensorMap& tm, int nrows, long long* d) {
    const int smem = kStages * kTile + 2048, tiles = 400;
    CK(cudaFuncSetAttribute(k<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    k<MODE><<<148, 320, smem>>>(tm, nrows, tiles, d); CK(cudaDeviceSynchronize());
    cudaEventRecord(e0);
    k<MODE><<<148, 320, smem>>>(tm, nrows, tiles, d);
    cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    long long h; CK(cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost));
    printf("%-52s %7.0f cycles/tile (%.0f per request)  aggregate %.0f GB/s\n", name, (double)h / tiles, (double)h / tiles / 40.0,
           148.0 * tiles * kTile / (ms * 1e-3) / 1e9);
    return 0;
}
int bench(int nrows) {
    printf("---- table of %d rows (%.0f MB)\n", nrows, nrows * 1152.0 / 1e6);
    void* tab; CK(cudaMalloc(&tab, (size_t)nrows * 1152)); CK(cudaMemset(tab, 0, (size_t)nrows * 1152));
    long long* d; CK(cudaMalloc(&d, 64));
    CUtensorMap tm;
    const uint64_t dims[2] = {576, (uint64_t)nrows}; const uint64_t str[1] = {1152}; const uint32_t box[2] = {64, 1};
    if (make_tmap(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, tab, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) { printf("tmap failed\n"); return 1; }
    run<0>("1 warp, 8 lanes x 5 requests (as the kernel)", tm, nrows, d);
    run<2>("4 warps, 2 lanes x 5 requests", tm, nrows, d);
    run<5>("8 warps, 1 lane x 5 requests", tm, nrows, d);
    run<7>("4 warps, 1 lane x 10 requests", tm, nrows, d);
    CK(cudaFree(tab)); CK(cudaFree(d));
    return 0;
}
int main() {
    if (bench(65536)) return 1;
    if (bench(1 << 21)) return 1;
    return 0;
}
