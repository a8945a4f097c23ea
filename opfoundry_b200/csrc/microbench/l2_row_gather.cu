// Micro-benchmark behind the roofline of the bf16 prefill: how fast all SMs together can pull random row slices
// out of an L2-resident table (the 4096-token prefill gathers 7.2 GB per step from a 4.7 MB cache), and how long
// a 20 KB tile takes to land, as a function of the tiles each SM keeps in flight.
// One CTA per SM; each of 8 loader warps copies rows of 512 or 640 bytes as 16-byte cp.async into shared memory
// (lane = row / 4, four lanes per row as in the kernel), `depth` tiles in flight per CTA.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o l2_row_gather l2_row_gather.cu
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include "../ptx.cuh"
using namespace dsa;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

constexpr int kRowBytes = 1152, kTileRows = 32, kTileBytes = 20480, kMaxDepth = 8;

__device__ __forceinline__ uint32_t rnd(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t x = a * 2654435761u ^ b * 40503u ^ c * 2246822519u;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    return x;
}

// slice_bytes: 512 (CTA 0) or 640 (CTA 1) per row; blockIdx parity picks which, as in a cluster pair.
__global__ void __launch_bounds__(256, 1) k(const uint8_t* table, int nrows, int tiles, int depth, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t full[kMaxDepth];
    __shared__ int abortf;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = blockIdx.x & 1;
    const int n_chunks = half ? 40 : 32;   // 16-byte chunks of the row slice
    if (tid == 0) {
        for (int i = 0; i < kMaxDepth; ++i) mbar_init(smem_u32(&full[i]), 128);   // four warps per tile, every lane arrives
        abortf = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const int grp = warp >> 2, l4 = warp & 3;      // two groups of four warps on alternate tiles
    const int r = 8 * l4 + (lane >> 2), c4 = lane & 3;
    long long lat_sum = 0;
    int lat_n = 0;
    const long long t0 = clock64();
    // tiles t = grp, grp + 2, ...: a tile's stage is reused `depth` tiles later, after its data has landed
    for (int t = grp; t < tiles; t += 2) {
        const int s = t % depth;
        if (t >= depth) {   // the tile that used this stage: wait for its data (this is the "landed" time)
            if (!warp_wait(smem_u32(&full[s]), ((t - depth) / depth) & 1, &abortf)) break;
        }
        const long long ti = clock64();
        const int row = (int)(rnd(blockIdx.x >> 1, t, r) % (uint32_t)nrows);
        const uint8_t* src = table + (size_t)row * kRowBytes + (half ? 512 : 0);
        const uint32_t dst_row = smem_u32(smem + s * kTileBytes) + r * 128;
#pragma unroll
        for (int j = 0; j < 10; ++j) {
            const int cc = c4 + 4 * j;
            if (cc < n_chunks) cp_async_16(dst_row + (cc >> 3) * 4096 + (((cc & 7) ^ (r & 7)) << 4), src + cc * 16, 16u);
        }
        cp_async_mbar_arrive_noinc(smem_u32(&full[s]));
        if ((t & 15) < 2) {   // sample the time from issue to landed on a few tiles (costs a wait)
            if (warp_wait(smem_u32(&full[s]), (t / depth) & 1, &abortf)) {
                lat_sum += clock64() - ti;
                ++lat_n;
            }
        }
    }
    // drain
    for (int i = 0; i < depth; ++i) {
        // every stage's last phase: tiles - 1 - i is the last tile of some stage
        const int t = tiles - 1 - i;
        if (t >= 0 && (t & 1) == grp) warp_wait(smem_u32(&full[t % depth]), (t / depth) & 1, &abortf);
    }
    const long long t1 = clock64();
    if (tid == 0) {
        out[3 * blockIdx.x] = t1 - t0;
        out[3 * blockIdx.x + 1] = lat_n ? lat_sum / lat_n : 0;
        out[3 * blockIdx.x + 2] = abortf;
    }
}

int main() {
    const int tiles = 2048;
    for (int nrows : {4096, 65536}) {
        uint8_t* table;
        CK(cudaMalloc(&table, (size_t)nrows * kRowBytes));
        CK(cudaMemset(table, 1, (size_t)nrows * kRowBytes));
        long long* d;
        CK(cudaMalloc(&d, 148 * 24));
        printf("---- table of %d rows (%.1f MB)\n", nrows, nrows * (double)kRowBytes / 1e6);
        for (int depth : {2, 4, 6, 8}) {   // even: a stage then always belongs to the same group of warps
            const int smem = kMaxDepth * kTileBytes + 1024;
            CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0); cudaEventCreate(&e1);
            k<<<148, 256, smem>>>(table, nrows, tiles, depth, d);
            CK(cudaDeviceSynchronize());
            cudaEventRecord(e0);
            k<<<148, 256, smem>>>(table, nrows, tiles, depth, d);
            cudaEventRecord(e1);
            CK(cudaDeviceSynchronize());
            float ms = 0;
            cudaEventElapsedTime(&ms, e0, e1);
            long long h[444];
            CK(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
            double cyc = 0, lat = 0;
            int bad = 0;
            for (int i = 0; i < 148; ++i) { cyc += (double)h[3 * i]; lat += (double)h[3 * i + 1]; bad |= (int)h[3 * i + 2]; }
            const double bytes = 74.0 * tiles * kTileRows * kRowBytes;   // a pair gathers 1152 bytes per row
            printf("%d tiles in flight per SM: %6.0f cycles per tile, issue-to-landed %5.0f cycles (sampled), aggregate %6.0f GB/s%s\n", depth,
                   cyc / 148 / tiles, lat / 148, bytes / (ms * 1e-3) / 1e9, bad ? "  [a wait expired]" : "");
        }
        cudaFree(table);
        cudaFree(d);
    }
    return 0;
}
