// Micro-benchmark behind the tile shape of the attention kernel: what one tcgen05.mma (cta_group::1, kind::f16,
// M = 128, K = 16) costs the issuing thread and the tensor pipe as a function of N, with A from tensor memory
// or from shared memory.  One CTA per SM; lane 0 of warp 0 issues `reps` instructions back to back into the
// same accumulator, commits, and waits (bounded) for the completion.  Operands are zeros.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue mma_issue.cu
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include "../ptx.cuh"
using namespace dsa;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

constexpr int kABytes = 128 * 128;       // 128 rows x 64 bf16, 128-byte swizzled rows
constexpr int kBBytes = 256 * 128;       // up to 256 rows x 64 bf16

// A_TMEM: A operand from tensor memory (columns 256..), else from shared memory.
template <int N, bool A_TMEM>
__global__ void __launch_bounds__(128, 1) k(int reps, long long* out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_base;
    __shared__ int abortf;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (kABytes + kBBytes) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        mbar_init(smem_u32(&done_bar), 1);
        abortf = 0;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base;
    {   // zero the TMEM columns used as A (and the accumulator, so no NaN patterns are read)
        uint32_t z[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = 0u;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        for (int c = 0; c < 512; c += 32) tmem_st32(lane_base + c, z);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    long long t_issue = 0, t_done = 0;
    if (warp == 0) {
        const uint32_t el = elect_one() ? 1u : 0u;
        constexpr uint32_t idesc = make_idesc_bf16(128, N, false);
        const uint64_t a_desc = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
        const uint64_t b_desc = make_smem_desc_sw128(smem_u32(smem + kABytes), 16, 1024);
        __syncwarp();
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
            const uint32_t ks = static_cast<uint32_t>(r & 3);   // the four K steps of a 64-column block
            if (A_TMEM) umma_ts_el(tmem, tmem + 256 + ks * 8, b_desc + ks * 2, idesc, 1u, el);
            else umma_ss_el(tmem, a_desc + ks * 2, b_desc + ks * 2, idesc, 1u, el);
        }
        const long long t1 = clock64();
        tc_commit_el(smem_u32(&done_bar), el);
        const bool ok = warp_wait(smem_u32(&done_bar), 0, &abortf);
        const long long t2 = clock64();
        t_issue = t1 - t0;
        t_done = ok ? t2 - t0 : -1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (tid == 0) {
        out[2 * blockIdx.x] = t_issue;
        out[2 * blockIdx.x + 1] = t_done;
    }
}

template <int N, bool A_TMEM>
int run(int reps) {
    long long* d;
    CK(cudaMalloc(&d, 148 * 16));
    const int smem = kABytes + kBBytes + 1024;
    CK(cudaFuncSetAttribute(k<N, A_TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    for (int rep = 0; rep < 2; ++rep) {
        k<N, A_TMEM><<<148, 128, smem>>>(reps, d);
        CK(cudaDeviceSynchronize());
    }
    long long h[296];
    CK(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
    double si = 0, sd = 0;
    bool bad = false;
    for (int i = 0; i < 148; ++i) {
        si += (double)h[2 * i];
        sd += (double)h[2 * i + 1];
        bad |= h[2 * i + 1] < 0;
    }
    const double ideal = 128.0 * N * 16 / 4096.0;   // cycles at 8192 dense bf16 FLOP per clock and SM
    printf("M=128 N=%3d K=16 A from %s: %5d instructions: issue %.1f clk each, complete %.1f clk each (ideal %.0f)%s\n", N,
           A_TMEM ? "TMEM" : "smem", reps, si / 148 / reps, sd / 148 / reps, ideal, bad ? "  [a wait expired]" : "");
    cudaFree(d);
    return 0;
}

int main() {
    for (int reps : {64, 512}) {
        run<32, true>(reps);
        run<64, true>(reps);
        run<128, true>(reps);
        run<256, true>(reps);
        run<32, false>(reps);
        run<64, false>(reps);
        run<128, false>(reps);
        run<256, false>(reps);
    }
    return 0;
}
