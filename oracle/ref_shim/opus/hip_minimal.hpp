// Test infrastructure only: stands in for the AMD `opus/hip_minimal.hpp` header so that the
// reference's host translation unit (opus_attn/dsa_v32/common/host.cc) compiles with nvcc.
// Only the CPU reference functions of that file are ever called through this build; the
// HIP runtime names below are mapped 1:1 to their CUDA runtime equivalents so the unused
// harness code still parses and links.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdio>

// nvcc cannot code-generate the native __bf16 in kernel template arguments; the CUDA type has
// the same round-to-nearest-even host conversions.
#define __bf16 __nv_bfloat16

#define hipError_t cudaError_t
#define hipSuccess cudaSuccess
#define hipGetErrorString cudaGetErrorString
#define hipGetLastError cudaGetLastError
#define hipMalloc cudaMalloc
#define hipFree cudaFree
#define hipMemcpy cudaMemcpy
#define hipMemset cudaMemset
#define hipMemcpyHostToDevice cudaMemcpyHostToDevice
#define hipMemcpyDeviceToHost cudaMemcpyDeviceToHost
#define hipDeviceSynchronize cudaDeviceSynchronize
#define hipEvent_t cudaEvent_t
#define hipEventCreate cudaEventCreate
#define hipEventRecord cudaEventRecord
#define hipEventSynchronize cudaEventSynchronize
#define hipEventElapsedTime cudaEventElapsedTime
#define hipEventDestroy cudaEventDestroy
