// Host-side construction of the TMA tensor maps the sparse-MLA kernels take as
// __grid_constant__ parameters.  The driver entry point is resolved through the runtime so
// the library does not link libcuda directly.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace dsa {

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_tiled() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    }
    return fn;
}

// rank <= 3.  dims[0] is the contiguous dimension; strides_bytes[i] is the byte stride of
// dims[i+1] (multiples of 16).  Out-of-range elements read as zero.
inline int make_tmap(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    encode_tiled_fn fn = get_encode_tiled();
    if (!fn) return -1;
    cuuint64_t d[3];
    cuuint64_t s[2];
    cuuint32_t b[3];
    cuuint32_t e[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    CUresult r = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, e,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace dsa
