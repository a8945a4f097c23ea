// Test infrastructure only (never shipped, never on the product path).
//
// Compiles the reference's own CPU implementation of the sparse-MLA decode path, unmodified,
// from where it lies (opus_attn/dsa_v32/common/host.cc, included below through the include
// path given on the command line) and exports its reference functions with C linkage so the
// CPU restatement in dsa_oracle.c can be pinned against them:
//   mla_decode_attention_ref_bf16   host.cc:508-548
//   mla_decode_attention_ref_fp8    host.cc:459-506
//   rand_vector / init_fp8_mla_split / init_kv_page_table   host.cc:191-261
//   float_to_fp8_e4m3 / fp8_e4m3_to_float                  defs.h:11-52
#define main reference_main
#include "common/host.cc"
#undef main

// host.cc only declares the device kernels; give them empty bodies so the harness code that
// launches them links.  They are never launched through this library.
template<class Traits> __global__ void opus_mla_decode_mxfp8_16mx8_32nx1_kernel(opus_mla_decode_mxfp8_kargs) {}
template<class Traits> __global__ void opus_mla_decode_a16w16_16mx4_64nx1_kernel(opus_mla_decode_kargs) {}
template<class Traits> __global__ void opus_mla_decode_a16w16_32mx1_16nx4_kernel(opus_mla_decode_kargs) {}
template<class Traits> __global__ void opus_mla_decode_a16w16_32mxt_32nx1_kernel(opus_mla_decode_kargs) {}
__global__ void get_mla_metadata_kernel(opus_mla_decode_metadata_kargs) {}
template<class Traits, int HEADS_PER_BLOCK> __global__ void mla_reduce_kernel(opus_mla_decode_reduce_kargs) {}

using RefBf16Traits = opus_mla_decode_a16w16_16mx4_64nx1_traits<>;
using RefFp8Traits  = opus_mla_decode_mxfp8_16mx8_32nx1_traits<>;

extern "C" {

int ref_main(int argc, char** argv) { return reference_main(argc, argv); }

void ref_attention_bf16(const void* q, const void* kv, void* out, float* lse,
                        const int* kv_indptr, const int* kv_indices, int B, int H, int seqlen_qo) {
    mla_decode_attention_ref_bf16<RefBf16Traits>(
        static_cast<const bf16_t*>(q), static_cast<const bf16_t*>(kv),
        static_cast<bf16_t*>(out), lse, kv_indptr, kv_indices, B, H, seqlen_qo);
}

void ref_attention_fp8(const void* q_nope, const uint8_t* q_scale, const void* q_rope,
                       const void* kv_nope, const uint8_t* kv_scale, const void* kv_rope,
                       void* out, float* lse, const int* kv_indptr, const int* kv_indices,
                       int B, int H, int seqlen_qo) {
    using T = RefFp8Traits;
    mla_decode_attention_ref_fp8<T>(
        static_cast<const typename T::D_NOPE*>(q_nope), q_scale, static_cast<const typename T::D_ROPE*>(q_rope),
        static_cast<const typename T::D_NOPE*>(kv_nope), kv_scale, static_cast<const typename T::D_ROPE*>(kv_rope),
        static_cast<typename T::D_OUT*>(out), lse, kv_indptr, kv_indices, B, H, seqlen_qo);
}

void ref_rand_bf16(void* ptr, size_t n) { rand_vector(static_cast<bf16_t*>(ptr), n); }

void ref_init_fp8_split(void* nope, uint8_t* scale, void* rope, size_t rows) {
    using T = RefFp8Traits;
    init_fp8_mla_split<T>(static_cast<typename T::D_NOPE*>(nope), scale,
                          static_cast<typename T::D_ROPE*>(rope), rows);
}

// Fills kv_indptr[B+1]; returns the number of indices written to kv_indices (capacity cap).
int ref_init_kv_page_table(int* kv_indptr, int* kv_indices, int cap, int B, int s, int varlen, unsigned seed) {
    std::vector<int> ip, ix;
    init_kv_page_table(ip, ix, B, s, varlen != 0, seed);
    if ((int)ix.size() > cap) return -1;
    std::copy(ip.begin(), ip.end(), kv_indptr);
    std::copy(ix.begin(), ix.end(), kv_indices);
    return (int)ix.size();
}

uint8_t ref_float_to_e4m3(float f) { return __builtin_bit_cast(uint8_t, float_to_fp8_e4m3(f)); }
float ref_e4m3_to_float(uint8_t b) { return fp8_e4m3_to_float(__builtin_bit_cast(fp8_t, b)); }
int ref_num_qo_tiles(int seqlen_qo, int H) { return mla_decode_num_qo_tiles(seqlen_qo, H); }
int ref_sizeof_work_info() { return (int)sizeof(opus_mla_decode_work_info); }

}  // extern "C"
