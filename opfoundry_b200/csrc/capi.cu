// extern "C" entry points declared in include/dsa_v32.h: argument checks, tensor-map creation,
// the plan registry and the launches.  Nothing here allocates device memory.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>
#include "defs.h"
#include "plan.h"
#include "tmap.h"

namespace dsa {
int max_resident_pairs(bool fp8, int* out);
cudaError_t launch_attn(bool fp8, bool ext, int num_lists, const CUtensorMap& tq, const CUtensorMap& tkv, const CUtensorMap& ttail,
                        const AttnParams& p, cudaStream_t stream);
cudaError_t launch_combine(const float* o_accum, const float* lse_accum, const int32_t* reduce_indptr,
                           const int32_t* reduce_slots, const ReduceDst* reduce_dst, int num_reduce_rows, const OutTargets& tgt,
                           int64_t stride_o_row, int64_t stride_o_head, int H, cudaStream_t stream);
cudaError_t launch_peer_sync(const PeerSync& s, cudaStream_t stream);
cudaError_t launch_peer_push(int n_peers, int my_rank, const void* src, void* const* dst, int64_t bytes, cudaStream_t stream);
cudaError_t launch_topk_select(const float* scores, int64_t stride_row, const int32_t* valid_len, int total_q, int kv_len, int topk,
                               int32_t* indices_out, cudaStream_t stream);
cudaError_t launch_debug_rows(const AttnParams& p, int total_q, int32_t* rows_out, cudaStream_t stream);
cudaError_t launch_wait_selftest(int32_t* status, int32_t* result, unsigned long long budget_ns, cudaStream_t stream);
cudaError_t launch_pack_fp8(const float* latent, const void* rope, const int64_t* dst_rows, void* out, int64_t num_rows,
                            cudaStream_t stream);

namespace {

// The host keeps the header of every planned workspace so a launch needs no device read-back.
// (The reference keeps the same facts in its host-side mla_decode_plan struct.)
struct Registry {
    std::mutex mu;
    struct Entry {
        const void* ws;
        WorkspaceHeader hdr;
        uint64_t last_use;
    };
    std::vector<Entry> entries;
    uint64_t clock = 0;
    static constexpr size_t kMaxEntries = 256;
    void put(const void* ws, const WorkspaceHeader& h) {
        std::lock_guard<std::mutex> g(mu);
        for (auto& e : entries)
            if (e.ws == ws) {
                e.hdr = h;
                e.last_use = ++clock;
                return;
            }
        if (entries.size() >= kMaxEntries) {   // drop the plan that has gone unused the longest
            size_t victim = 0;
            for (size_t i = 1; i < entries.size(); ++i)
                if (entries[i].last_use < entries[victim].last_use) victim = i;
            entries.erase(entries.begin() + victim);
        }
        entries.push_back(Entry{ws, h, ++clock});
    }
    bool get(const void* ws, WorkspaceHeader* h) {
        std::lock_guard<std::mutex> g(mu);
        for (auto& e : entries)
            if (e.ws == ws) {
                *h = e.hdr;
                e.last_use = ++clock;
                return true;
            }
        return false;
    }
    bool drop(const void* ws) {
        std::lock_guard<std::mutex> g(mu);
        for (size_t i = 0; i < entries.size(); ++i)
            if (entries[i].ws == ws) {
                entries.erase(entries.begin() + i);
                return true;
            }
        return false;
    }
};
Registry& registry() {
    static Registry r;
    return r;
}

// Processors the planner may count on: twice the number of CTA pairs (clusters of two) the device
// keeps resident at once, which can be below the SM count when a GPC holds an odd number of SMs.
int device_sm_count(int* out) {
    int a = 0, b = 0;
    int rc = max_resident_pairs(true, &a);
    if (rc) return rc;
    rc = max_resident_pairs(false, &b);
    if (rc) return rc;
    const int pairs = a < b ? a : b;
    if (pairs < 1) return DSA_V32_ERR_DRIVER;
    *out = 2 * pairs;
    return 0;
}

int resolve_sms(const dsa_v32_shape* shape, int* sms) {
    if (shape->num_sms > 0) {
        *sms = shape->num_sms;
        return 0;
    }
    return device_sm_count(sms);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_args(const dsa_v32_attn_args* a, int want_dtype, WorkspaceHeader* hdr, const WorkspaceHeader* known = nullptr) {
    if (!a || !a->q || !a->kv || !a->out || !a->indices || !a->workspace) return DSA_V32_ERR_NULL;
    if (a->kv_dtype != want_dtype) return DSA_V32_ERR_DTYPE;
    if (a->total_q <= 0 || a->H <= 0 || a->topk <= 0 || a->s_q <= 0 || a->total_q % a->s_q != 0) return DSA_V32_ERR_SHAPE;
    if (a->num_kv_rows <= 0 || a->num_kv_rows >= (int64_t(1) << 31) - 1) return DSA_V32_ERR_SHAPE;
    if (a->block_table != nullptr && (a->page_block_size <= 0 || a->block_table_stride <= 0)) return DSA_V32_ERR_SHAPE;
    if (a->block_table == nullptr && a->kv_batch_stride_rows < 0) return DSA_V32_ERR_SHAPE;
    if (a->stride_q_head < kDQK || a->stride_q_row < int64_t(a->H - 1) * a->stride_q_head + kDQK) return DSA_V32_ERR_SHAPE;
    if (a->stride_o_head < kDV || a->stride_o_row < int64_t(a->H - 1) * a->stride_o_head + kDV) return DSA_V32_ERR_SHAPE;
    if (!(a->sm_scale > 0.0f) || !std::isfinite(a->sm_scale)) return DSA_V32_ERR_SHAPE;
    // TMA: 16-byte aligned bases and strides; the epilogue stores 16-byte vectors
    if (!aligned16(a->q) || !aligned16(a->kv) || !aligned16(a->out)) return DSA_V32_ERR_ALIGN;
    if ((a->stride_q_head % 8) || (a->stride_q_row % 8) || (a->stride_o_head % 8) || (a->stride_o_row % 8)) return DSA_V32_ERR_ALIGN;
    if (reinterpret_cast<uintptr_t>(a->workspace) & 255u) return DSA_V32_ERR_ALIGN;
    if (known) *hdr = *known;
    else if (!registry().get(a->workspace, hdr)) return DSA_V32_ERR_WORKSPACE;
    if (hdr->total_q != a->total_q || hdr->H != a->H || hdr->topk != a->topk || hdr->s_q != a->s_q) return DSA_V32_ERR_WORKSPACE;
    if (hdr->total_bytes > a->workspace_bytes) return DSA_V32_ERR_WORKSPACE;
    return DSA_V32_OK;
}

// page size and, when it is a power of two, its log2 (the kernels then shift and mask instead of dividing)
void set_page(AttnParams* p, int page_block_size) {
    p->page_block_size = page_block_size > 0 ? page_block_size : 1;
    p->page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if (p->page_block_size == (1 << sh)) p->page_shift = sh;
}

void fill_params(const dsa_v32_attn_args* a, const WorkspaceHeader& h, AttnParams* p) {
    uint8_t* ws = reinterpret_cast<uint8_t*>(a->workspace);
    p->q = a->q;
    p->kv = a->kv;
    p->stride_q_row = a->stride_q_row;
    p->stride_q_head = a->stride_q_head;
    p->indices = a->indices;
    p->block_table = a->block_table;
    p->out = a->out;
    p->lse = a->lse;
    p->o_accum = reinterpret_cast<float*>(ws + h.off_o_accum);
    p->lse_accum = reinterpret_cast<float*>(ws + h.off_lse_accum);
    p->list_indptr = reinterpret_cast<const int32_t*>(ws + h.off_list_indptr);
    p->works = reinterpret_cast<const dsa_v32_work_info*>(ws + h.off_works);
    p->status = reinterpret_cast<int32_t*>(ws + offsetof(WorkspaceHeader, status));
    p->stride_o_row = a->stride_o_row;
    p->stride_o_head = a->stride_o_head;
    p->kv_batch_stride_rows = a->kv_batch_stride_rows;
    p->num_kv_rows = a->num_kv_rows;
    p->H = a->H;
    p->topk = a->topk;
    p->s_q = a->s_q;
    p->block_table_stride = a->block_table_stride;
    set_page(p, a->page_block_size);
    p->scale_log2 = a->sm_scale * 1.4426950408889634f;
    p->n_peers = 0;
    p->lse_stride_row = a->H;
    for (int i = 0; i < DSA_V32_MAX_PEERS; ++i) {
        p->out_peers[i] = nullptr;
        p->lse_peers[i] = nullptr;
    }
    p->attn_sink = nullptr;
    p->kv2 = nullptr;
    p->pool_split = nullptr;
    p->num_kv2_rows = 0;
}

int check_peers(const dsa_v32_peer_outputs* pe) {
    if (!pe) return DSA_V32_ERR_NULL;
    if (pe->num_peers < 1 || pe->num_peers > DSA_V32_MAX_PEERS || pe->my_rank < 0 || pe->my_rank >= pe->num_peers) return DSA_V32_ERR_SHAPE;
    if (pe->lse_stride_row <= 0) return DSA_V32_ERR_SHAPE;
    for (int i = 0; i < pe->num_peers; ++i) {
        if (!pe->out[i] || !pe->flags[i]) return DSA_V32_ERR_NULL;
        if (!aligned16(pe->out[i])) return DSA_V32_ERR_ALIGN;
    }
    return DSA_V32_OK;
}

// Encoded tensor maps depend only on (base pointer, extents, strides): a serving loop passes the same
// buffers every step, so the last few are kept instead of calling the driver's encoder on every launch.
struct TmapCache {
    struct Key {
        const void* base;
        uint64_t d0, d1, d2, s0, s1;
        uint32_t b0, b1, b2;
        int dtype, rank, swizzle;
        bool operator==(const Key& o) const {
            return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s0 == o.s0 && s1 == o.s1 && b0 == o.b0 &&
                   b1 == o.b1 && b2 == o.b2 && dtype == o.dtype && rank == o.rank && swizzle == o.swizzle;
        }
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        uint64_t last_use;
    };
    std::mutex mu;
    std::vector<Entry> entries;
    uint64_t clock = 0;
    int get(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims, const uint64_t* str,
            const uint32_t* box, CUtensorMapSwizzle swizzle) {
        Key k{base, dims[0], rank > 1 ? dims[1] : 0, rank > 2 ? dims[2] : 0, rank > 1 ? str[0] : 0, rank > 2 ? str[1] : 0,
              box[0], rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0, (int)dtype, rank, (int)swizzle};
        std::lock_guard<std::mutex> g(mu);
        for (auto& e : entries)
            if (e.key == k) {
                e.last_use = ++clock;
                *out = e.map;
                return 0;
            }
        CUtensorMap m;
        if (make_tmap(&m, dtype, rank, base, dims, str, box, swizzle)) return -1;
        if (entries.size() >= 32) {
            size_t victim = 0;
            for (size_t i = 1; i < entries.size(); ++i)
                if (entries[i].last_use < entries[victim].last_use) victim = i;
            entries.erase(entries.begin() + victim);
        }
        entries.push_back(Entry{k, m, ++clock});
        *out = m;
        return 0;
    }
};
TmapCache& tmap_cache() {
    static TmapCache c;
    return c;
}

int launch_attention(const dsa_v32_attn_args* a, int want_dtype, cudaStream_t stream, const WorkspaceHeader* known = nullptr,
                     const dsa_v32_peer_outputs* peers = nullptr, const dsa_v32_v4_ext* ext = nullptr) {
    WorkspaceHeader h;
    int rc = check_args(a, want_dtype, &h, known);
    if (rc) return rc;
    AttnParams p;
    fill_params(a, h, &p);
    if (peers) {
        p.n_peers = peers->num_peers;
        p.lse_stride_row = peers->lse_stride_row;
        for (int i = 0; i < peers->num_peers; ++i) {
            p.out_peers[i] = peers->out[i];
            p.lse_peers[i] = peers->lse[i];
        }
    }
    if (ext) {
        if (ext->kv2 != nullptr) {
            if (want_dtype != DSA_V32_KV_BF16) return DSA_V32_ERR_DTYPE;   // the second pool holds bf16 rows
            if (!ext->pool_split || ext->num_kv2_rows <= 0 || !aligned16(ext->kv2)) return DSA_V32_ERR_SHAPE;
        }
        p.attn_sink = ext->attn_sink;
        p.kv2 = ext->kv2;
        p.pool_split = ext->kv2 ? ext->pool_split : nullptr;
        p.num_kv2_rows = ext->num_kv2_rows;
    }
    // bf16 cache: the kernel reads Q and the cache rows with plain loads and takes no tensor map
    CUtensorMap tq, tkv, ttail;
    std::memset(&tq, 0, sizeof(tq));
    std::memset(&tkv, 0, sizeof(tkv));
    std::memset(&ttail, 0, sizeof(ttail));
    const bool fp8 = want_dtype == DSA_V32_KV_FP8;
    if (fp8) {
        {   // Q: the 64 rope columns of a head block, 128-byte swizzle (the latent columns go to TMEM by plain loads)
            const uint64_t dims[3] = {uint64_t(kDQK), uint64_t(a->H), uint64_t(a->total_q)};
            const uint64_t str[2] = {uint64_t(a->stride_q_head) * 2, uint64_t(a->stride_q_row) * 2};
            const uint32_t box[3] = {64, uint32_t(a->H < kHeadsPerBlock ? a->H : kHeadsPerBlock), 1};
            if (tmap_cache().get(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
                return DSA_V32_ERR_DRIVER;
        }
        // the 656-byte rows seen as 164 32-bit elements (a box may then be wider than 256 bytes):
        // CTA 0 gathers elements [0, 64) = its 256 latent bytes, CTA 1 elements [64, 164) = its 256 latent
        // bytes + the 16 scale bytes + the 128 rope bytes
        const uint64_t dims[2] = {uint64_t(kFp8RowBytes / 4), uint64_t(a->num_kv_rows)};
        const uint64_t str[1] = {uint64_t(kFp8RowBytes)};
        const uint32_t box_a[2] = {64, 1};
        const uint32_t box_b[2] = {100, 1};
        if (tmap_cache().get(&tkv, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a->kv, dims, str, box_a, CU_TENSOR_MAP_SWIZZLE_NONE))
            return DSA_V32_ERR_DRIVER;
        if (tmap_cache().get(&ttail, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a->kv, dims, str, box_b, CU_TENSOR_MAP_SWIZZLE_NONE))
            return DSA_V32_ERR_DRIVER;
    }
    const bool use_ext = h.has_stacked != 0 || p.attn_sink != nullptr || p.kv2 != nullptr || p.n_peers > 0;
    cudaError_t e = launch_attn(fp8, use_ext, h.num_lists, tq, tkv, ttail, p, stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int launch_merge(const dsa_v32_attn_args* a, cudaStream_t stream, const WorkspaceHeader* known = nullptr,
                 const dsa_v32_peer_outputs* peers = nullptr) {
    WorkspaceHeader h;
    if (!a) return DSA_V32_ERR_NULL;
    int rc = check_args(a, a->kv_dtype, &h, known);
    if (rc) return rc;
    OutTargets tgt;
    std::memset(&tgt, 0, sizeof(tgt));
    if (peers) {
        tgt.n_peers = peers->num_peers;
        tgt.lse_stride_row = peers->lse_stride_row;
        for (int i = 0; i < peers->num_peers; ++i) {
            tgt.out[i] = peers->out[i];
            tgt.lse[i] = peers->lse[i];
        }
    } else {
        tgt.n_peers = 1;
        tgt.lse_stride_row = a->H;
        tgt.out[0] = a->out;
        tgt.lse[0] = a->lse;
    }
    uint8_t* ws = reinterpret_cast<uint8_t*>(a->workspace);
    cudaError_t e = launch_combine(reinterpret_cast<const float*>(ws + h.off_o_accum),
                                   reinterpret_cast<const float*>(ws + h.off_lse_accum),
                                   reinterpret_cast<const int32_t*>(ws + h.off_reduce_indptr),
                                   reinterpret_cast<const int32_t*>(ws + h.off_reduce_slots),
                                   reinterpret_cast<const ReduceDst*>(ws + h.off_reduce_dst), h.num_reduce_rows, tgt,
                                   a->stride_o_row, a->stride_o_head, a->H, stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

}  // namespace
}  // namespace dsa

using namespace dsa;

extern "C" {

int dsa_v32_abi_version(void) { return 1; }

const char* dsa_v32_error_string(int status) {
    switch (status) {
        case DSA_V32_OK: return "ok";
        case DSA_V32_ERR_NULL: return "a required pointer is NULL";
        case DSA_V32_ERR_SHAPE: return "shape or stride out of range";
        case DSA_V32_ERR_ALIGN: return "pointer or stride not 16-byte aligned (workspace: 256)";
        case DSA_V32_ERR_WORKSPACE: return "workspace missing, too small, or not planned for this shape";
        case DSA_V32_ERR_DTYPE: return "kv_dtype does not match the entry point";
        case DSA_V32_ERR_DRIVER: return "tensor-map creation failed";
        case DSA_V32_ERR_SCRATCH_TOO_SMALL: return "the plan for this shape does not fit the library's static scratch array";
        case DSA_V32_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int dsa_v32_plan_info_get(const dsa_v32_shape* shape, dsa_v32_plan_info* info) {
    if (!shape || !info) return DSA_V32_ERR_NULL;
    int sms = 0;
    int rc = resolve_sms(shape, &sms);
    if (rc) return rc;
    HostPlan P;
    rc = build_plan(*shape, sms, P);
    if (rc) return rc;
    info->workspace_bytes = P.hdr.total_bytes;
    info->num_lists = P.hdr.num_lists;
    info->num_works = P.hdr.num_works;
    info->num_partials = P.hdr.num_partials;
    info->num_reduce_rows = P.hdr.num_reduce_rows;
    return DSA_V32_OK;
}

// Host-only variant used by the CPU tests: serialises header + tables into host memory.
int dsa_v32_plan_host(const dsa_v32_shape* shape, void* blob, int64_t blob_bytes, int64_t* needed) {
    if (!shape) return DSA_V32_ERR_NULL;
    int sms = 0;
    int rc = resolve_sms(shape, &sms);
    if (rc) return rc;
    HostPlan P;
    rc = build_plan(*shape, sms, P);
    if (rc) return rc;
    if (needed) *needed = plan_meta_bytes(P);
    if (!blob) return DSA_V32_OK;
    if (blob_bytes < plan_meta_bytes(P)) return DSA_V32_ERR_WORKSPACE;
    serialize_plan(P, reinterpret_cast<uint8_t*>(blob));
    return DSA_V32_OK;
}

int dsa_v32_plan(const dsa_v32_shape* shape, void* workspace, int64_t workspace_bytes, void* stream) {
    if (!shape || !workspace) return DSA_V32_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return DSA_V32_ERR_ALIGN;
    int sms = 0;
    int rc = resolve_sms(shape, &sms);
    if (rc) return rc;
    HostPlan P;
    rc = build_plan(*shape, sms, P);
    if (rc) return rc;
    if (workspace_bytes < P.hdr.total_bytes) return DSA_V32_ERR_WORKSPACE;
    std::vector<uint8_t> blob((size_t)plan_meta_bytes(P));
    serialize_plan(P, blob.data());
    // pageable source: the runtime stages the bytes before returning, so `blob` may go away
    cudaError_t e = cudaMemcpyAsync(workspace, blob.data(), blob.size(), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    registry().put(workspace, P.hdr);
    return DSA_V32_OK;
}

int dsa_v32_plan_read(const void* workspace, int64_t workspace_bytes, dsa_v32_work_info* works_out, int32_t max_works,
                      int32_t* list_indptr_out, int32_t max_lists_plus1, void* stream) {
    if (!workspace) return DSA_V32_ERR_NULL;
    WorkspaceHeader h;
    if (!registry().get(workspace, &h)) return DSA_V32_ERR_WORKSPACE;
    if (h.total_bytes > workspace_bytes) return DSA_V32_ERR_WORKSPACE;
    const uint8_t* ws = reinterpret_cast<const uint8_t*>(workspace);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    if (works_out) {
        if (max_works < h.num_works) return DSA_V32_ERR_SHAPE;
        e = cudaMemcpyAsync(works_out, ws + h.off_works, size_t(h.num_works) * sizeof(dsa_v32_work_info), cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return (int)e;
    }
    if (list_indptr_out) {
        if (max_lists_plus1 < h.num_lists + 1) return DSA_V32_ERR_SHAPE;
        e = cudaMemcpyAsync(list_indptr_out, ws + h.off_list_indptr, size_t(h.num_lists + 1) * 4, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return (int)e;
    }
    e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_decode_bf16(const dsa_v32_attn_args* args, void* stream) {
    return launch_attention(args, DSA_V32_KV_BF16, (cudaStream_t)stream);
}
int dsa_v32_decode_fp8(const dsa_v32_attn_args* args, void* stream) {
    return launch_attention(args, DSA_V32_KV_FP8, (cudaStream_t)stream);
}
int dsa_v32_prefill_bf16(const dsa_v32_attn_args* args, void* stream) {
    return launch_attention(args, DSA_V32_KV_BF16, (cudaStream_t)stream);
}

int dsa_v32_combine(const dsa_v32_attn_args* a, void* stream) { return launch_merge(a, (cudaStream_t)stream); }

int dsa_v32_decode_pipeline_v4(const dsa_v32_attn_args* a, const dsa_v32_v4_ext* ext, void* stream) {
    if (!a || !ext) return DSA_V32_ERR_NULL;
    int rc = launch_attention(a, a->kv_dtype, (cudaStream_t)stream, nullptr, nullptr, ext);
    if (rc) return rc;
    return launch_merge(a, (cudaStream_t)stream);
}

int dsa_v32_plan_release(const void* workspace) {
    if (!workspace) return DSA_V32_ERR_NULL;
    return registry().drop(workspace) ? DSA_V32_OK : DSA_V32_ERR_WORKSPACE;
}

int dsa_v32_decode_pipeline(const dsa_v32_attn_args* a, int run_plan, void* stream) {
    if (!a) return DSA_V32_ERR_NULL;
    if (run_plan) {
        dsa_v32_shape sh;
        std::memset(&sh, 0, sizeof(sh));
        sh.total_q = a->total_q;
        sh.H = a->H;
        sh.topk = a->topk;
        sh.s_q = a->s_q;
        int rc = dsa_v32_plan(&sh, a->workspace, a->workspace_bytes, stream);
        if (rc) return rc;
    }
    int rc = launch_attention(a, a->kv_dtype, (cudaStream_t)stream);
    if (rc) return rc;
    return dsa_v32_combine(a, stream);
}

int dsa_v32_decode_pipeline_allgather(const dsa_v32_attn_args* a, const dsa_v32_peer_outputs* peers, void* stream) {
    if (!a) return DSA_V32_ERR_NULL;
    int rc = check_peers(peers);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // Stores from the epilogue reach every peer while the attention runs - as long as an item's output is
    // small (head-sharded: few live rows per item).  When this rank owns whole rows of all heads (sequences
    // sharded: 128 rows x 512 columns per item to every peer) the remote stores would hold up the epilogue
    // between items; the slice is one contiguous block then, so the kernels write this GPU's own gathered
    // buffer and one copy kernel pushes the block to the peers after them.
    const bool contiguous_slice = a->stride_o_head == kDV && a->stride_o_row == int64_t(a->H) * kDV &&
                                  peers->lse_stride_row == a->H;
    const bool push_after = contiguous_slice && peers->num_peers > 1 && a->H > 64;
    dsa_v32_peer_outputs own = *peers;
    if (push_after) {
        own.num_peers = 1;
        own.my_rank = 0;
        own.out[0] = peers->out[peers->my_rank];
        own.lse[0] = peers->lse[peers->my_rank];
        own.flags[0] = peers->flags[peers->my_rank];
    }
    rc = launch_attention(a, a->kv_dtype, st, nullptr, push_after ? &own : peers);
    if (rc) return rc;
    rc = launch_merge(a, st, nullptr, push_after ? &own : peers);
    if (rc) return rc;
    cudaError_t e;
    if (push_after) {
        const int64_t o_bytes = int64_t(a->total_q) * a->stride_o_row * 2, l_bytes = int64_t(a->total_q) * a->H * 4;
        void* od[DSA_V32_MAX_PEERS];
        void* ld[DSA_V32_MAX_PEERS];
        bool with_lse = true;
        for (int r = 0; r < peers->num_peers; ++r) {
            od[r] = peers->out[r];
            ld[r] = peers->lse[r];
            with_lse = with_lse && peers->lse[r] != nullptr;
        }
        e = launch_peer_push(peers->num_peers, peers->my_rank, peers->out[peers->my_rank], od, o_bytes, st);
        if (e != cudaSuccess) return (int)e;
        if (with_lse && (l_bytes % 16) == 0 && aligned16(peers->lse[peers->my_rank])) {
            e = launch_peer_push(peers->num_peers, peers->my_rank, peers->lse[peers->my_rank], ld, l_bytes, st);
            if (e != cudaSuccess) return (int)e;
        } else if (with_lse) {
            for (int r = 0; r < peers->num_peers; ++r) {
                if (r == peers->my_rank) continue;
                e = cudaMemcpyAsync(peers->lse[r], peers->lse[peers->my_rank], size_t(l_bytes), cudaMemcpyDeviceToDevice, st);
                if (e != cudaSuccess) return (int)e;
            }
        }
    }
    PeerSync s;
    std::memset(&s, 0, sizeof(s));
    s.n_peers = peers->num_peers;
    s.my_rank = peers->my_rank;
    s.step = peers->step;
    for (int i = 0; i < peers->num_peers; ++i) s.flags[i] = peers->flags[i];
    s.status = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(a->workspace) + offsetof(WorkspaceHeader, status));
    e = launch_peer_sync(s, st);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_ipc_export(const void* dev_ptr, void* handle64_out, int64_t* offset_out) {
    if (!dev_ptr || !handle64_out || !offset_out) return DSA_V32_ERR_NULL;
    // the handle names the whole allocation the pointer lies in: find its base
    typedef CUresult (*range_fn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static range_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return DSA_V32_ERR_DRIVER;
        fn = reinterpret_cast<range_fn>(p);
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS) return DSA_V32_ERR_DRIVER;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
    if (e != cudaSuccess) return (int)e;
    std::memcpy(handle64_out, &h, sizeof(h));
    *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
    return DSA_V32_OK;
}

int dsa_v32_ipc_open(const void* handle64, void** base_out) {
    if (!handle64 || !base_out) return DSA_V32_ERR_NULL;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    std::memcpy(&h, handle64, sizeof(h));
    void* ptr = nullptr;
    // mapped for the CURRENT device, with peer access to the exporting GPU enabled as part of the call
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *base_out = ptr;
    return DSA_V32_OK;
}

int dsa_v32_ipc_close(void* base) {
    if (!base) return DSA_V32_ERR_NULL;
    cudaError_t e = cudaIpcCloseMemHandle(base);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_decode_pipeline_host(const dsa_v32_attn_args* a, const dsa_v32_host_io* io, void* stream) {
    if (!a || !io) return DSA_V32_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (io->q_host) {
        if (io->q_bytes <= 0) return DSA_V32_ERR_SHAPE;
        e = cudaMemcpyAsync(const_cast<void*>(a->q), io->q_host, (size_t)io->q_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return (int)e;
    }
    if (io->indices_host) {
        e = cudaMemcpyAsync(const_cast<int32_t*>(a->indices), io->indices_host, (size_t)a->total_q * a->topk * 4,
                            cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return (int)e;
    }
    int rc = dsa_v32_decode_pipeline(a, 0, stream);
    if (rc) return rc;
    if (io->out_host) {
        if (io->out_bytes <= 0) return DSA_V32_ERR_SHAPE;
        e = cudaMemcpyAsync(io->out_host, a->out, (size_t)io->out_bytes, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return (int)e;
    }
    if (io->lse_host && a->lse) {
        e = cudaMemcpyAsync(io->lse_host, a->lse, (size_t)a->total_q * a->H * 4, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return (int)e;
    }
    return DSA_V32_OK;
}

// ------------------------------------------------------------------ host-buffer pipeline in chunks
// Copy streams and events of the chunked host-buffer call, created once per device and kept.
namespace {
struct ChunkStreams {
    cudaStream_t in = nullptr, out = nullptr;
    std::vector<cudaStream_t> lane;   // compute streams of the lanes beyond the caller's own stream
    std::vector<cudaEvent_t> ev;      // start, done, then (copied-in, computed) per chunk
    cudaError_t ensure(size_t n_events, size_t n_lanes) {
        cudaError_t e;
        if (!in && (e = cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if (!out && (e = cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking)) != cudaSuccess) return e;
        while (lane.size() < n_lanes) {
            cudaStream_t x;
            if ((e = cudaStreamCreateWithFlags(&x, cudaStreamNonBlocking)) != cudaSuccess) return e;
            lane.push_back(x);
        }
        while (ev.size() < n_events) {
            cudaEvent_t x;
            if ((e = cudaEventCreateWithFlags(&x, cudaEventDisableTiming)) != cudaSuccess) return e;
            ev.push_back(x);
        }
        return cudaSuccess;
    }
};
std::mutex g_chunk_mu;
ChunkStreams g_chunk_streams[64];

// The step in `num_chunks` groups of sequences.  Lane l (its own compute stream and its own planned workspace)
// takes the chunks c with c % num_lanes == l; lane 0 runs on the caller's stream when there is only one lane.
int host_chunked_impl(const dsa_v32_attn_args* a, const dsa_v32_host_io* io, int32_t num_chunks, void* const* lane_ws,
                      const int64_t* lane_ws_bytes, int32_t num_lanes, void* stream) {
    if (num_chunks > 64 || a->s_q <= 0 || a->total_q % (num_chunks * a->s_q) != 0) return DSA_V32_ERR_SHAPE;
    if (!io->q_host || !io->indices_host || !io->out_host) return DSA_V32_ERR_NULL;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DSA_V32_ERR_SHAPE;
    std::lock_guard<std::mutex> guard(g_chunk_mu);
    ChunkStreams& cs = g_chunk_streams[dev];
    e = cs.ensure(2 + 2 * size_t(num_chunks), num_lanes > 1 ? size_t(num_lanes) : 0);
    if (e != cudaSuccess) return (int)e;
    cudaStream_t st = (cudaStream_t)stream;
    const int rows = a->total_q / num_chunks;          // query rows per chunk
    const int seqs = rows / a->s_q;
    const size_t q_row_bytes = size_t(a->stride_q_row) * 2, o_row_bytes = size_t(a->stride_o_row) * 2;
    // everything queued on `stream` before this call precedes the first copy and the first kernel
    if ((e = cudaEventRecord(cs.ev[0], st)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamWaitEvent(cs.in, cs.ev[0], 0)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamWaitEvent(cs.out, cs.ev[0], 0)) != cudaSuccess) return (int)e;
    if (num_lanes > 1)
        for (int l = 0; l < num_lanes; ++l)
            if ((e = cudaStreamWaitEvent(cs.lane[l], cs.ev[0], 0)) != cudaSuccess) return (int)e;
    // All copies in are queued first (they depend on nothing but the start), then the kernels and the copies
    // out chunk by chunk: a copy in never sits behind a copy out that is still waiting for its kernels.  The
    // index lists of all chunks go in one copy (a small copy costs 7-30 us on a busy link whatever its size).
    e = cudaMemcpyAsync(const_cast<int32_t*>(a->indices), io->indices_host, size_t(a->total_q) * a->topk * 4,
                        cudaMemcpyHostToDevice, cs.in);
    if (e != cudaSuccess) return (int)e;
    for (int c = 0; c < num_chunks; ++c) {
        const size_t r0 = size_t(c) * rows;
        e = cudaMemcpyAsync(const_cast<uint8_t*>(reinterpret_cast<const uint8_t*>(a->q)) + r0 * q_row_bytes,
                            reinterpret_cast<const uint8_t*>(io->q_host) + r0 * q_row_bytes, size_t(rows) * q_row_bytes,
                            cudaMemcpyHostToDevice, cs.in);
        if (e != cudaSuccess) return (int)e;
        if ((e = cudaEventRecord(cs.ev[2 + 2 * c], cs.in)) != cudaSuccess) return (int)e;
    }
    for (int c = 0; c < num_chunks; ++c) {
        const size_t r0 = size_t(c) * rows;
        const int l = c % num_lanes;
        cudaStream_t kst = num_lanes > 1 ? cs.lane[l] : st;
        dsa_v32_attn_args b = *a;
        b.total_q = rows;
        b.workspace = lane_ws[l];
        b.workspace_bytes = lane_ws_bytes[l];
        b.q = reinterpret_cast<const uint8_t*>(a->q) + r0 * q_row_bytes;
        b.out = reinterpret_cast<uint8_t*>(a->out) + r0 * o_row_bytes;
        b.lse = a->lse ? a->lse + r0 * a->H : nullptr;
        b.indices = a->indices + r0 * a->topk;
        if (a->block_table) {
            b.block_table = a->block_table + size_t(c) * seqs * a->block_table_stride;
        } else {   // contiguous cache: the chunk's sequences start kv_batch_stride_rows * seqs rows further on
            const size_t row_bytes = a->kv_dtype == DSA_V32_KV_FP8 ? size_t(DSA_V32_FP8_ROW_BYTES) : size_t(DSA_V32_BF16_ROW_BYTES);
            const int64_t skip = int64_t(c) * seqs * a->kv_batch_stride_rows;
            b.kv = reinterpret_cast<const uint8_t*>(a->kv) + size_t(skip) * row_bytes;
            b.num_kv_rows = a->num_kv_rows - skip;
        }
        // the chunk computes once its queries and lists are in, while the later chunks' are still on their way
        if ((e = cudaStreamWaitEvent(kst, cs.ev[2 + 2 * c], 0)) != cudaSuccess) return (int)e;
        int rc = dsa_v32_decode_pipeline(&b, 0, kst);
        if (rc) return rc;
        // ... and its outputs leave on the other copy stream while the next chunks compute
        if ((e = cudaEventRecord(cs.ev[3 + 2 * c], kst)) != cudaSuccess) return (int)e;
        if ((e = cudaStreamWaitEvent(cs.out, cs.ev[3 + 2 * c], 0)) != cudaSuccess) return (int)e;
        e = cudaMemcpyAsync(reinterpret_cast<uint8_t*>(io->out_host) + r0 * o_row_bytes, b.out, size_t(rows) * o_row_bytes,
                            cudaMemcpyDeviceToHost, cs.out);
        if (e != cudaSuccess) return (int)e;
    }
    // lse of all chunks in one copy: the copy stream has by now waited for every chunk's kernels
    if (io->lse_host && a->lse) {
        e = cudaMemcpyAsync(io->lse_host, a->lse, size_t(a->total_q) * a->H * 4, cudaMemcpyDeviceToHost, cs.out);
        if (e != cudaSuccess) return (int)e;
    }
    // the call's work is complete when `stream` is: it waits for the last copy out (which follows every kernel)
    if ((e = cudaEventRecord(cs.ev[1], cs.out)) != cudaSuccess) return (int)e;
    if ((e = cudaStreamWaitEvent(st, cs.ev[1], 0)) != cudaSuccess) return (int)e;
    return DSA_V32_OK;
}
}  // namespace

int dsa_v32_decode_pipeline_host_chunked(const dsa_v32_attn_args* a, const dsa_v32_host_io* io, int32_t num_chunks, void* stream) {
    if (!a || !io) return DSA_V32_ERR_NULL;
    if (num_chunks <= 1) return dsa_v32_decode_pipeline_host(a, io, stream);
    void* ws = a->workspace;
    const int64_t ws_bytes = a->workspace_bytes;
    return host_chunked_impl(a, io, num_chunks, &ws, &ws_bytes, 1, stream);
}

int dsa_v32_decode_pipeline_host_lanes(const dsa_v32_attn_args* a, const dsa_v32_host_io* io, int32_t num_chunks,
                                       void* const* lane_workspaces, const int64_t* lane_workspace_bytes, int32_t num_lanes,
                                       void* stream) {
    if (!a || !io || !lane_workspaces || !lane_workspace_bytes) return DSA_V32_ERR_NULL;
    if (num_lanes < 1 || num_lanes > 8 || num_chunks < num_lanes) return DSA_V32_ERR_SHAPE;
    for (int l = 0; l < num_lanes; ++l)
        if (!lane_workspaces[l]) return DSA_V32_ERR_NULL;
    return host_chunked_impl(a, io, num_chunks, lane_workspaces, lane_workspace_bytes, num_lanes, stream);
}

// ------------------------------------------------------------------ no-allocation variant
// Scratch for callers that may not allocate: lives in the library's device image.  In host code the
// name below is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[DSA_V32_STATIC_SCRATCH_BYTES];

namespace {
struct StaticScratchState {
    void* dev_ptr = nullptr;   // device address of g_static_scratch on this device
    dsa_v32_shape planned{};   // shape the array is currently planned for
    WorkspaceHeader hdr{};     // header of that plan (kept here: the static path does not depend on the plan registry)
    bool has_plan = false;
};
std::mutex g_static_mu;
StaticScratchState g_static_state[64];
}  // namespace

int dsa_v32_decode_pipeline_static(const dsa_v32_attn_args* a, void* stream) {
    if (!a) return DSA_V32_ERR_NULL;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DSA_V32_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    std::lock_guard<std::mutex> guard(g_static_mu);
    StaticScratchState& S = g_static_state[dev];
    if (S.dev_ptr == nullptr) {
        // once per device, with that device current
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr) return DSA_V32_ERR_DRIVER;
        S.dev_ptr = ptr;
    }
    const bool same = S.has_plan && S.planned.total_q == a->total_q && S.planned.H == a->H &&
                      S.planned.topk == a->topk && S.planned.s_q == a->s_q;
    if (!same) {
        dsa_v32_shape sh;
        std::memset(&sh, 0, sizeof(sh));
        sh.total_q = a->total_q;
        sh.H = a->H;
        sh.topk = a->topk;
        sh.s_q = a->s_q;
        int sms = 0;
        int rc = resolve_sms(&sh, &sms);
        if (rc) return rc;
        HostPlan P;
        rc = build_plan(sh, sms, P);
        if (rc) return rc;
        if (P.hdr.total_bytes > (int64_t)DSA_V32_STATIC_SCRATCH_BYTES) return DSA_V32_ERR_SCRATCH_TOO_SMALL;
        S.has_plan = false;
        std::vector<uint8_t> blob((size_t)plan_meta_bytes(P));
        serialize_plan(P, blob.data());
        // pageable source: the runtime stages the bytes before returning, so `blob` may go away
        e = cudaMemcpyAsync(S.dev_ptr, blob.data(), blob.size(), cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return (int)e;
        S.hdr = P.hdr;
        S.planned = sh;
        S.has_plan = true;
    }
    // the array keeps the last call's contents: the status word has to start at zero
    e = cudaMemsetAsync(reinterpret_cast<uint8_t*>(S.dev_ptr) + offsetof(WorkspaceHeader, status), 0, 4, st);
    if (e != cudaSuccess) return (int)e;
    dsa_v32_attn_args b = *a;
    b.workspace = S.dev_ptr;
    b.workspace_bytes = DSA_V32_STATIC_SCRATCH_BYTES;
    int rc = launch_attention(&b, b.kv_dtype, st, &S.hdr);
    if (rc) return rc;
    return launch_merge(&b, st, &S.hdr);
}

// Device address of the static scratch on the current device (after the first static call); lets a
// caller read the status word with dsa_v32_device_status by passing it as args->workspace.
void* dsa_v32_static_scratch_address(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> guard(g_static_mu);
    return g_static_state[dev].dev_ptr;
}

int dsa_v32_device_status(const dsa_v32_attn_args* a, void* stream) {
    if (!a || !a->workspace) return DSA_V32_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* dev = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(a->workspace) + offsetof(WorkspaceHeader, status));
    int32_t v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, dev, 4, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    if (v != 0) {
        e = cudaMemsetAsync(dev, 0, 4, st);
        if (e != cudaSuccess) return (int)e;
    }
    return v;
}

int dsa_v32_selftest_wait_expiry(void* workspace, int32_t* result_dev, int64_t budget_us, void* stream) {
    if (!workspace || !result_dev) return DSA_V32_ERR_NULL;
    if (budget_us <= 0 || budget_us > 1000000) return DSA_V32_ERR_SHAPE;   // at most a second
    int32_t* status = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(workspace) + offsetof(WorkspaceHeader, status));
    cudaError_t e = launch_wait_selftest(status, result_dev, (unsigned long long)budget_us * 1000ull, (cudaStream_t)stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_debug_rows(const dsa_v32_attn_args* a, int32_t* rows_out, void* stream) {
    if (!a || !rows_out || !a->indices) return DSA_V32_ERR_NULL;
    if (a->total_q <= 0 || a->topk <= 0 || a->s_q <= 0) return DSA_V32_ERR_SHAPE;
    AttnParams p;
    std::memset(&p, 0, sizeof(p));
    p.indices = a->indices;
    p.block_table = a->block_table;
    p.kv_batch_stride_rows = a->kv_batch_stride_rows;
    p.num_kv_rows = a->num_kv_rows;
    p.topk = a->topk;
    p.s_q = a->s_q;
    p.block_table_stride = a->block_table_stride;
    set_page(&p, a->page_block_size);
    cudaError_t e = launch_debug_rows(p, a->total_q, rows_out, (cudaStream_t)stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_topk_select(const float* scores, int64_t stride_row, const int32_t* valid_len, int32_t total_q, int32_t kv_len,
                        int32_t topk, int32_t* indices_out, void* stream) {
    if (!scores || !indices_out) return DSA_V32_ERR_NULL;
    if (total_q < 0 || kv_len <= 0 || topk <= 0 || stride_row < kv_len) return DSA_V32_ERR_SHAPE;
    cudaError_t e = launch_topk_select(scores, stride_row, valid_len, total_q, kv_len, topk, indices_out, (cudaStream_t)stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

int dsa_v32_pack_fp8_rows(const float* latent, const void* rope_bf16, const int64_t* dst_rows, void* kv_rows_out,
                          int64_t num_rows, void* stream) {
    if (!latent || !rope_bf16 || !kv_rows_out) return DSA_V32_ERR_NULL;
    if (num_rows < 0) return DSA_V32_ERR_SHAPE;
    if (!aligned16(latent) || (reinterpret_cast<uintptr_t>(rope_bf16) & 3u) || (reinterpret_cast<uintptr_t>(kv_rows_out) & 3u))
        return DSA_V32_ERR_ALIGN;
    cudaError_t e = launch_pack_fp8(latent, rope_bf16, dst_rows, kv_rows_out, num_rows, (cudaStream_t)stream);
    return e == cudaSuccess ? DSA_V32_OK : (int)e;
}

}  // extern "C"
