/*
 * dsa_v32.h - C ABI of the B200 (sm_100a) sparse-MLA attention library.
 *
 * The library replaces, for NVIDIA B200, the host launcher layer of the reference lab
 * opus_attn/dsa_v32 (kaiyang-1/OpFoundry): metadata -> decode kernel -> split-KV reduce.
 * Every entry point is extern "C", takes plain pointers and sizes, returns an int status
 * (0 = ok, < 0 = argument error, > 0 = a cudaError_t or a device-side status), never exits
 * the process and never allocates device memory: the caller owns every buffer, including the
 * split workspace, exactly as the reference's caller owns `mla_decode_plan`
 * (common/host.cc:69-88, :151-189).
 *
 * Shapes (one shared latent KV head):
 *   q        bf16 [total_q, H, 576]        576 = 512 latent + 64 rope; element strides given
 *   kv       bf16 rows of 576 values (1152 bytes), or
 *            fp8 rows of 656 bytes: 512 e4m3 | 4 x fp32 scale (one per 128 values) | 64 bf16 rope
 *   indices  int32 [total_q, topk]         token position inside the query's sequence, -1 = padding
 *   block_table int32 [num_seqs, block_table_stride] or NULL
 *            NULL : physical row = (query / s_q) * kv_batch_stride_rows + position
 *            else : physical row = block_table[query / s_q][position / page_block_size]
 *                                  * page_block_size + position % page_block_size
 *   out      bf16 [total_q, H, 512]        V = the first 512 values of the same KV row
 *   lse      fp32 [total_q, H]             natural log; may be NULL
 * A query whose list holds no valid position yields out = 0 and lse = +inf
 * (common/host.cc:486-490).  A position that is negative is treated as padding; a position
 * whose physical row lies outside [0, num_kv_rows) is never dereferenced and is masked too.
 */
#ifndef DSA_V32_H
#define DSA_V32_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSA_V32_D_QK 576
#define DSA_V32_D_V 512
#define DSA_V32_D_ROPE 64
#define DSA_V32_BF16_ROW_BYTES 1152
#define DSA_V32_FP8_ROW_BYTES 656

#define DSA_V32_KV_BF16 0
#define DSA_V32_KV_FP8 1

/* status codes (< 0: rejected before any launch) */
#define DSA_V32_OK 0
#define DSA_V32_ERR_NULL (-1)        /* a required pointer is NULL */
#define DSA_V32_ERR_SHAPE (-2)       /* H, topk, total_q, s_q or a stride is out of range */
#define DSA_V32_ERR_ALIGN (-3)       /* a pointer or stride breaks the 16-byte rule of the TMA engine */
#define DSA_V32_ERR_WORKSPACE (-4)   /* workspace missing, too small, or not planned for this shape */
#define DSA_V32_ERR_DTYPE (-5)       /* kv_dtype does not match the entry point */
#define DSA_V32_ERR_DRIVER (-6)      /* tensor-map creation failed or the driver entry point is missing */
#define DSA_V32_ERR_DEVICE_WAIT 1001 /* a bounded device-side wait ran out; results are invalid */

/*
 * One unit of work for one CTA pair: a contiguous slice [k_begin, k_end) of the top-k list of
 * one query row and one block of 128 heads.  Same role and size as the reference's
 * opus_mla_decode_work_info (common/defs.h:64-73).
 *   partial_slot < 0 : the slice is the whole list; out/lse are written directly.
 *   partial_slot >= 0: normalised fp32 partial output and its lse go to the workspace slot and are
 *                      merged by dsa_v32_combine.
 */
typedef struct dsa_v32_work_info {
    int32_t q_row;
    int32_t partial_slot;
    int32_t k_begin;
    int32_t k_end;
    int32_t head_block;
    int32_t reduce_row; /* index into the reduce tables, -1 when not split */
    int32_t stacked_rows; /* > 1: the item carries this many consecutive query rows of one sequence that share
                             one index list (MTP), stacked along the heads: tile row r = query q_row + r / H, head r % H */
    int32_t _pad;
} dsa_v32_work_info;

/*
 * Planner flag: limit the number of work lists a small problem is cut into, as the reference's metadata
 * kernel does with auto_split (common/get_mla_metadata.hpp:8-13): at most
 * round(1.2 * sqrt(total cost in tile steps * lists available)) lists are used.
 */
#define DSA_V32_PLAN_AUTO_SPLIT 1

/* Problem shape the planner needs (no data pointers). */
typedef struct dsa_v32_shape {
    int32_t total_q;   /* number of query rows = batches * s_q */
    int32_t H;         /* heads handled by this device */
    int32_t topk;      /* slots per query row */
    int32_t s_q;       /* query rows per sequence (1 = plain decode, 2 = one MTP token, ...) */
    int32_t num_sms;   /* 0 = ask the device */
    int32_t flags;     /* DSA_V32_PLAN_* bits, 0 = defaults */
    const int32_t* valid_len_hint; /* optional host array [total_q]: slots >= this are known to be -1 */
    const uint8_t* mtp_shared;     /* optional host array [total_q / s_q]: non-zero = the s_q query rows of the sequence
                                      carry the same index list; when s_q * H <= 128 (and H is a multiple of 8) they are
                                      planned as one item that gathers the rows once (the reference packs the s_q tokens
                                      of a batch into one qo tile the same way: common/defs.h:186-190) */
} dsa_v32_shape;

/* What dsa_v32_plan_info reports; all byte counts refer to the caller's workspace. */
typedef struct dsa_v32_plan_info {
    int64_t workspace_bytes;
    int32_t num_lists;    /* CTA pairs = work lists */
    int32_t num_works;
    int32_t num_partials; /* partial slots (each H_block x 128 heads x 512 fp32 + lse) */
    int32_t num_reduce_rows;
} dsa_v32_plan_info;

/*
 * Arguments of the attention kernels; the analogue of opus_mla_decode_kargs
 * (common/defs.h:109-131) with the per-query index list, block table and softmax scale the
 * reference keeps outside (CSR page table, scale fixed at 1/sqrt(576): common/host.cc:437).
 */
typedef struct dsa_v32_attn_args {
    const void* q;
    const void* kv;
    void* out;
    float* lse;
    const int32_t* indices;
    const int32_t* block_table;
    void* workspace;
    int64_t workspace_bytes;
    int64_t num_kv_rows;
    int64_t kv_batch_stride_rows;
    int64_t stride_q_row; /* elements */
    int64_t stride_q_head;
    int64_t stride_o_row;
    int64_t stride_o_head;
    int32_t total_q;
    int32_t H;
    int32_t topk;
    int32_t s_q;
    int32_t block_table_stride;
    int32_t page_block_size;
    int32_t kv_dtype; /* DSA_V32_KV_BF16 or DSA_V32_KV_FP8 */
    float sm_scale;
} dsa_v32_attn_args;

/* Library / build identification. */
int dsa_v32_abi_version(void);
const char* dsa_v32_error_string(int status);

/*
 * Sizes the workspace and the work list for a shape.  Host only.  Replaces the sizing half of
 * mla_decode_plan_create (common/host.cc:151-163).
 */
int dsa_v32_plan_info_get(const dsa_v32_shape* shape, dsa_v32_plan_info* info);

/*
 * Builds the work list and the reduce tables on the host and uploads them into the workspace
 * on `stream` (cudaStream_t passed as void*).  This is the metadata stage: it replaces
 * get_mla_metadata_kernel (common/get_mla_metadata.hpp:17-158) and, like it, depends only on
 * shapes, so it is run once per shape and kept out of timed loops (common/host.cc:266-283).
 */
int dsa_v32_plan(const dsa_v32_shape* shape, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Host-only form of the planner: serialises the plan header and tables (everything the device
 * needs except the partial buffers) into host memory.  `blob` may be NULL to query `needed`.
 * Needs no GPU when shape->num_sms is given; used by CPU tests of the planner.
 */
int dsa_v32_plan_host(const dsa_v32_shape* shape, void* blob, int64_t blob_bytes, int64_t* needed);

/* Copies the planned work list back to host memory (tests, debugging). */
int dsa_v32_plan_read(const void* workspace, int64_t workspace_bytes, dsa_v32_work_info* works_out, int32_t max_works,
                      int32_t* list_indptr_out, int32_t max_lists_plus1, void* stream);

/*
 * Forgets the plan recorded for `workspace` (call before freeing or re-using the memory for something
 * else; the library keeps the headers of the 256 most recently used plans).  The reference frees its plan
 * with mla_decode_plan_destroy (common/host.cc:180-189); here the memory is the caller's, only the
 * host-side record goes.  Returns DSA_V32_ERR_WORKSPACE when no plan is recorded for the pointer.
 */
int dsa_v32_plan_release(const void* workspace);

/*
 * The attention kernel alone (final rows written directly, split rows as fp32 partials).
 * Replaces mla_decode_launch for the bf16 traits (common/host.cc:39-65) / the mxfp8 traits
 * (common/host.cc:32-37).  Prefill is the same kernel with one query row per token and no
 * splitting; it has no counterpart in dsa_v32 and follows the launch shape of
 * opus_attn/dsa_v4/common/mla_v4_host.cc:629-631 (one work item per token and head block).
 */
int dsa_v32_decode_bf16(const dsa_v32_attn_args* args, void* stream);
int dsa_v32_decode_fp8(const dsa_v32_attn_args* args, void* stream);
int dsa_v32_prefill_bf16(const dsa_v32_attn_args* args, void* stream);

/* Merges split partials into out/lse.  Replaces mla_reduce_kernel (common/mla_reduce.hpp:158-184). */
int dsa_v32_combine(const dsa_v32_attn_args* args, void* stream);

/*
 * plan (optional) -> attention -> combine on one stream: the drop-in for
 * mla_decode_launch_pipeline (common/host.cc:114-138).  The return code covers argument checks and
 * launch errors only: the launches are asynchronous, so a bounded device-side wait that ran out
 * (DSA_V32_ERR_DEVICE_WAIT) is reported by dsa_v32_device_status, not here.
 */
int dsa_v32_decode_pipeline(const dsa_v32_attn_args* args, int run_plan, void* stream);

/*
 * The pipeline with the two features of the reference's v4 prefill kernels
 * (opus_attn/dsa_v4/common/mla_v4_host.cc:455-532, dsa_v4/README.md "Attention Model"):
 *   attn_sink   device array [H] of fp32 or NULL: exp(sink[h]) joins the softmax denominator of every query row
 *               of head h (scaled-score units, as in mla_v4_host.cc:469-472); lse includes it, and a row without
 *               any valid position gets out = 0, lse = sink[h].  (The running maximum of the scores stays the
 *               reference of the exponentials: a sink more than ~88 above every score of a row overflows.)
 *   kv2, pool_split, num_kv2_rows   a second pool of bf16 rows (the v4 "extend" rows: K/V produced by the current
 *               chunk, next to the cache of earlier state): slots k >= pool_split[q] of query row q hold PHYSICAL
 *               rows of kv2, the slots before it positions in args->kv as usual.  bf16 caches only.
 * The work list of a split query must start its first piece at slot 0 (every plan does).
 */
typedef struct dsa_v32_v4_ext {
    const float* attn_sink;
    const void* kv2;
    const int32_t* pool_split; /* device array [total_q] */
    int64_t num_kv2_rows;
} dsa_v32_v4_ext;
int dsa_v32_decode_pipeline_v4(const dsa_v32_attn_args* args, const dsa_v32_v4_ext* ext, void* stream);

/*
 * The pipeline fused with the all-gather that follows it when the heads or the sequences are sharded over
 * the GPUs of one box: instead of args->out / args->lse the kernels store every finished output row
 * straight into the gathered buffers of all peers (this GPU's own among them) through peer-mapped
 * pointers - plain global stores over NVLink that overlap the rest of the attention - and a one-warp kernel
 * then publishes "rank my_rank has written step `step`" in every peer's flag array and waits (bounded, one
 * second) until all peers have published the same step here.  When the call's work on `stream` is complete,
 * this GPU's gathered buffer holds every rank's slice.  The caller maps the buffers once (CUDA IPC or any
 * peer mapping; no multicast object is involved) and passes, for every peer r:
 *   out[r], lse[r]  where THIS rank's slice starts inside peer r's gathered out / lse buffer; the element
 *                   strides are args->stride_o_row / stride_o_head and lse_stride_row for all peers,
 *   flags[r]        peer r's array of DSA_V32_MAX_PEERS uint32 arrival flags (zero before the first step).
 * `step` must grow by one with every call.  When this rank's slice is one contiguous block of whole rows of
 * more than 64 heads (sequences sharded), the kernels write this GPU's own buffer and the block is pushed to the
 * peers by one copy kernel after them: an item's full 128 x 512 output stored to every peer from the
 * epilogue would hold up the hand-over between items.  No counterpart in the reference, which is single-GPU; the
 * collective it replaces is the NCCL all-gather of the head-sharded decode configuration.
 */
#define DSA_V32_MAX_PEERS 8
typedef struct dsa_v32_peer_outputs {
    int32_t num_peers; /* 1 .. DSA_V32_MAX_PEERS, this GPU included */
    int32_t my_rank;   /* index of this GPU among the peers */
    void* out[DSA_V32_MAX_PEERS];
    float* lse[DSA_V32_MAX_PEERS]; /* all NULL: lse is not produced */
    uint32_t* flags[DSA_V32_MAX_PEERS];
    int64_t lse_stride_row; /* elements between query rows of the gathered lse */
    uint32_t step;
    uint32_t _pad;
} dsa_v32_peer_outputs;
int dsa_v32_decode_pipeline_allgather(const dsa_v32_attn_args* args, const dsa_v32_peer_outputs* peers, void* stream);
/*
 * Helpers for the mapping: export the 64-byte CUDA IPC handle of the cudaMalloc allocation a device pointer
 * lies in, with the pointer's byte offset inside it; open such a handle exported by another process of the
 * box FOR THE CURRENT DEVICE, enabling peer access to the exporting GPU on the way
 * (kernels on this GPU may then store through the returned base address), and close it again.  A handle
 * names a whole allocation: open it once per process and add the buffer's offset inside it.
 */
int dsa_v32_ipc_export(const void* dev_ptr, void* handle64_out, int64_t* offset_out);
int dsa_v32_ipc_open(const void* handle64, void** base_out);
int dsa_v32_ipc_close(void* base);

/*
 * Host-buffer form of the pipeline, the call a serving loop makes once per step: copies this
 * step's queries and top-k lists from (pinned) host memory into args->q / args->indices, runs
 * attention + merge, and copies out / lse back to host memory, all asynchronously on `stream`.
 * The cache, block table and workspace in `args` stay resident on the device.  Any of the host
 * pointers may be NULL to skip that copy.  No counterpart in the reference, whose harness copies
 * with hipMemcpy around the launch (common/host.cc:640-645, :599-600).
 */
typedef struct dsa_v32_host_io {
    const void* q_host;          /* bf16, laid out like args->q */
    const int32_t* indices_host; /* [total_q, topk] */
    void* out_host;              /* bf16, laid out like args->out */
    float* lse_host;             /* [total_q, H] */
    int64_t q_bytes;
    int64_t out_bytes;
} dsa_v32_host_io;
int dsa_v32_decode_pipeline_host(const dsa_v32_attn_args* args, const dsa_v32_host_io* io, void* stream);
/*
 * The same step cut into `num_chunks` equal groups of sequences so that the PCIe copies overlap the
 * kernels: chunk c's queries and lists come in on an internal copy stream while chunk c-1 computes on
 * `stream`, and its outputs leave on a second copy stream while chunk c+1 computes.  `args` describes the
 * whole batch; `args->workspace` must be planned for ONE CHUNK's shape (total_q / num_chunks rows; the
 * chunks run one after the other on `stream` and share it).  total_q must be a multiple of num_chunks * s_q;
 * q / out / lse rows are taken as dense (row stride = stride_q_row / stride_o_row elements, lse [total_q, H]).
 * The host buffers must stay valid, and `stream` complete, before the results are read.  The copy streams
 * and events are created on the first call on a device and kept.
 */
int dsa_v32_decode_pipeline_host_chunked(const dsa_v32_attn_args* args, const dsa_v32_host_io* io, int32_t num_chunks,
                                         void* stream);
/*
 * The chunked step with `num_lanes` kernels in flight at once: lane l has its own workspace, planned for
 * one chunk's shape with shape.num_sms = (the device's SMs) / num_lanes, and its own internal compute stream;
 * it takes the chunks c with c % num_lanes == l.  A chunk's kernels then occupy only their share of the SMs,
 * so the start-up and tail of one chunk's kernels overlap the steady part of another's, and with enough
 * chunks the step takes about as long as the longer of its two PCIe directions.  args->workspace is not
 * used.  1 <= num_lanes <= 8, num_chunks >= num_lanes; everything else as for the chunked call.
 */
int dsa_v32_decode_pipeline_host_lanes(const dsa_v32_attn_args* args, const dsa_v32_host_io* io, int32_t num_chunks,
                                       void* const* lane_workspaces, const int64_t* lane_workspace_bytes, int32_t num_lanes,
                                       void* stream);

/*
 * The same pipeline for callers that cannot allocate device memory at all: code running where
 * cudaMalloc is off limits (a plugin loaded into a host that owns the memory pool, a real-time
 * serving loop that must not touch the allocator, a process whose memory was handed out at start-up).
 * It has no counterpart in the reference, whose harness always allocates its plan with hipMalloc.
 * args->workspace / workspace_bytes are ignored: the work list, reduce tables and split partials live
 * in a fixed array inside the library's device image, DSA_V32_STATIC_SCRATCH_BYTES long, which every
 * GPU that loads the library holds until the process exits.  Shapes whose plan does not fit are
 * rejected with DSA_V32_ERR_SCRATCH_TOO_SMALL before anything is launched.  The call allocates nothing
 * on the device (no cudaMalloc / cudaFree, no allocating library call).
 *   - The first call on a device looks up the array's device address (with that device current) and
 *     uploads the plan for the shape; a call with a new shape re-plans.  Make the first call for a
 *     shape before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents; the status
 *     word is cleared at the start of every call, everything else is rewritten before it is read.
 *     Two calls that overlap on the GPU (different streams, no dependency) race on it: serialise them.
 *   - Inputs and outputs are still the caller's buffers, exactly as in dsa_v32_decode_pipeline.
 */
#define DSA_V32_STATIC_SCRATCH_BYTES (48u << 20)
#define DSA_V32_ERR_SCRATCH_TOO_SMALL (-7)
int dsa_v32_decode_pipeline_static(const dsa_v32_attn_args* args, void* stream);
/* Device address of that array on the current device, NULL before the first static call there. */
void* dsa_v32_static_scratch_address(void);

/*
 * Reads (and clears) the device status word of the workspace after synchronising `stream`:
 * 0, or DSA_V32_ERR_DEVICE_WAIT when a bounded wait inside a kernel ran out.
 */
int dsa_v32_device_status(const dsa_v32_attn_args* args, void* stream);

/*
 * Self-test of the bounded device-side wait: launches one warp that waits, for `budget_us` microseconds
 * (1 .. 1000000), on an initialised barrier nothing arrives at.  The wait must run out, the kernel must
 * record DSA_V32_ERR_DEVICE_WAIT in the status word of `workspace` (any planned workspace) and exit
 * normally; result_dev[0] = 1 when the wait gave up, result_dev[1] = the abort flag it raised.  Afterwards
 * dsa_v32_device_status reports and clears the code.  Nothing traps and nothing is left waiting, so the
 * context stays usable.  No counterpart in the reference, whose kernels wait without a bound.
 */
int dsa_v32_selftest_wait_expiry(void* workspace, int32_t* result_dev, int64_t budget_us, void* stream);

/*
 * Debug entry point for index parity: writes, for every (query row, slot), the physical KV row
 * the kernel's translation resolves to (-1 for padding or an out-of-range row), using the
 * same device function as the attention kernel's loader warps.
 */
int dsa_v32_debug_rows(const dsa_v32_attn_args* args, int32_t* rows_out, void* stream);

/*
 * Producer of the index lists: for every query row the positions of the `topk` largest scores among the
 * row's first valid_len[q] positions (all kv_len when valid_len is NULL), written in ascending position
 * order and padded with -1; ties at the threshold go to the lower positions, NaN scores are never preferred.
 * scores: fp32 [total_q, kv_len] with row stride `stride_row` elements (the indexer's logits); all pointers
 * are device pointers.  This is the output stage of the DSA indexer upstream of the attention; the reference
 * has no counterpart (its harness draws the lists at random, common/host.cc:239-261).
 */
int dsa_v32_topk_select(const float* scores, int64_t stride_row, const int32_t* valid_len, int32_t total_q, int32_t kv_len,
                        int32_t topk, int32_t* indices_out, void* stream);

/*
 * KV-cache write path: quantises [num_rows, 512] fp32 latent values and [num_rows, 64] bf16
 * rope values (device pointers) into 656-byte fp8 cache rows at the given physical rows
 * (dst_rows == NULL: row i -> i).  Per 128 values: scale = amax / 448 (1.0 for an all-zero
 * group), byte = e4m3(x / scale) with round-to-nearest-even and saturation, the codec of
 * common/defs.h:11-38.  The reference only has a host-side generator (common/host.cc:207-237).
 */
int dsa_v32_pack_fp8_rows(const float* latent, const void* rope_bf16, const int64_t* dst_rows, void* kv_rows_out,
                          int64_t num_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSA_V32_H */
