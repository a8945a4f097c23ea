/*
 * TEST INFRASTRUCTURE ONLY.  CPU oracle for the sparse-MLA (DeepSeek sparse attention)
 * decode / prefill path.  Nothing in the shipped library links, loads or calls this file;
 * it exists so the CUDA kernels can be checked against the reference's arithmetic.
 *
 * It is a plain-C restatement of the reference's CPU implementation
 * (kaiyang-1/OpFoundry, opus_attn/dsa_v32):
 *
 *   e4m3 codec ............ common/defs.h:11-38 (encode), :40-52 (decode)
 *   per-(query, head) math  common/host.cc:431-457  mla_decode_attention_compute
 *   bf16 driver ........... common/host.cc:508-548  mla_decode_attention_ref_bf16
 *   fp8 driver ............ common/host.cc:459-506  mla_decode_attention_ref_fp8
 *   row dequantisation .... common/host.cc:418-429  dequant_mla_row_fp8
 *   empty selection ....... common/host.cc:486-490, :530-534  (out = 0, lse = +inf)
 *   worker threads ........ common/parallel.h:11-57
 *
 * extended to the inputs the CUDA path takes: a per-query top-k list of int32 token positions
 * with -1 as padding (anywhere in the list), an optional paged block table, a caller-supplied
 * softmax scale, and the packed fp8 cache row (512 e4m3 | 4 fp32 scales, one per 128 | 64 bf16).
 *
 * Arithmetic order is the reference's, element for element:
 *   s_p   = (sum_{d ascending} q_d * k_pd) * scale            fp32, multiply then add, no FMA
 *   m     = max_p s_p ;  e_p = expf(s_p - m) ;  L = sum_{p ascending} e_p
 *   lse   = logf(L) + m
 *   P_p   = float(bf16(e_p / L))
 *   out_d = bf16(sum_{p ascending} P_p * kv_pd),  d < 512
 * Heads are evaluated eight at a time and output columns are vectorised, which changes
 * which independent sums run side by side but not the order of operations inside any sum,
 * so results are bit-identical to the reference functions (this is checked by the tests
 * against a build of the reference's own host.cc).  Build with -ffp-contract=off.
 *
 * As in opus_attn/dsa_v41/common/mla_v41_host.cc:458-516, a query's selected rows are
 * converted to fp32 once and shared by all of its heads.
 */
#define _GNU_SOURCE
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define D_QK 576
#define D_V 512
#define D_ROPE 64
#define FP8_ROW_BYTES 656 /* 512 e4m3 + 4 fp32 + 64 bf16 */
#define HEAD_GROUP 8

/* ---------------------------------------------------------------- scalar codecs */

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, the conversion static_cast<bf16_t>(float) performs on the host */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* defs.h:11-38: RNE, saturates to +-448 (0x7E), NaN/Inf -> 0x7F, subnormal step 2^-9 */
uint8_t dsa_oracle_f32_to_e4m3(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    const uint32_t mag = bits & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) return (uint8_t)(sign | 0x7Fu);
    if (mag >= 0x43E00000u) return (uint8_t)(sign | 0x7Eu);
    const int exp = (int)(mag >> 23) - 127;
    uint8_t payload;
    uint32_t dropped, halfway;
    if (exp >= -6) {
        const uint32_t mant = mag & 0x7FFFFFu;
        payload = (uint8_t)(((exp + 7) << 3) | (mant >> 20));
        dropped = mant & 0xFFFFFu;
        halfway = 0x80000u;
    } else {
        const int shift = -exp - 6;
        if (shift > 11) return sign;
        const uint32_t mant = (mag & 0x7FFFFFu) | 0x800000u;
        const uint32_t width = 20u + (uint32_t)shift;
        payload = (uint8_t)(mant >> width);
        dropped = mant & ((1u << width) - 1u);
        halfway = 1u << (width - 1u);
    }
    if (dropped > halfway || (dropped == halfway && (payload & 1u))) payload++;
    return (uint8_t)(sign | payload);
}

/* defs.h:40-52 */
float dsa_oracle_e4m3_to_f32(uint8_t b) {
    const uint32_t sign = (uint32_t)(b & 0x80u) << 24;
    const uint32_t exp = (b >> 3) & 0x0Fu;
    const uint32_t mant = b & 0x07u;
    uint32_t u;
    float f;
    if (exp == 0x0Fu && mant == 0x07u) {
        u = sign | 0x7FC00000u;
        memcpy(&f, &u, 4);
        return f;
    }
    if (exp == 0) {
        const float m = (float)mant * 0x1p-9f;
        return (b & 0x80u) ? -m : m;
    }
    u = sign | ((exp + 120u) << 23) | (mant << 20);
    memcpy(&f, &u, 4);
    return f;
}

uint16_t dsa_oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
float dsa_oracle_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }

/*
 * Packs one cache row in the fp8 format: for each group of 128 latent values
 * scale = amax / 448 (fp32; 1.0 when the group is all zero), bytes = e4m3(x / scale);
 * then the four scales, then 64 rope values already in bf16.
 */
void dsa_oracle_pack_fp8_rows(const float* latent, const uint16_t* rope_bf16, uint8_t* rows_out,
                              int64_t num_rows) {
    for (int64_t r = 0; r < num_rows; ++r) {
        const float* x = latent + r * D_V;
        uint8_t* row = rows_out + r * FP8_ROW_BYTES;
        float scales[4];
        for (int g = 0; g < 4; ++g) {
            float amax = 0.0f;
            for (int i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(x[g * 128 + i]));
            const float scale = (amax > 0.0f) ? amax / 448.0f : 1.0f;
            scales[g] = scale;
            for (int i = 0; i < 128; ++i) row[g * 128 + i] = dsa_oracle_f32_to_e4m3(x[g * 128 + i] / scale);
        }
        memcpy(row + D_V, scales, 16);
        memcpy(row + D_V + 16, rope_bf16 + r * D_ROPE, D_ROPE * 2);
    }
}

/* host.cc:418-429 with an fp32 scale per 128 values instead of an E8M0 byte per 32 */
static void dequant_row_fp8(const uint8_t* row, float* out) {
    float scales[4];
    memcpy(scales, row + D_V, 16);
    for (int d = 0; d < D_V; ++d) out[d] = dsa_oracle_e4m3_to_f32(row[d]) * scales[d / 128];
    const uint16_t* rope = (const uint16_t*)(row + D_V + 16);
    for (int j = 0; j < D_ROPE; ++j) out[D_V + j] = bf16_to_f32(rope[j]);
}

void dsa_oracle_dequant_fp8_rows(const uint8_t* rows, float* out, int64_t num_rows) {
    for (int64_t r = 0; r < num_rows; ++r) dequant_row_fp8(rows + r * FP8_ROW_BYTES, out + r * D_QK);
}

/* ---------------------------------------------------------------- per-query work */

typedef struct {
    const uint16_t* q;
    int64_t q_stride_q, q_stride_h; /* elements */
    const uint8_t* kv;
    int kv_is_fp8;
    int64_t kv_row_bytes;
    int64_t num_kv_rows;
    int64_t kv_batch_stride_rows; /* used when block_table == NULL */
    const int32_t* indices;
    int topk;
    const int32_t* block_table;
    int block_table_stride;
    int page_block_size;
    int s_q;
    float sm_scale;
    uint16_t* out; /* [total_q, H, 512] bf16 */
    float* lse;    /* [total_q, H] */
    int32_t* rows_dbg; /* optional [total_q, topk]: physical row per slot, -1 for padding */
    int total_q, H;
    const int32_t* subset;
    int n_items;
    /* v4-style extensions (opus_attn/dsa_v4/common/mla_v4_host.cc:455-532): attention sink, second KV pool */
    const float* attn_sink;     /* [H] or NULL: joins the row maximum and the denominator (mla_v4_host.cc:469-472) */
    const uint8_t* kv2;         /* second pool (bf16 rows) or NULL */
    int64_t num_kv2_rows;
    const int32_t* pool_split;  /* [total_q]: slots >= pool_split[q] index kv2 directly by physical row */
    /* shared state */
    volatile int next;
    volatile int error;
} job_t;

/* s[h] = (sum_d qT[d][h] * k[d]) for HEAD_GROUP heads at once; each sum runs d ascending. */
__attribute__((target_clones("avx2", "default"))) static void
dots_group(const float* qT, const float* kv_dense, int n, float scale, float* scores /* [HEAD_GROUP][n] */) {
    for (int p = 0; p < n; ++p) {
        const float* k = kv_dense + (size_t)p * D_QK;
        float acc[HEAD_GROUP];
        for (int g = 0; g < HEAD_GROUP; ++g) acc[g] = 0.0f;
        for (int d = 0; d < D_QK; ++d) {
            const float kd = k[d];
            const float* qd = qT + (size_t)d * HEAD_GROUP;
            for (int g = 0; g < HEAD_GROUP; ++g) acc[g] += qd[g] * kd;
        }
        for (int g = 0; g < HEAD_GROUP; ++g) scores[(size_t)g * n + p] = acc[g] * scale;
    }
}

/* acc[d] = sum_p prob[p] * kv[p][d], p ascending for every d */
__attribute__((target_clones("avx2", "default"))) static void
pv_row(const float* prob, const float* kv_dense, int n, float* acc /* [D_V] */) {
    for (int d = 0; d < D_V; ++d) acc[d] = 0.0f;
    for (int p = 0; p < n; ++p) {
        const float w = prob[p];
        const float* v = kv_dense + (size_t)p * D_QK;
        for (int d = 0; d < D_V; ++d) acc[d] += w * v[d];
    }
}

static int run_query(job_t* J, int qi, float* kv_dense, float* qT, float* scores) {
    const int H = J->H, topk = J->topk;
    const int b = qi / J->s_q;
    const int32_t* idx = J->indices + (size_t)qi * topk;
    int n = 0;
    for (int j = 0; j < topk; ++j) {
        const int32_t i = idx[j];
        int64_t row = -1;
        if (i != -1 && J->kv2 && J->pool_split && j >= J->pool_split[qi]) {
            /* "extend" rows: physical rows of the second pool (mla_v4_host.cc:524-526) */
            if (i < -1) return 1;
            row = i;
            if (row >= J->num_kv2_rows) return 3;
            const uint16_t* s16 = (const uint16_t*)(J->kv2 + (size_t)row * D_QK * 2);
            float* dst = kv_dense + (size_t)n * D_QK;
            for (int d = 0; d < D_QK; ++d) dst[d] = bf16_to_f32(s16[d]);
            ++n;
        } else if (i != -1) {
            if (i < -1) return 1; /* only -1 is padding; anything else negative is a caller error */
            if (J->block_table) {
                const int blk = i / J->page_block_size;
                if (blk >= J->block_table_stride) return 2;
                row = (int64_t)J->block_table[(size_t)b * J->block_table_stride + blk] * J->page_block_size +
                      i % J->page_block_size;
            } else {
                row = (int64_t)b * J->kv_batch_stride_rows + i;
            }
            if (row < 0 || row >= J->num_kv_rows) return 3;
            const uint8_t* src = J->kv + (size_t)row * J->kv_row_bytes;
            float* dst = kv_dense + (size_t)n * D_QK;
            if (J->kv_is_fp8) {
                dequant_row_fp8(src, dst);
            } else {
                const uint16_t* s16 = (const uint16_t*)src;
                for (int d = 0; d < D_QK; ++d) dst[d] = bf16_to_f32(s16[d]);
            }
            ++n;
        }
        if (J->rows_dbg) J->rows_dbg[(size_t)qi * topk + j] = (int32_t)row;
    }

    for (int h0 = 0; h0 < H; h0 += HEAD_GROUP) {
        const int hg = (H - h0 < HEAD_GROUP) ? H - h0 : HEAD_GROUP;
        uint16_t* o_base = J->out + ((size_t)qi * H + h0) * D_V;
        float* lse_base = J->lse + (size_t)qi * H + h0;
        if (n == 0) { /* host.cc:486-490; with a sink the denominator is exp(sink): out 0 (mla_v4_host.cc:507-510), lse = sink */
            for (int g = 0; g < hg; ++g) {
                memset(o_base + (size_t)g * D_V, 0, D_V * 2);
                lse_base[g] = J->attn_sink ? J->attn_sink[h0 + g] : INFINITY;
            }
            continue;
        }
        for (int d = 0; d < D_QK; ++d)
            for (int g = 0; g < HEAD_GROUP; ++g)
                qT[(size_t)d * HEAD_GROUP + g] =
                    (g < hg) ? bf16_to_f32(J->q[(size_t)qi * J->q_stride_q + (size_t)(h0 + g) * J->q_stride_h + d])
                             : 0.0f;
        dots_group(qT, kv_dense, n, J->sm_scale, scores);
        for (int g = 0; g < hg; ++g) {
            float* s = scores + (size_t)g * n;
            float m = s[0];
            for (int p = 1; p < n; ++p)
                if (s[p] > m) m = s[p];
            if (J->attn_sink && J->attn_sink[h0 + g] > m) m = J->attn_sink[h0 + g]; /* mla_v4_host.cc:469 */
            float sum = 0.0f;
            for (int p = 0; p < n; ++p) {
                s[p] = expf(s[p] - m);
                sum += s[p];
            }
            if (J->attn_sink) sum += expf(J->attn_sink[h0 + g] - m); /* mla_v4_host.cc:472 */
            lse_base[g] = logf(sum) + m;
            for (int p = 0; p < n; ++p) s[p] = bf16_to_f32(f32_to_bf16(s[p] / sum));
            float acc[D_V];
            pv_row(s, kv_dense, n, acc);
            uint16_t* o = o_base + (size_t)g * D_V;
            for (int d = 0; d < D_V; ++d) o[d] = f32_to_bf16(acc[d]);
        }
    }
    return 0;
}

static void* worker(void* arg) {
    job_t* J = (job_t*)arg;
    const int topk = J->topk > 0 ? J->topk : 1;
    float* kv_dense = (float*)malloc((size_t)topk * D_QK * sizeof(float));
    float* qT = (float*)malloc((size_t)D_QK * HEAD_GROUP * sizeof(float));
    float* scores = (float*)malloc((size_t)HEAD_GROUP * topk * sizeof(float));
    if (!kv_dense || !qT || !scores) {
        J->error = 100;
    } else {
        for (;;) {
            const int item = __sync_fetch_and_add(&J->next, 1);
            if (item >= J->n_items || J->error) break;
            const int qi = J->subset ? J->subset[item] : item;
            if (qi < 0 || qi >= J->total_q) { J->error = 4; break; }
            const int rc = run_query(J, qi, kv_dense, qT, scores);
            if (rc) { J->error = rc; break; }
        }
    }
    free(kv_dense);
    free(qT);
    free(scores);
    return NULL;
}

/*
 * Sparse MLA attention for every query (or for the listed subset of queries).
 *   q            bf16 [total_q, H, 576] with element strides q_stride_q / q_stride_h
 *   kv           bf16 rows (576 values) or packed fp8 rows (656 bytes), kv_row_bytes apart
 *   indices      int32 [total_q, topk]; token position inside the query's sequence, -1 = padding
 *   block_table  NULL: physical row = (query / s_q) * kv_batch_stride_rows + position
 *                else: physical row = block_table[query / s_q][position / page_block_size]
 *                                     * page_block_size + position % page_block_size
 *   out          bf16 [total_q, H, 512];  lse fp32 [total_q, H]  (only subset rows are written)
 *   rows_dbg     optional int32 [total_q, topk]: the physical row each slot resolved to
 * Returns 0, or a positive code: 1 negative index other than -1, 2 position beyond the block
 * table, 3 physical row out of range, 4 bad subset entry, 100 out of memory.
 */
static int run_job(job_t* J, int num_threads) {
    if (num_threads < 1) num_threads = 1;
    if (num_threads > 256) num_threads = 256;
    if (num_threads > J->n_items) num_threads = J->n_items > 0 ? J->n_items : 1;
    pthread_t tids[256];
    int started = 0;
    for (int t = 1; t < num_threads; ++t)
        if (pthread_create(&tids[started], NULL, worker, J) == 0) ++started;
    worker(J);
    for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
    return J->error;
}

/*
 * The same with the two v4 features (opus_attn/dsa_v4/common/mla_v4_host.cc:455-532, README "Attention
 * Model"): attn_sink [H] joins every row's maximum and denominator; slots >= pool_split[q] of query q index
 * the second pool kv2 (bf16 rows) by physical row, the slots before it the first pool as usual.
 */
int dsa_oracle_sparse_mla_v4(const uint16_t* q, int64_t q_stride_q, int64_t q_stride_h, const void* kv, int kv_is_fp8,
                             int64_t kv_row_bytes, int64_t num_kv_rows, int64_t kv_batch_stride_rows,
                             const int32_t* indices, int topk, const int32_t* block_table, int block_table_stride,
                             int page_block_size, int s_q, float sm_scale, uint16_t* out, float* lse, int total_q, int H,
                             const float* attn_sink, const void* kv2, int64_t num_kv2_rows, const int32_t* pool_split,
                             int num_threads) {
    job_t J;
    memset(&J, 0, sizeof(J));
    J.q = q; J.q_stride_q = q_stride_q; J.q_stride_h = q_stride_h;
    J.kv = (const uint8_t*)kv; J.kv_is_fp8 = kv_is_fp8; J.kv_row_bytes = kv_row_bytes;
    J.num_kv_rows = num_kv_rows; J.kv_batch_stride_rows = kv_batch_stride_rows;
    J.indices = indices; J.topk = topk;
    J.block_table = block_table; J.block_table_stride = block_table_stride;
    J.page_block_size = page_block_size > 0 ? page_block_size : 1;
    J.s_q = s_q > 0 ? s_q : 1;
    J.sm_scale = sm_scale; J.out = out; J.lse = lse;
    J.total_q = total_q; J.H = H; J.n_items = total_q;
    J.attn_sink = attn_sink; J.kv2 = (const uint8_t*)kv2; J.num_kv2_rows = num_kv2_rows; J.pool_split = pool_split;
    return run_job(&J, num_threads);
}

int dsa_oracle_sparse_mla(const uint16_t* q, int64_t q_stride_q, int64_t q_stride_h, const void* kv, int kv_is_fp8,
                          int64_t kv_row_bytes, int64_t num_kv_rows, int64_t kv_batch_stride_rows,
                          const int32_t* indices, int topk, const int32_t* block_table, int block_table_stride,
                          int page_block_size, int s_q, float sm_scale, uint16_t* out, float* lse,
                          int32_t* rows_dbg, int total_q, int H, const int32_t* subset, int n_subset,
                          int num_threads) {
    job_t J;
    memset(&J, 0, sizeof(J));
    J.q = q; J.q_stride_q = q_stride_q; J.q_stride_h = q_stride_h;
    J.kv = (const uint8_t*)kv; J.kv_is_fp8 = kv_is_fp8; J.kv_row_bytes = kv_row_bytes;
    J.num_kv_rows = num_kv_rows; J.kv_batch_stride_rows = kv_batch_stride_rows;
    J.indices = indices; J.topk = topk;
    J.block_table = block_table; J.block_table_stride = block_table_stride;
    J.page_block_size = page_block_size > 0 ? page_block_size : 1;
    J.s_q = s_q > 0 ? s_q : 1;
    J.sm_scale = sm_scale; J.out = out; J.lse = lse; J.rows_dbg = rows_dbg;
    J.total_q = total_q; J.H = H;
    J.subset = subset; J.n_items = subset ? n_subset : total_q;
    return run_job(&J, num_threads);
}

/*
 * Split-KV merge, restating common/mla_reduce.hpp:6-21 and :92-156 in fp32 on the host:
 *   m = max_i lse_i ; w_i = exp2((lse_i - m) * log2e) (0 when lse_i is the "empty" marker)
 *   out = (sum_i w_i * O_i) / sum_i w_i ; lse = m + log2(sum_i w_i) * ln2 ; sum == 0 -> out 0, lse +inf
 * o_parts [ns, 512] fp32 (already normalised per split), lse_parts [ns]; empty marker = -FLT_MAX.
 * Used by the CPU tests of the planner (split + merge must reproduce the unsplit result).
 */
void dsa_oracle_merge(const float* o_parts, const float* lse_parts, int ns, float* out_f32, float* lse_out) {
    const float lowest = -3.402823466e+38f;
    float m = lowest;
    for (int i = 0; i < ns; ++i)
        if (lse_parts[i] > m) m = lse_parts[i];
    float denom = 0.0f;
    for (int i = 0; i < ns; ++i)
        denom += (lse_parts[i] > lowest) ? exp2f((lse_parts[i] - m) * 1.4426950408889634f) : 0.0f;
    *lse_out = (denom > 0.0f) ? (m + log2f(denom) * 0.69314718055994531f) : INFINITY;
    const float inv = (denom > 0.0f) ? 1.0f / denom : 0.0f;
    for (int d = 0; d < D_V; ++d) out_f32[d] = 0.0f;
    for (int i = 0; i < ns; ++i) {
        const float w = (lse_parts[i] > lowest) ? exp2f((lse_parts[i] - m) * 1.4426950408889634f) : 0.0f;
        for (int d = 0; d < D_V; ++d) out_f32[d] += w * o_parts[(size_t)i * D_V + d];
    }
    for (int d = 0; d < D_V; ++d) out_f32[d] *= inv;
}
