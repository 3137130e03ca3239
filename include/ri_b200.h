/*
 * ri_b200.h — C ABI of libri_b200.so: wave-index decode attention for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every function returns 0 on success or a negative ri_status; ri_last_error() gives the
 *    message of the calling thread's last failure.
 *  - Pointers named d_* are device pointers, h_* host pointers; the caller owns every buffer.
 *  - No function allocates device memory or synchronises the device unless it says so.
 *  - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *  - Element type `dtype`: RI_BF16 or RI_F16 (16-bit storage, fp32 accumulation).
 *  - G = batch * kv_heads "groups"; gs = q_heads / kv_heads (<= 8); head_dim is 128.
 *
 * Each entry cites the reference interface it replaces (paths inside the reference project).
 */
#ifndef RI_B200_H
#define RI_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ri_status {
  RI_OK = 0,
  RI_ERR_INVALID = -1,   /* bad argument (null pointer, unsupported size or dtype) */
  RI_ERR_CUDA = -2,      /* a CUDA runtime call or launch failed */
  RI_ERR_TIMEOUT = -3,   /* a bounded device-side wait ran out */
  RI_ERR_STATE = -4      /* call order violated (e.g. update before access) */
} ri_status;

enum { RI_BF16 = 0, RI_F16 = 1 };
enum { RI_HEAD_DIM = 128 };

const char* ri_last_error(void);
int ri_version(void);

/* ------------------------------------------------------------------------------------------
 * Fused decode path (all clusters resident in HBM in cluster-contiguous order).
 * Replaces, per layer and decode step, the whole body of
 * cache_hub/retroinfer_cache.py:549-697 (`retroinfer_cache.compute`):
 * batch_gemm_softmax + sum/masked_fill/topk (:569-575), gather_copy_vectors (:601-605),
 * weighted_flash_decoding on the estimation zone (:611-617), the page-budget rule of
 * WaveBufferCPU::batch_access (wave_buffer_cpu.cpp:207-216), gather_copy_and_concat
 * (:642-648) and the merging weighted_flash_decoding (:666-674).
 * ------------------------------------------------------------------------------------------ */
typedef struct ri_wave_layer {
  /* geometry */
  int32_t groups;            /* G */
  int32_t group_size;        /* gs, 1..8 */
  int32_t n_centroids;       /* C (multiple of 8, <= 65535) */
  int32_t nprobe;            /* P: clusters attended exactly */
  int32_t n_estimate;        /* E: clusters approximated by their centroid */
  int32_t page_size;         /* tokens per page (reference: cache_unit_size = 8) */
  int32_t buffer_pages;      /* page budget per group for retrieved clusters */
  int32_t dtype;             /* RI_BF16 / RI_F16 */
  int64_t tokens_per_group;  /* N: rows of d_keys/d_values per group */
  int32_t steady_stride;     /* rows allocated per group in the steady zone */
  int32_t max_exact_rows;    /* capacity of d_rows per group (>= buffer_pages*page_size) */
  /* meta index (cache_hub/retroinfer_cache.py:212-227) */
  const void* d_centroids;       /* [G, C, 128] */
  const void* d_value_sum;       /* [G, C, 128] */
  const void* d_cluster_size;    /* [G, C] in `dtype` (the reference stores sizes in the KV dtype, :432) */
  const int32_t* d_cluster_count;  /* [G, C] exact sizes; 0 marks an empty (masked) cluster */
  const int32_t* d_cluster_offset; /* [G, C+1] first row of each cluster in d_keys/d_values */
  /* cluster-contiguous KV (the reference's list_keys/list_values, :264-274, kept in HBM) */
  const void* d_keys;            /* [G, N, 128] */
  const void* d_values;          /* [G, N, 128] */
  /* steady zone (:83-92) and its current length for this layer (:559), read on the device */
  const void* d_steady_keys;     /* [G, steady_stride, 128] */
  const void* d_steady_values;
  const int32_t* d_static_len;   /* [1] */
  /* query and output */
  const void* d_q;               /* [G, gs, 128]  (== [B, 1, Hq, 128]) */
  void* d_out;                   /* [G, gs, 128] */
  /* scratch owned by the caller, sizes from ri_wave_scratch_bytes(); reusable across layers */
  void* d_scratch;
  /* optional outputs (may be NULL) */
  int64_t* d_retrieved_ids;      /* [G, P] ranked cluster ids (reference: cluster_ids, :575) */
  int32_t* d_retrieved_kept;     /* [G] how many of them fit the page budget */
  int64_t* d_estimated_ids;      /* [G, E] */
  /* optional (may be NULL, both or neither): this step's key/value rows [G, 128].  When given, the decode entry
   * points store them into the steady zone at row *d_static_len - 1 before attending, which saves the separate
   * ri_steady_append launch (decode_update_kv_cache + compute of the reference in one launch). */
  const void* d_new_keys;
  const void* d_new_values;
} ri_wave_layer;

/* Bytes of scratch one ri_wave_decode_layer call needs for this geometry (no device work). */
int64_t ri_wave_scratch_bytes(const ri_wave_layer* p);

/* Launch scan + select + attend for one layer on `stream`.  The scratch needs no initialisation:
 * every stage writes what a later stage reads. */
int ri_wave_decode_layer(const ri_wave_layer* p, void* stream);

/* Same work as ri_wave_decode_layer for callers that cannot allocate device memory at all: an
 * inference server that gave all of HBM to its own pool at start-up, or a decode loop that must
 * not call cudaMalloc/cudaFree because those stall the whole device.  `p->d_scratch` is ignored;
 * the scratch is a fixed RI_WAVE_STATIC_SCRATCH_BYTES array inside the library image, set aside
 * on every GPU that loads the library until the process exits.  Geometries that need more are
 * refused with RI_ERR_INVALID (config 1 of the benchmark, 32 groups x 8192 centroids, needs
 * about 8 MB).  The call allocates nothing and finds the previous call's leftovers in the array,
 * which no stage depends on.  All calls share the one
 * array, so calls whose GPU work overlaps (other streams, unordered threads) race: order them.
 * The first call on each device looks up the array's device address; make it at start-up,
 * before any stream capture.  This entry point has no counterpart in the reference. */
#define RI_WAVE_STATIC_SCRATCH_BYTES (16u << 20)
int ri_wave_decode_layer_static(const ri_wave_layer* p, void* stream);

/* The three stages on their own (same parameter block), for tests and profiling. */
int ri_wave_scan(const ri_wave_layer* p, void* stream);    /* q.C^T scores -> scratch */
int ri_wave_select(const ri_wave_layer* p, void* stream);  /* softmax, group sum, top-k split */
int ri_wave_attend(const ri_wave_layer* p, void* stream);  /* weighted split-K flash decoding */

/* Selection made ahead of time with ANOTHER query (the reference's `use_cluster_estimation`, model_hub/LLM.py:102-107 and
 * cache_hub/retroinfer_cache.py:582-595: the next layer's clusters are searched one layer early with an estimate of
 * its query): run ri_wave_scan + ri_wave_select with the estimated query on the layer's own scratch; when the real
 * query arrives, ri_wave_rescore recomputes the estimation entries' scores for it (p->d_q = the real query) and
 * ri_wave_attend attends the pre-selected clusters. */
int ri_wave_rescore(const ri_wave_layer* p, void* stream);

/* Host tier: the attend stage over an execution buffer assembled by ri_gather_copy_and_concat
 * (steady zone ++ missed pages from the host list ++ hit pages from the GPU page cache).  The
 * estimation part is as in ri_wave_attend (it uses what ri_wave_select left in the scratch); the
 * exact rows are the first d_valid_lengths[g] rows of d_exec_keys/values [G, exec_stride, 128].
 * Replaces the merging weighted_flash_decoding call on the reference's execution buffer
 * (cache_hub/retroinfer_cache.py:666-674). */
int ri_wave_attend_buffer(const ri_wave_layer* p, const void* d_exec_keys, const void* d_exec_values,
                          int32_t exec_stride, const int32_t* d_valid_lengths, void* stream);

/* The same, also returning the log-sum-exp (natural log) of every (group, head) in d_lse_out [G, gs], so that the result can
 * be merged with attention over further rows (ri_weighted_flash_decoding with d_previous_out/d_previous_lse): the host tier
 * attends the estimation zone and the steady zone while the missed pages are still on their way from the host. */
int ri_wave_attend_buffer_lse(const ri_wave_layer* p, const void* d_exec_keys, const void* d_exec_values,
                              int32_t exec_stride, const int32_t* d_valid_lengths, float* d_lse_out, void* stream);

/* ---- several GPUs: the output gather done by the decode kernel itself ------------------------------
 * The path shards by (request, KV head) group with no exchange inside the attention; the one
 * exchange is the gather of the ranks' [G, gs, 128] output slices before the model's output
 * projection (the reference has no multi-GPU form of this path).  Instead of a collective after
 * the kernel, ri_wave_decode_layer_gather makes the decode kernel store every output value into the
 * gather buffer of EVERY rank of the group (peer-mapped addresses over NVLink; plain stores, no
 * fence inside the kernel — a system-scope fence in each of its CTAs cost 7 us per layer).
 * ri_wave_gather_wait, enqueued behind it on the same stream, runs one small kernel that (1) writes
 * the step's epoch into this rank's flag word on every rank — the decode kernel has completed by
 * then, so its stores are ordered before the flags, and each flag store follows a system-scope fence
 * — and (2) waits until the flag words of all ranks hold the epoch; whatever is enqueued after it
 * may read the complete gather buffer.  The wait is bounded: after wait_limit_us it sets *d_error
 * and returns, so a missing rank never hangs the GPU.
 * *d_epoch is read on the device: the caller increases it once per step (the same value on every
 * rank) before the step's first launch. */
typedef struct ri_wave_gather {
  int32_t n_ranks;                 /* ranks of the gather group, 2..64 */
  int32_t rank;                    /* this rank's place in it */
  int32_t wait_limit_us;           /* <= 0: one second */
  int32_t reserved;
  void* const* d_out_slots;        /* device array [n_ranks]: where this rank's output slice goes on each rank */
  uint32_t* const* d_flag_slots;   /* device array [n_ranks]: this rank's flag word (this layer) on each rank */
  const uint32_t* d_flags;         /* local: this layer's flag words, one per rank */
  const uint32_t* d_epoch;         /* local: [1] the current step's epoch */
  int32_t* d_error;                /* local: set to 1 when a wait ran out */
  unsigned long long* d_stamps;    /* optional (may be NULL), local [3]: the wait kernel's global-timer readings (ns) at
                                      entry, after this rank's flags are raised, and when the last rank's flag was seen */
} ri_wave_gather;
/* ri_wave_decode_layer plus the stores described above (p->d_out is written too).  Geometries beyond the single
 * decode kernel (more than 8192 centroids, e.g. after a re-index of generated tokens) run the three stage
 * kernels, whose attend stage does the stores. */
int ri_wave_decode_layer_gather(const ri_wave_layer* p, const ri_wave_gather* g, void* stream);
/* Raise this rank's flags, then wait (bounded) for every rank's. */
int ri_wave_gather_wait(const ri_wave_gather* g, void* stream);

/* Views into the scratch (device pointers valid after ri_wave_select), for tests. */
typedef struct ri_wave_views {
  const float* d_scores;        /* [G, gs, C] alpha*q.c in fp32 */
  const uint16_t* d_dist_keys;  /* [G, C] order-preserving 16-bit key of the group distance */
  const int32_t* d_exact_rows;  /* [G, max_exact_rows] */
  const int32_t* d_n_exact;     /* [G] retrieved rows (without the steady zone) */
} ri_wave_views;
int ri_wave_scratch_views(const ri_wave_layer* p, ri_wave_views* out);
/* Test hook: limit the estimation entries a CTA of the single decode kernel keeps in shared memory (0 forces its
 * global lists, a small value the mixed case); negative restores the default.  Process-wide. */
int ri_wave_test_local_cap(int cap);

/* Append this step's key/value to the steady zone at row *d_position.
 * Replaces cache_hub/retroinfer_cache.py:538-540 (`decode_update_kv_cache`).
 * d_k/d_v: [G, 128] (== [B, 1, Hk, 128]); steady tensors [G, steady_stride, 128]. */
int ri_steady_append(const void* d_k, const void* d_v, void* d_steady_keys, void* d_steady_values,
                     const int32_t* d_position, int32_t groups, int32_t steady_stride, void* stream);

/* ------------------------------------------------------------------------------------------
 * Element-wise kernels of the decode layer around the attention (the caller of this path,
 * model_hub/LLM.py:90-126 `layer_decode`).  The projections stay library GEMMs; these three
 * replace the flashinfer calls between them.  Rows = batch (one token per request).
 * ------------------------------------------------------------------------------------------ */

/* out = rmsnorm(h) * weight with h = x, or, when d_residual is given, h = d_residual + x rounded
 * to `dtype` and written back to d_residual first.  Replaces flashinfer.rmsnorm
 * (model_hub/llama.py:304-309) and the residual additions of LLM.py:118-119, :124.
 * d_x, d_residual, d_out: [rows, dim]; d_weight: [dim]; dim a multiple of 8, <= 16384. */
int ri_rmsnorm(const void* d_x, void* d_residual, const void* d_weight, void* d_out, int32_t rows,
               int32_t dim, float eps, int32_t dtype, void* stream);

/* Rotary embedding (first-half/second-half pairing) of the query and key heads of a fused QKV
 * projection, and its split into contiguous tensors.  Replaces the split of model_hub/llama.py:232-235
 * and flashinfer.rope.apply_rope_with_cos_sin_cache_inplace(..., is_neox=True) (:312-320).
 * d_qkv: [rows, (q_heads + 2*kv_heads) * 128]; d_cos_sin: fp32 [max_positions, 128], cosines in
 * columns 0..63, sines in 64..127 (:81-84, :109); d_positions: [rows] int64, read on the device
 * (values outside [0, max_positions) are clamped); d_q: [rows, q_heads, 128]; d_k, d_v: [rows, kv_heads, 128]. */
int ri_rope_split(const void* d_qkv, const float* d_cos_sin, const int64_t* d_positions, void* d_q,
                  void* d_k, void* d_v, int32_t rows, int32_t q_heads, int32_t kv_heads,
                  int64_t max_positions, int32_t dtype, void* stream);

/* out[r, j] = silu(in[r, j]) * in[r, inter + j].  Replaces flashinfer.activation.silu_and_mul
 * (model_hub/llama.py:267-275).  d_in: [rows, 2*inter]; d_out: [rows, inter]; inter a multiple of 8. */
int ri_silu_and_mul(const void* d_in, void* d_out, int32_t rows, int32_t inter, int32_t dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Dense prefill attention over the prompt, head_dim 128.  Replaces attn_hub/retroinfer_attn.py:4-13
 * (`retroinfer_prefill_attn`: flash_attn_with_kvcache(q, k_cache, v_cache, causal)) and attn_hub/flash_attn.py:4-13.
 * d_q, d_out: [batch, seq_len, q_heads, 128]; d_k, d_v: [batch, seq_len, kv_heads, 128] (token-major, contiguous);
 * query head h attends kv head h / (q_heads / kv_heads); causal != 0: token i sees tokens 0..i.
 * d_scratch: ri_prefill_attn_scratch_bytes() bytes (the transposed copy of V), contents irrelevant;
 * d_error: [1], must be zero on entry; set non-zero if a bounded device-side wait ran out.
 * ------------------------------------------------------------------------------------------ */
int64_t ri_prefill_attn_scratch_bytes(int32_t batch, int32_t seq_len, int32_t kv_heads);
int ri_prefill_attn(const void* d_q, const void* d_k, const void* d_v, void* d_out, void* d_scratch, int32_t* d_error,
                    int32_t batch, int32_t seq_len, int32_t q_heads, int32_t kv_heads, int32_t causal, int32_t dtype,
                    void* stream);

/* ------------------------------------------------------------------------------------------
 * Prefill clustering.  Replaces cache_hub/kmeans.py:224-259 (`segment_k_means`: Triton assign,
 * update, index-add and reverse-index kernels) and, with `center` = 1, also its caller's
 * wrapping in cache_hub/retroinfer_cache.py:416-432 (mean-centring, centroid + mean, sizes in
 * the KV dtype) and the CPU re-layout of K/V into cluster-contiguous order
 * (wave_buffer_cpu.cpp:513-567, `parse_clusters` + `organize_kv`).
 *
 * Schedule: iterations 1..n_iters-1 run per segment (contiguous ranges of n_tokens/n_segments
 * tokens with n_centroids/n_segments centroids each, tail tokens ignored) with L2-normalised
 * centroids; the last iteration assigns every token against all centroids and takes the plain
 * mean.  Assignment = arg-max inner product (first maximum wins).  Empty clusters keep their
 * previous centroid, get a zero value sum and count 0.
 * ------------------------------------------------------------------------------------------ */
typedef struct ri_kmeans {
  int32_t groups;        /* Z: independent (batch, kv-head) groups in this call */
  int32_t n_tokens;      /* N rows per group */
  int32_t n_centroids;   /* C; C/n_segments must be a multiple of 32 */
  int32_t n_segments;
  int32_t n_iters;       /* reference default 10 */
  int32_t dtype;         /* RI_BF16 / RI_F16 */
  int32_t center;        /* 0: d_keys are already centred (pure segment_k_means);
                            1: subtract the per-group mean key first and add it back to the centroids */
  int32_t reserved;
  const void* d_keys;        /* [Z, N, 128] */
  const void* d_values;      /* [Z, N, 128] */
  void* d_centroids;         /* out [Z, C, 128] */
  void* d_value_sum;         /* out [Z, C, 128] */
  void* d_cluster_size;      /* out [Z, C] in `dtype` */
  int32_t* d_cluster_count;  /* out [Z, C], may be NULL */
  int32_t* d_cluster_offset; /* out [Z, C+1] exclusive prefix sums of the counts, may be NULL */
  int32_t* d_assign;         /* out [Z, N] cluster of every token (reference: max_idx), may be NULL */
  int32_t* d_order;          /* out [Z, N] token ids cluster by cluster, ascending inside a cluster
                                (the reference's inverted lists, flattened), may be NULL */
  void* d_keys_out;          /* out [Z, N, 128] K rows in d_order order, may be NULL (then no layout) */
  void* d_values_out;        /* out [Z, N, 128] */
  void* d_mean_key;          /* out [Z, 128] (only with center = 1), may be NULL */
  void* d_scratch;           /* ri_kmeans_scratch_bytes() bytes, contents irrelevant */
  int32_t* d_error;          /* out [1]: 1 if a device-side bounded wait ran out, may be NULL */
} ri_kmeans;

int64_t ri_kmeans_scratch_bytes(const ri_kmeans* p);
int ri_kmeans_build(const ri_kmeans* p, void* stream);

/* ------------------------------------------------------------------------------------------
 * Gather/copy operators of the host tier (rows of 128 16-bit elements, pages of 8 rows).  Same
 * argument order and meaning as the reference's pybind functions
 * (library/retroinfer/retroinfer_kernels/src/gather_copy.cu:288-305), with tensors replaced by
 * pointers and the stream made explicit.  Index arrays, and key_data2/value_data2 of the concat,
 * may be pinned host memory (read through UVA), as in cache_hub/retroinfer_cache.py:124-173, :264-274.
 * ------------------------------------------------------------------------------------------ */
/* batch_gemm_softmax.cu:171-198 (bound at :201-208) — D[b] = alpha * A[b] . B[b]^T rounded to the 16-bit type,
 * softmax[b] = row-wise softmax of D[b], rounded.  A [batch, m, 128] with m <= 8 (the GQA group), B [batch, n, 128]
 * with n a multiple of 8, D and softmax [batch, m, n]; norm and sum are scratch of batch * m * ceil(n / 256) floats
 * each (per-block maxima and sums, as in the reference, where callers never read them); k must be 128, beta 0.
 * The decode path itself does not use this operator: its kernel fuses the scores with the selection. */
int ri_batch_gemm_softmax(const void* A, const void* B, void* D, float* norm, float* sum, void* softmax,
                          int32_t batch_count, int32_t m, int32_t n, int32_t k, float alpha, float beta,
                          int32_t dtype, void* stream);

/* weighted_flash_decoding as an operator (the reference imports it from an external package; its call sites are
 * cache_hub/retroinfer_cache.py:611-617 and :666-674).  Per group g and query head h, over the first d_seqlens[g]
 * rows j of d_k/d_v [G, rows_stride, 128]:  s_j = q_h.k_j / sqrt(128),  w_j = d_weights[g, j] (1 when NULL),
 *   out = sum_j e^{s_j} v_j / sum_j w_j e^{s_j},   lse = log sum_j w_j e^{s_j};
 * when d_previous_out [G, gs, 128] and d_previous_lse [G, gs] are given, the result is merged with that partial
 * result by log-sum-exp.  d_lse_out [G, gs] (natural log) may be NULL.  The decode path does not use this entry
 * point (its kernel attends clusters in place); it serves callers of the operator. */
int ri_weighted_flash_decoding(const void* d_q, const void* d_k, const void* d_v, const void* d_weights,
                               const int32_t* d_seqlens, const void* d_previous_out, const float* d_previous_lse,
                               void* d_out, float* d_lse_out, int32_t groups, int32_t group_size, int64_t rows_stride,
                               int32_t dtype, void* stream);

/* gather_copy.cu:25-96 — rows data_offsets[g, copy_start : copy_start+copy_num] of keys, values and
 * the per-row 16-bit metadata go to the first copy_num rows of the buffers. */
int ri_gather_copy_vectors(const void* key_data, void* key_buffer, const void* value_data, void* value_buffer,
                           const void* src_metadata, void* dst_metadata, const int64_t* data_offsets,
                           int32_t groups, int32_t data_length, int32_t buffer_length, int32_t index_size,
                           int32_t copy_start, int32_t copy_num, void* stream);
/* gather_copy.cu:100-212 — buffer rows = data1[:copy_vectors1] ++ listed pages of data2 (row-level
 * start index) ++ listed pages of data3 (page-level index); valid_lengths[g] = rows written.
 * data_length1/2 in rows, data_length3 in pages, buffer_length in rows. */
int ri_gather_copy_and_concat(const void* key_data1, const void* key_data2, const void* key_data3,
                              void* key_buffer, const void* value_data1, const void* value_data2,
                              const void* value_data3, void* value_buffer, const int32_t* data_offsets2,
                              const int32_t* data_copy_sizes2, const int32_t* buffer_offsets2,
                              const int32_t* copy_chunks2, const int32_t* data_offsets3,
                              const int32_t* data_copy_sizes3, const int32_t* buffer_offsets3,
                              const int32_t* copy_chunks3, int32_t* valid_lengths, int32_t groups,
                              int32_t data_length1, int64_t data_length2, int32_t data_length3,
                              int32_t buffer_length, int32_t offset_length, int32_t copy_vectors1, void* stream);
/* gather_copy.cu:216-283 — for each listed page: copy_sizes rows starting at s_copy_start + s_offsets of
 * the source rows go to the first rows of destination page d_offsets. */
int ri_gather_copy_and_scatter(const void* key_data, void* key_buffer, const void* value_data,
                               void* value_buffer, const int32_t* s_offsets, const int32_t* copy_sizes,
                               const int32_t* d_offsets, const int32_t* copy_chunks, int32_t groups,
                               int32_t data_length, int32_t buffer_length, int32_t offset_length,
                               int32_t s_copy_start, void* stream);

/* ------------------------------------------------------------------------------------------
 * Host-side wave buffer for the host tier (clusters whose KV stays in pinned host memory and is
 * cached page-wise on the GPU).  Replaces the descriptor/LRU part of `WaveBufferCPU`
 * (library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp:261-816 and its pybind
 * interface :822-849): `set_indices` :442-486, the `parse_clusters` step of
 * `async_construction` :513-542/:592-616, the descriptor step of `update_kv` :646-684,
 * `batch_access` (`para_batch_access`) :789-809 and `sync` :811-814.  The KV re-layout
 * (`organize_kv` :545-567) is not here: ri_kmeans_build writes it on the GPU.
 *
 * All index arrays are host memory owned by the caller (the reference pins them so that kernels
 * read them through UVA), laid out [groups, buffer_size] / [groups] exactly as in
 * cache_hub/retroinfer_cache.py:124-185.  Page ids are handed out lowest-free-first.
 * ------------------------------------------------------------------------------------------ */
typedef struct ri_wave_buffer ri_wave_buffer;

ri_wave_buffer* ri_wb_create(int32_t batch_size, int32_t group_num, int32_t nprobe, int32_t block_size,
                             int32_t n_centroids, int32_t final_n_centroids, int32_t buffer_size,
                             int32_t capacity, int32_t threads);   /* NULL on bad arguments */
void ri_wb_destroy(ri_wave_buffer* wb);
int ri_wb_set_indices(ri_wave_buffer* wb, int32_t* hit_ids, int32_t* hit_sizes, int32_t* hit_cumsum,
                      int32_t* hit_nums, int32_t* miss_ids, int32_t* miss_sizes, int32_t* miss_cumsum,
                      int32_t* miss_nums, int32_t* update_buffer_indices, int32_t* update_sizes,
                      int32_t* update_cache_indices, int32_t* update_nums, const int64_t* searched_clusters);
/* cluster sizes of one request: [group_num, n_centroids]; resets that request's page cache */
int ri_wb_set_clusters(ri_wave_buffer* wb, int32_t batch_idx, const int32_t* cluster_sizes);
/* clusters added by a re-index during decoding: [batch*group_num, n_new] */
int ri_wb_append_clusters(ri_wave_buffer* wb, const int32_t* cluster_sizes, int32_t n_new);
/* Blocks until the hit/miss lists are written, then starts the LRU update in the background.
 * Returns the number of groups whose retrieval was cut by the page budget (>= 0) or an error. */
int ri_wb_batch_access(ri_wave_buffer* wb);
int ri_wb_sync(ri_wave_buffer* wb);          /* waits for the background update (update lists valid) */
/* Between ri_wb_batch_access and the execution-buffer assembly: the worker threads copy every missed page from the cluster
 * store in host memory (h_src_*: [groups, src_rows_per_group] rows of row_bytes) into a pinned staging area
 * (h_stage_*: [groups, stage_rows_per_group] rows), page j of group g at row miss_cumsum[g][j]; blocks until done and
 * returns the largest number of staged rows of any group in *max_rows_out.  ri_stage_upload then sends the first `rows` rows
 * of every group's slot to the device-side staging buffers with ONE strided copy per tensor on `stream`, and
 * ri_gather_copy_and_concat reads the pages from there (data_offsets2 = miss_cumsum).  The reference's kernel reads the
 * missed pages from pinned memory through UVA instead (library/.../gather_copy.cu:100-212, cache_hub/retroinfer_cache.py:642-648). */
int ri_wb_stage_misses(ri_wave_buffer* wb, const void* h_src_keys, const void* h_src_values, int64_t src_rows_per_group,
                       void* h_stage_keys, void* h_stage_values, int64_t stage_rows_per_group, int32_t row_bytes,
                       int32_t* max_rows_out);
int ri_stage_upload(void* d_stage_keys, void* d_stage_values, const void* h_stage_keys, const void* h_stage_values,
                    int32_t groups, int64_t stage_rows_per_group, int32_t rows, int32_t row_bytes, void* stream);
int64_t ri_wb_rows_used(const ri_wave_buffer* wb, int32_t group);

#ifdef __cplusplus
}
#endif
#endif /* RI_B200_H */
