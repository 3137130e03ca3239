// C entry points of the wave-index decode path for one layer: scan -> select -> attend, either as
// one kernel (ri_wave_fused.cu, the default of ri_wave_decode_layer) or as three stage kernels
// (ri_wave_scan.cu, ri_wave_select.cu, ri_wave_attend.cu), plus the steady-zone append.
#include "ri_wave_internal.cuh"

using namespace ri_wave;

namespace {

int validate_geometry_only(const ri_wave_layer* p) {
  RI_REQUIRE(p != nullptr, "ri_wave_layer is null");
  RI_REQUIRE(p->groups > 0 && p->groups <= 65535, "groups=%d out of range", p->groups);
  RI_REQUIRE(p->group_size >= 1 && p->group_size <= kMaxHeads, "group_size=%d unsupported (1..8)", p->group_size);
  RI_REQUIRE(p->n_centroids > 0 && p->n_centroids % 8 == 0 && p->n_centroids <= 65528,
             "n_centroids=%d must be a positive multiple of 8 below 65536", p->n_centroids);
  RI_REQUIRE(p->nprobe >= 1 && p->nprobe <= 1024, "nprobe=%d unsupported (1..1024)", p->nprobe);
  RI_REQUIRE(p->n_estimate >= 0 && p->nprobe + p->n_estimate <= p->n_centroids,
             "nprobe+n_estimate=%d exceeds n_centroids=%d", p->nprobe + p->n_estimate, p->n_centroids);
  RI_REQUIRE(p->page_size >= 1 && p->buffer_pages >= 1, "page_size/buffer_pages must be positive");
  RI_REQUIRE((int64_t)p->buffer_pages * p->page_size <= p->max_exact_rows,
             "max_exact_rows=%d smaller than buffer_pages*page_size", p->max_exact_rows);
  RI_REQUIRE(p->dtype == RI_BF16 || p->dtype == RI_F16, "dtype=%d unsupported", p->dtype);
  RI_REQUIRE(p->steady_stride >= 1 && p->tokens_per_group >= 0, "bad steady_stride/tokens_per_group");
  return RI_OK;
}

int validate(const ri_wave_layer* p) {
  const int rc = validate_geometry_only(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(p->d_centroids && p->d_value_sum && p->d_cluster_size && p->d_cluster_count && p->d_cluster_offset,
             "meta-index pointer is null");
  RI_REQUIRE(p->d_keys && p->d_values && p->d_steady_keys && p->d_steady_values && p->d_static_len,
             "KV pointer is null");
  RI_REQUIRE(p->d_q && p->d_out && p->d_scratch, "q/out/scratch pointer is null");
  RI_REQUIRE(((uintptr_t)p->d_centroids | (uintptr_t)p->d_value_sum | (uintptr_t)p->d_keys | (uintptr_t)p->d_values |
              (uintptr_t)p->d_steady_keys | (uintptr_t)p->d_steady_values | (uintptr_t)p->d_q) % 16 == 0,
             "tensor pointers must be 16-byte aligned");
  RI_REQUIRE((uintptr_t)p->d_scratch % 128 == 0, "the scratch must be 128-byte aligned");
  RI_REQUIRE((p->d_new_keys == nullptr) == (p->d_new_values == nullptr), "d_new_keys and d_new_values go together");
  RI_REQUIRE(((uintptr_t)p->d_new_keys | (uintptr_t)p->d_new_values) % 16 == 0, "new key/value rows must be 16-byte aligned");
  return RI_OK;
}

__global__ void steady_append_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, uint4* sk, uint4* sv,
                                     const int32_t* __restrict__ pos, int pos_offset, int groups, int stride) {
  ri_pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece each
  if (i >= groups * 16) return;
  const int g = i >> 4, c = i & 15;
  const int p = *pos + pos_offset;
  if (p < 0 || p >= stride) return;
  sk[((int64_t)g * stride + p) * 16 + c] = k[i];
  sv[((int64_t)g * stride + p) * 16 + c] = v[i];
}

// Scores of the estimation entries that are in the scratch, recomputed for ANOTHER query: one warp per entry, fp32 dot
// products of the entry's centroid with the group's query heads, stored in the log2 domain where the attend stage
// expects them.
template <int DT>
__global__ void __launch_bounds__(256) wave_rescore_kernel(const uint2* __restrict__ q, const uint2* __restrict__ cent,
                                                           const int32_t* __restrict__ est_ids, float* __restrict__ est_s2,
                                                           int C, int gs, int E, int e_pad, float scale2) {
  const int g = blockIdx.y, lane = threadIdx.x & 31, i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= E) return;
  const int c = min(max(est_ids[(int64_t)g * e_pad + i], 0), C - 1);
  const uint2 cw = cent[((int64_t)g * C + c) * 32 + lane];         // this lane's four channels
  const float c0 = Elem<DT>::from_bits((uint16_t)(cw.x & 0xffffu)), c1 = Elem<DT>::from_bits((uint16_t)(cw.x >> 16));
  const float c2 = Elem<DT>::from_bits((uint16_t)(cw.y & 0xffffu)), c3 = Elem<DT>::from_bits((uint16_t)(cw.y >> 16));
  for (int h = 0; h < gs; ++h) {
    const uint2 qw = q[((int64_t)g * gs + h) * 32 + lane];
    float s = c0 * Elem<DT>::from_bits((uint16_t)(qw.x & 0xffffu)) + c1 * Elem<DT>::from_bits((uint16_t)(qw.x >> 16)) +
              c2 * Elem<DT>::from_bits((uint16_t)(qw.y & 0xffffu)) + c3 * Elem<DT>::from_bits((uint16_t)(qw.y >> 16));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) est_s2[((int64_t)g * kMaxHeads + h) * e_pad + i] = s * scale2;
  }
}

}  // namespace

extern "C" int ri_wave_rescore(const ri_wave_layer* p, void* stream) {
  const int rc = validate(p);
  if (rc != RI_OK) return rc;
  if (p->n_estimate == 0) return RI_OK;
  const Layout L = make_layout(*p);
  uint8_t* sc = static_cast<uint8_t*>(p->d_scratch);
  const dim3 grid((p->n_estimate + 7) / 8, p->groups);
  const float scale2 = RI_LOG2E * 0.08838834764831845f;
  auto* ids = reinterpret_cast<const int32_t*>(sc + L.est_ids);
  auto* s2 = reinterpret_cast<float*>(sc + L.est_s2);
  if (p->dtype == RI_BF16)
    wave_rescore_kernel<RI_BF16><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint2*>(p->d_q), static_cast<const uint2*>(p->d_centroids), ids, s2, p->n_centroids, p->group_size,
        p->n_estimate, L.e_pad, scale2);
  else
    wave_rescore_kernel<RI_F16><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint2*>(p->d_q), static_cast<const uint2*>(p->d_centroids), ids, s2, p->n_centroids, p->group_size,
        p->n_estimate, L.e_pad, scale2);
  RI_LAUNCH_OK("wave_rescore_kernel");
  return RI_OK;
}

extern "C" int64_t ri_wave_scratch_bytes(const ri_wave_layer* p) {
  if (validate_geometry_only(p) != RI_OK) return RI_ERR_INVALID;
  return make_layout(*p).total;
}

extern "C" int ri_wave_scratch_views(const ri_wave_layer* p, ri_wave_views* out) {
  int rc = validate_geometry_only(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(out != nullptr && p->d_scratch != nullptr, "views or scratch pointer is null");
  const Layout L = make_layout(*p);
  uint8_t* sc = static_cast<uint8_t*>(p->d_scratch);
  out->d_scores = reinterpret_cast<const float*>(sc + L.scores);
  out->d_dist_keys = reinterpret_cast<const uint16_t*>(sc + L.dist_keys);
  out->d_exact_rows = reinterpret_cast<const int32_t*>(sc + L.rows);
  out->d_n_exact = reinterpret_cast<const int32_t*>(sc + L.n_exact);
  return RI_OK;
}

extern "C" int ri_wave_scan(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return launch_scan(*p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_select(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return launch_select(*p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_attend(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return launch_attend(*p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_attend_buffer(const ri_wave_layer* p, const void* d_exec_keys, const void* d_exec_values,
                                     int32_t exec_stride, const int32_t* d_valid_lengths, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(d_exec_keys && d_exec_values && d_valid_lengths && exec_stride > 0, "ri_wave_attend_buffer: bad buffer");
  RI_REQUIRE(((uintptr_t)d_exec_keys | (uintptr_t)d_exec_values) % 16 == 0, "execution buffers must be 16-byte aligned");
  const Layout L = make_layout(*p);
  const ExecBuffer eb = {d_exec_keys, d_exec_values, exec_stride, d_valid_lengths, nullptr};
  return launch_attend(*p, L, static_cast<cudaStream_t>(stream), &eb);
}

extern "C" int ri_wave_attend_buffer_lse(const ri_wave_layer* p, const void* d_exec_keys, const void* d_exec_values,
                                         int32_t exec_stride, const int32_t* d_valid_lengths, float* d_lse_out, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(d_exec_keys && d_exec_values && d_valid_lengths && d_lse_out && exec_stride > 0, "ri_wave_attend_buffer_lse: bad buffer");
  RI_REQUIRE(((uintptr_t)d_exec_keys | (uintptr_t)d_exec_values) % 16 == 0, "execution buffers must be 16-byte aligned");
  const Layout L = make_layout(*p);
  const ExecBuffer eb = {d_exec_keys, d_exec_values, exec_stride, d_valid_lengths, d_lse_out};
  return launch_attend(*p, L, static_cast<cudaStream_t>(stream), &eb);
}

namespace {
// One layer's decode step: the single kernel where it covers the geometry, else the three stage kernels.
int decode_layer(const ri_wave_layer* p, const ri_wave_gather* gather, cudaStream_t s) {
  int rc;
  const Layout L = make_layout(*p);
  // RI_WAVE_STAGED=1 keeps the three-kernel form (profiling one stage at a time, A/B timing)
  static const bool staged = getenv("RI_WAVE_STAGED") && atoi(getenv("RI_WAVE_STAGED")) != 0;
  if (!staged && fused_supported(*p)) return launch_fused(*p, L, s, gather);
  if (p->d_new_keys) {   // the three-kernel form appends with the stand-alone kernel (row *d_static_len - 1)
    const int n = p->groups * 16;
    RI_CUDA_OK(ri_launch_pdl_id(4, steady_append_kernel, dim3((n + 255) / 256), dim3(256), 0, s,
                                static_cast<const uint4*>(p->d_new_keys), static_cast<const uint4*>(p->d_new_values),
                                static_cast<uint4*>(const_cast<void*>(p->d_steady_keys)),
                                static_cast<uint4*>(const_cast<void*>(p->d_steady_values)), p->d_static_len, -1, p->groups,
                                p->steady_stride));
  }
  if ((rc = launch_scan(*p, L, s)) != RI_OK) return rc;
  if ((rc = launch_select(*p, L, s)) != RI_OK) return rc;
  return launch_attend(*p, L, s, nullptr, gather);
}
}  // namespace

extern "C" int ri_wave_decode_layer(const ri_wave_layer* p, void* stream) {
  const int rc = validate(p);
  if (rc != RI_OK) return rc;
  return decode_layer(p, nullptr, static_cast<cudaStream_t>(stream));
}

namespace {
int validate_gather(const ri_wave_gather* g) {
  RI_REQUIRE(g != nullptr, "ri_wave_gather is null");
  RI_REQUIRE(g->n_ranks >= 2 && g->n_ranks <= 64, "n_ranks=%d unsupported (2..64)", g->n_ranks);
  RI_REQUIRE(g->rank >= 0 && g->rank < g->n_ranks, "rank=%d outside the group of %d", g->rank, g->n_ranks);
  RI_REQUIRE(g->d_out_slots && g->d_flag_slots && g->d_flags && g->d_epoch && g->d_error, "ri_wave_gather: null pointer");
  return RI_OK;
}
}  // namespace

extern "C" int ri_wave_decode_layer_gather(const ri_wave_layer* p, const ri_wave_gather* g, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  if ((rc = validate_gather(g)) != RI_OK) return rc;
  return decode_layer(p, g, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_gather_wait(const ri_wave_gather* g, void* stream) {
  const int rc = validate_gather(g);
  if (rc != RI_OK) return rc;
  return launch_gather_wait(*g, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_weighted_flash_decoding(const void* d_q, const void* d_k, const void* d_v, const void* d_weights,
                                          const int32_t* d_seqlens, const void* d_previous_out,
                                          const float* d_previous_lse, void* d_out, float* d_lse_out, int32_t groups,
                                          int32_t group_size, int64_t rows_stride, int32_t dtype, void* stream) {
  RI_REQUIRE(d_q && d_k && d_v && d_seqlens && d_out, "ri_weighted_flash_decoding: null pointer");
  RI_REQUIRE((d_previous_out == nullptr) == (d_previous_lse == nullptr), "previous_out and previous_lse go together");
  RI_REQUIRE(groups >= 1 && groups <= 65535 && group_size >= 1 && group_size <= kMaxHeads && rows_stride >= 1,
             "ri_weighted_flash_decoding: bad sizes");
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v) % 16 == 0, "q, k and v must be 16-byte aligned");
  return launch_weighted_decoding(d_q, d_k, d_v, d_weights, d_seqlens, d_previous_out, d_previous_lse, d_out, d_lse_out,
                                  groups, group_size, rows_stride, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_steady_append(const void* d_k, const void* d_v, void* d_steady_keys, void* d_steady_values,
                                const int32_t* d_position, int32_t groups, int32_t steady_stride, void* stream) {
  RI_REQUIRE(d_k && d_v && d_steady_keys && d_steady_values && d_position, "ri_steady_append: null pointer");
  RI_REQUIRE(groups > 0 && steady_stride > 0, "ri_steady_append: bad sizes");
  const int n = groups * 16;
  RI_CUDA_OK(ri_launch_pdl_id(4, steady_append_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           static_cast<const uint4*>(d_k), static_cast<const uint4*>(d_v),
                           static_cast<uint4*>(d_steady_keys), static_cast<uint4*>(d_steady_values), d_position, 0, groups,
                           steady_stride));
  return RI_OK;
}
