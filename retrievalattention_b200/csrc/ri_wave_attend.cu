// Stand-alone attend kernel: a fixed, SM-filling grid of 8-CTA clusters, each working on one group
// at a time through the shared per-group body (ri_wave_attend.cuh).
#include "ri_wave_attend.cuh"

namespace ri_wave {
namespace {

template <int DT>
__global__ void __cluster_dims__(kAttendCluster, 1, 1) __launch_bounds__(128, kCtasPerSm) wave_attend_kernel(AttendArgs a) {
  ri_pdl_enter();
  extern __shared__ __align__(16) uint8_t ring[];
  cg::cluster_group cluster = cg::this_cluster();
  const int groups_per_pass = (int)gridDim.x / kAttendCluster;      // clusters in the grid
  const int cl = (int)cluster.block_rank();
  for (int g = (int)blockIdx.x / kAttendCluster; g < a.G; g += groups_per_pass)   // uniform over the cluster
    attend_group<DT>(a, g, cl, ring);
}

int attend_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kAttendMaxCtas;
  if (cached[dev] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cached[dev] = sms * kCtasPerSm < kAttendMaxCtas ? sms * kCtasPerSm : kAttendMaxCtas;
  }
  return cached[dev];
}

template <int DT>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ExecBuffer* eb, const ri_wave_gather* gather) {
  AttendArgs a;
  fill_attend_args(p, L, eb, a);
  if (gather) {
    a.copies = reinterpret_cast<uint16_t* const*>(gather->d_out_slots);
    a.n_copies = gather->n_ranks;
  }
  const int clusters = min(p.groups, max(1, attend_ctas() / kAttendCluster));
  const int ctas = clusters * kAttendCluster;
  RI_CUDA_OK(cudaFuncSetAttribute(wave_attend_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
  RI_CUDA_OK(ri_launch_pdl_id(2, wave_attend_kernel<DT>, dim3(ctas), dim3(128), (size_t)kRingBytes, s, a));
  return RI_OK;
}

template <int DT>
int launch_operator(const AttendArgs& a, cudaStream_t s) {
  const int clusters = min(a.G, max(1, attend_ctas() / kAttendCluster));
  RI_CUDA_OK(cudaFuncSetAttribute(wave_attend_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
  RI_CUDA_OK(ri_launch_pdl_id(2, wave_attend_kernel<DT>, dim3(clusters * kAttendCluster), dim3(128), (size_t)kRingBytes, s, a));
  return RI_OK;
}

}  // namespace

// weighted_flash_decoding as an operator (call sites: cache_hub/retroinfer_cache.py:611-617, :666-674): dense
// keys/values with a valid length per group, optional weights in the softmax denominator, optional merge with
// a previous partial result, optional log-sum-exp output.  Runs the attend kernel over exact rows only.
int launch_weighted_decoding(const void* q, const void* k, const void* v, const void* weights, const int32_t* seqlens,
                             const void* prev_out, const float* prev_lse, void* out, float* lse_out, int groups,
                             int group_size, int64_t stride, int dtype, cudaStream_t s) {
  AttendArgs a = {};
  a.q = static_cast<const uint4*>(q);
  a.keys = static_cast<const uint4*>(k);
  a.values = static_cast<const uint4*>(v);
  a.n_exact = seqlens;
  a.out = out;
  a.N = stride;
  a.G = groups; a.gs = group_size;
  a.scale2 = RI_LOG2E * 0.08838834764831845f;
  a.cost_est = RI_COST_EST; a.cost_exact = RI_COST_EXACT;
  a.row_w = static_cast<const uint16_t*>(weights);
  a.prev_out = static_cast<const uint16_t*>(prev_out);
  a.prev_lse = prev_lse;
  a.lse_out = lse_out;
  return dtype == RI_BF16 ? launch_operator<RI_BF16>(a, s) : launch_operator<RI_F16>(a, s);
}

int launch_attend(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ExecBuffer* eb,
                  const ri_wave_gather* gather) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s, eb, gather) : launch<RI_F16>(p, L, s, eb, gather);
}

}  // namespace ri_wave
