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
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ExecBuffer* eb) {
  AttendArgs a;
  fill_attend_args(p, L, eb, a);
  const int clusters = min(p.groups, max(1, attend_ctas() / kAttendCluster));
  const int ctas = clusters * kAttendCluster;
  RI_CUDA_OK(cudaFuncSetAttribute(wave_attend_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
  RI_CUDA_OK(ri_launch_pdl_id(2, wave_attend_kernel<DT>, dim3(ctas), dim3(128), (size_t)kRingBytes, s, a));
  return RI_OK;
}

}  // namespace

int launch_attend(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ExecBuffer* eb) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s, eb) : launch<RI_F16>(p, L, s, eb);
}

}  // namespace ri_wave
