// Stand-alone selection kernel: softmax statistics from the scan's per-tile partials, then the
// shared selection body (ri_wave_select.cuh).
#include "ri_wave_select.cuh"

namespace ri_wave {
namespace {

template <int DT>
__global__ void __cluster_dims__(kSelectCluster, 1, 1) __launch_bounds__(kSelectThreads)
wave_select_kernel(SelectArgs a) {
  ri_pdl_enter();
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ float s_max[kMaxHeads], s_inv[kMaxHeads];
  const int g = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // ---- 1. softmax statistics (warp h reduces head h) ----
  if (warp < a.gs) {
    const float* tm = a.tile_max + ((int64_t)g * kMaxHeads + warp) * a.n_tiles;
    const float* ts = a.tile_sum + ((int64_t)g * kMaxHeads + warp) * a.n_tiles;
    float M = -INFINITY, S = 0.f;           // running (max, sum) pair, merged pairwise
    for (int i = lane; i < a.n_tiles; i += 32) {
      const float m = tm[i], sv = ts[i];
      const float Mn = fmaxf(M, m);
      if (Mn > -INFINITY) S = S * exp2f((M - Mn) * RI_LOG2E) + sv * exp2f((m - Mn) * RI_LOG2E);
      M = Mn;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, M, o), s2 = __shfl_xor_sync(0xffffffffu, S, o);
      const float Mn = fmaxf(M, m2);
      if (Mn > -INFINITY) S = S * exp2f((M - Mn) * RI_LOG2E) + s2 * exp2f((m2 - Mn) * RI_LOG2E);
      M = Mn;
    }
    if (lane == 0) { s_max[warp] = M; s_inv[warp] = 1.0f / S; }
  }
  select_body<DT, kSelectThreads, false>(a, dyn, g, s_max, s_inv);
}

template <int DT>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  SelectArgs a;
  const int rc = fill_select_args(p, L, a);
  if (rc != RI_OK) return rc;
  const size_t smem = select_dyn_bytes(a);
  if (smem > 48 * 1024)
    RI_CUDA_OK(cudaFuncSetAttribute(wave_select_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RI_CUDA_OK(ri_launch_pdl_id(1, wave_select_kernel<DT>, dim3(kSelectCluster, p.groups), dim3(kSelectThreads), smem, s, a));
  return RI_OK;
}

}  // namespace

int launch_select(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s) : launch<RI_F16>(p, L, s);
}

}  // namespace ri_wave
