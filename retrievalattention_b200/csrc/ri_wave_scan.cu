// scan: s = alpha * q.C^T over every centroid of every group — the only pass over the 2*C*d-byte
// centroid table — plus, per 256-centroid tile and head, the maximum and the sum of exponentials
// of the 16-bit-rounded scores, so that the selection stage gets the softmax statistics for free.
//
// Tensor-core use: warp-level m16n8k16 MMA with the GQA group packed into M.  Lane (r = lane/4,
// t = lane%4) loads, from row r of an 8-row tile, the four 16-byte pieces at byte offsets
// 16*t + 64*kk (kk = 0..3).  Piece kk feeds MMA k-steps 2kk and 2kk+1: its four 32-bit words are
// (b0, b1) of step 2kk and (b0, b1) of step 2kk+1.  The query row of head r is loaded with the
// very same pattern and used as (a0, a2), so both operands see the same permutation of the 128
// channels and the dot product is unchanged; no shared-memory transpose is needed.
#include "ri_wave_internal.cuh"

namespace ri_wave {
namespace {

template <int DT>
__global__ void __launch_bounds__(128) wave_scan_kernel(const uint4* __restrict__ q, const uint4* __restrict__ cent,
                                                        float* __restrict__ scores, float* __restrict__ tile_max,
                                                        float* __restrict__ tile_sum, int C, int gs, int n_tiles,
                                                        float alpha) {
  ri_pdl_enter();
  const int g = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, t = lane & 3;
  __shared__ float sm_m[4][kMaxHeads], sm_s[4][kMaxHeads];

  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < gs ? ri_ldg16(q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

  float m_run = -INFINITY, s_run = 0.f;   // softmax statistics of head r over this warp's centroids
#pragma unroll 1
  for (int round = 0; round < kScanTile / 128; ++round) {
    const int base = blockIdx.x * kScanTile + round * 128 + warp * 32;
    if (base >= C) break;
    uint4 kb[4][4];
    const uint4* crow = cent + ((int64_t)g * C + base + r) * 16 + t;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = base + j * 8 < C;   // C % 8 == 0: an 8-row tile is entirely in or out
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) kb[j][kk] = ok ? ri_ldg16(crow + j * 8 * 16 + kk * 4) : make_uint4(0, 0, 0, 0);
    }
    float rv[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        Elem<DT>::mma16816(acc, qa[kk].x, 0u, qa[kk].y, 0u, kb[j][kk].x, kb[j][kk].y);
        Elem<DT>::mma16816(acc, qa[kk].z, 0u, qa[kk].w, 0u, kb[j][kk].z, kb[j][kk].w);
      }
      const int c0 = base + j * 8 + 2 * t;
      const float v0 = alpha * acc[0], v1 = alpha * acc[1];
      const bool ok = r < gs && c0 < C;
      if (ok) *reinterpret_cast<float2*>(scores + ((int64_t)g * gs + r) * C + c0) = make_float2(v0, v1);
      rv[j][0] = ok ? Elem<DT>::round(v0) : -INFINITY;
      rv[j][1] = ok ? Elem<DT>::round(v1) : -INFINITY;
    }
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) mx = fmaxf(mx, fmaxf(rv[j][0], rv[j][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    if (m_new > -INFINITY) {
      float add = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) add += exp2f((rv[j][0] - m_new) * RI_LOG2E) + exp2f((rv[j][1] - m_new) * RI_LOG2E);
      s_run = s_run * exp2f((m_run - m_new) * RI_LOG2E) + add;   // m_run = -inf: factor 0, s_run was 0
      m_run = m_new;
    }
  }
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 1);
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 2);
  if (t == 0) { sm_m[warp][r] = m_run; sm_s[warp][r] = s_run; }
  __syncthreads();
  if (threadIdx.x < gs) {
    const int h = threadIdx.x;
    float M = fmaxf(fmaxf(sm_m[0][h], sm_m[1][h]), fmaxf(sm_m[2][h], sm_m[3][h]));
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (sm_m[w][h] > -INFINITY) S += sm_s[w][h] * exp2f((sm_m[w][h] - M) * RI_LOG2E);
    tile_max[((int64_t)g * kMaxHeads + h) * n_tiles + blockIdx.x] = M;
    tile_sum[((int64_t)g * kMaxHeads + h) * n_tiles + blockIdx.x] = S;
  }
}

template <int DT>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  dim3 grid(L.n_tiles, p.groups);
  RI_CUDA_OK(ri_launch_pdl_id(0, wave_scan_kernel<DT>, grid, dim3(128), 0, s, static_cast<const uint4*>(p.d_q),
                           static_cast<const uint4*>(p.d_centroids), reinterpret_cast<float*>(sc + L.scores),
                           reinterpret_cast<float*>(sc + L.tile_max), reinterpret_cast<float*>(sc + L.tile_sum),
                           p.n_centroids, p.group_size, L.n_tiles, 0.08838834764831845f));
  return RI_OK;
}

}  // namespace

int launch_scan(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s) : launch<RI_F16>(p, L, s);
}

}  // namespace ri_wave
