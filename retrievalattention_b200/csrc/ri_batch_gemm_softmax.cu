// Operator-level batch_gemm_softmax: D = alpha * A.B^T rounded to the 16-bit type, then a softmax over
// every row of D, also rounded (reference: library/retroinfer/retroinfer_kernels/src/
// batch_gemm_softmax.cu:171-198, checked there against bmm -> scale -> softmax,
// library/retroinfer/test/test_batch_gemm_softmax.py:9-18).  The decode path does not go through this
// operator (its kernels fuse the scores with the selection); it exists for callers of the operator.
//
// Two kernels: (1) scores with the fragment scheme of ri_wave_scan.cu (A rows packed into the M of
// m16n8k16 MMAs, 16-byte pieces straight from global memory, one pass over B) plus, per 256-column
// block and row, the maximum and the sum of exponentials of the rounded scores; (2) per row, the
// blocks' pairs are merged and the row of D is turned into probabilities.
#include "ri_common.cuh"

namespace {

constexpr int kBlockCols = 256;   // columns per CTA of kernel 1 = columns per (Norm, Sum) pair
constexpr int kMaxRows = 8;

template <int DT>
__global__ void __launch_bounds__(128) bgs_scores_kernel(const uint4* __restrict__ A, const uint4* __restrict__ B,
                                                         uint16_t* __restrict__ D, float* __restrict__ norm,
                                                         float* __restrict__ sum, int m, int n, int n_blocks, float alpha) {
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, t = lane & 3;
  __shared__ float sm_m[4][kMaxRows], sm_s[4][kMaxRows];

  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < m ? ri_ldg16(A + ((int64_t)b * m + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

  float m_run = -INFINITY, s_run = 0.f;
#pragma unroll 1
  for (int round = 0; round < kBlockCols / 128; ++round) {
    const int base = blockIdx.x * kBlockCols + round * 128 + warp * 32;
    if (base >= n) break;
    uint4 kb[4][4];
    const uint4* brow = B + ((int64_t)b * n + base + r) * 16 + t;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = base + j * 8 < n;   // n % 8 == 0: an 8-row tile is entirely in or out
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) kb[j][kk] = ok ? ri_ldg16(brow + j * 8 * 16 + kk * 4) : make_uint4(0, 0, 0, 0);
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
      const bool ok = r < m && c0 < n;
      const float v0 = Elem<DT>::round(alpha * acc[0]), v1 = Elem<DT>::round(alpha * acc[1]);
      if (ok) *reinterpret_cast<uint32_t*>(D + ((int64_t)b * m + r) * n + c0) = Elem<DT>::pack2(v0, v1);
      rv[j][0] = ok ? v0 : -INFINITY;
      rv[j][1] = ok ? v1 : -INFINITY;
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
      s_run = s_run * exp2f((m_run - m_new) * RI_LOG2E) + add;
      m_run = m_new;
    }
  }
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 1);
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 2);
  if (t == 0) { sm_m[warp][r] = m_run; sm_s[warp][r] = s_run; }
  __syncthreads();
  if (threadIdx.x < m) {
    const int h = threadIdx.x;
    const float M = fmaxf(fmaxf(sm_m[0][h], sm_m[1][h]), fmaxf(sm_m[2][h], sm_m[3][h]));
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (sm_m[w][h] > -INFINITY) S += sm_s[w][h] * exp2f((sm_m[w][h] - M) * RI_LOG2E);
    norm[((int64_t)b * m + h) * n_blocks + blockIdx.x] = M;
    sum[((int64_t)b * m + h) * n_blocks + blockIdx.x] = S;
  }
}

template <int DT>
__global__ void __launch_bounds__(256) bgs_softmax_kernel(const uint16_t* __restrict__ D, const float* __restrict__ norm,
                                                          const float* __restrict__ sum, uint16_t* __restrict__ P, int n,
                                                          int n_blocks) {
  const int64_t row = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ float s_m[8], s_s[8], s_stat[2];
  float M = -INFINITY, S = 0.f;
  for (int i = threadIdx.x; i < n_blocks; i += 256) {
    const float mi = norm[row * n_blocks + i], si = sum[row * n_blocks + i];
    const float Mn = fmaxf(M, mi);
    if (Mn > -INFINITY) S = S * exp2f((M - Mn) * RI_LOG2E) + si * exp2f((mi - Mn) * RI_LOG2E);
    M = Mn;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, M, o), s2 = __shfl_xor_sync(0xffffffffu, S, o);
    const float Mn = fmaxf(M, m2);
    if (Mn > -INFINITY) S = S * exp2f((M - Mn) * RI_LOG2E) + s2 * exp2f((m2 - Mn) * RI_LOG2E);
    M = Mn;
  }
  if (lane == 0) { s_m[warp] = M; s_s[warp] = S; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float Mt = -INFINITY, St = 0.f;
    for (int w = 0; w < 8; ++w) {
      const float Mn = fmaxf(Mt, s_m[w]);
      if (Mn > -INFINITY) St = St * exp2f((Mt - Mn) * RI_LOG2E) + s_s[w] * exp2f((s_m[w] - Mn) * RI_LOG2E);
      Mt = Mn;
    }
    s_stat[0] = Mt;
    s_stat[1] = 1.0f / St;
  }
  __syncthreads();
  const float Mt = s_stat[0], inv = s_stat[1];
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;       // 8 columns per thread, n % 8 == 0
  if (c < n) {
    const uint4 d = *reinterpret_cast<const uint4*>(D + row * n + c);
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a0 = Elem<DT>::from_bits((uint16_t)(w[i] & 0xffffu)), a1 = Elem<DT>::from_bits((uint16_t)(w[i] >> 16));
      o[i] = Elem<DT>::pack2(exp2f((a0 - Mt) * RI_LOG2E) * inv, exp2f((a1 - Mt) * RI_LOG2E) * inv);
    }
    *reinterpret_cast<uint4*>(P + row * n + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int DT>
int run(const void* A, const void* B, void* D, float* norm, float* sum, void* P, int batch, int m, int n, float alpha,
        cudaStream_t s) {
  const int n_blocks = (n + kBlockCols - 1) / kBlockCols;
  bgs_scores_kernel<DT><<<dim3(n_blocks, batch), 128, 0, s>>>(static_cast<const uint4*>(A), static_cast<const uint4*>(B),
                                                             static_cast<uint16_t*>(D), norm, sum, m, n, n_blocks, alpha);
  RI_LAUNCH_OK("bgs_scores_kernel");
  bgs_softmax_kernel<DT><<<dim3((n + 2047) / 2048, batch * m), 256, 0, s>>>(static_cast<const uint16_t*>(D), norm, sum,
                                                                           static_cast<uint16_t*>(P), n, n_blocks);
  RI_LAUNCH_OK("bgs_softmax_kernel");
  return RI_OK;
}

}  // namespace

extern "C" int ri_batch_gemm_softmax(const void* A, const void* B, void* D, float* norm, float* sum, void* softmax,
                                     int32_t batch_count, int32_t m, int32_t n, int32_t k, float alpha, float beta,
                                     int32_t dtype, void* stream) {
  RI_REQUIRE(A && B && D && norm && sum && softmax, "ri_batch_gemm_softmax: null pointer");
  RI_REQUIRE(batch_count >= 1 && batch_count <= 65535, "batch_count=%d out of range", batch_count);
  RI_REQUIRE(m >= 1 && m <= kMaxRows, "m=%d unsupported (1..8 rows of A per batch entry)", m);
  RI_REQUIRE(n >= 8 && n % 8 == 0, "n=%d must be a positive multiple of 8", n);
  RI_REQUIRE(k == RI_HEAD_DIM, "k=%d unsupported (128)", k);
  RI_REQUIRE(beta == 0.f, "beta must be 0 (there is no C operand)");
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)A | (uintptr_t)B | (uintptr_t)D | (uintptr_t)softmax) % 16 == 0, "pointers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == RI_BF16 ? run<RI_BF16>(A, B, D, norm, sum, softmax, batch_count, m, n, alpha, s)
                          : run<RI_F16>(A, B, D, norm, sum, softmax, batch_count, m, n, alpha, s);
}
