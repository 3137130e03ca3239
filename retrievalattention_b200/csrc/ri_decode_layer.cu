// The small element-wise kernels of one decode layer around the wave-index attention: RMS norm
// (with the residual add that precedes it), rotary embedding fused with the split of the fused
// QKV projection, and SiLU(gate) * up.  They replace the flashinfer calls of the reference's
// layer loop (model_hub/llama.py:304-309 rmsnorm, :312-320 apply_rope_with_cos_sin_cache_inplace,
// :267-275 silu_and_mul); the projections themselves stay plain library GEMMs.
// All three are launch-bound at decode batch sizes (a few rows of a few thousand elements), so
// each does as much of the neighbouring work as one pass allows and is meant to be replayed from
// a CUDA graph.  16-bit storage, fp32 arithmetic, one rounding per output element.
#include "ri_common.cuh"

namespace {

constexpr int kNormThreads = 256;

template <int DT>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = Elem<DT>::from_bits((uint16_t)(w[i] & 0xffffu));
    f[2 * i + 1] = Elem<DT>::from_bits((uint16_t)(w[i] >> 16));
  }
}

template <int DT>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(Elem<DT>::pack2(f[0], f[1]), Elem<DT>::pack2(f[2], f[3]), Elem<DT>::pack2(f[4], f[5]),
                    Elem<DT>::pack2(f[6], f[7]));
}

// One CTA per row.  residual != null: residual <- round(residual + x) first (the reference's
// `hidden_states = residual + hidden_states` in the 16-bit type), and the norm is taken of that.
// A thread keeps its pieces in registers between the two passes (dim <= 8 * 256 * kMaxPieces).
constexpr int kMaxPieces = 8;   // dim <= 16384

template <int DT>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const uint4* __restrict__ x, uint4* residual,
                                                              const uint4* __restrict__ weight, uint4* out,
                                                              int pieces, float eps, float inv_dim) {
  __shared__ float warp_sum[kNormThreads / 32];
  __shared__ float s_scale;
  ri_pdl_enter();
  const int row = blockIdx.x, tid = threadIdx.x;
  const int64_t base = (int64_t)row * pieces;
  float v[kMaxPieces][8];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int p = tid + u * kNormThreads;
    if (p < pieces) {
      unpack8<DT>(x[base + p], v[u]);
      if (residual != nullptr) {
        float r[8];
        unpack8<DT>(residual[base + p], r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = Elem<DT>::round(v[u][i] + r[i]);
        residual[base + p] = pack8<DT>(v[u]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[u][i] * v[u][i];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) warp_sum[tid >> 5] = ss;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) t += warp_sum[w];
    s_scale = rsqrtf(t * inv_dim + eps);
  }
  __syncthreads();
  const float scale = s_scale;
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int p = tid + u * kNormThreads;
    if (p < pieces) {
      float w[8], o[8];
      unpack8<DT>(weight[p], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[u][i] * scale * w[i];
      out[base + p] = pack8<DT>(o);
    }
  }
}

// grid (rows, q_heads + 2 * kv_heads), 16 threads per head: thread t owns elements [8t, 8t+8) of the
// first half when t < 8, of the second half otherwise, and reads its partner piece from the other
// half (neox pairing: element j with element j + 64).  cos_sin: fp32 [positions, 128], cosines in
// the first 64 columns, sines in the last 64, as the reference builds it (model_hub/llama.py:81-84, :109).
template <int DT>
__global__ void __launch_bounds__(16) rope_split_kernel(const uint4* __restrict__ qkv, const float4* __restrict__ cos_sin,
                                                        const int64_t* __restrict__ positions, uint4* q, uint4* k, uint4* v,
                                                        int q_heads, int kv_heads, int64_t max_positions) {
  ri_pdl_enter();
  const int row = blockIdx.x, head = blockIdx.y, t = threadIdx.x;
  const int heads = q_heads + 2 * kv_heads;
  const uint4* src = qkv + ((int64_t)row * heads + head) * 16;
  const uint4 mine = src[t];
  if (head >= q_heads + kv_heads) {   // values: a copy
    v[((int64_t)row * kv_heads + head - q_heads - kv_heads) * 16 + t] = mine;
    return;
  }
  const uint4 other = src[t ^ 8];
  int64_t pos = positions[row];
  pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
  const int c = (t & 7) * 2;          // float4 index of this piece's cosines; the sines lie 16 float4 further
  const float4 c0 = cos_sin[pos * 32 + c], c1 = cos_sin[pos * 32 + c + 1];
  const float4 s0 = cos_sin[pos * 32 + 16 + c], s1 = cos_sin[pos * 32 + 16 + c + 1];
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float a[8], b[8], o[8];
  unpack8<DT>(mine, a);
  unpack8<DT>(other, b);
  const float sign = t < 8 ? -1.f : 1.f;   // first half: x1*cos - x2*sin; second half: x2*cos + x1*sin
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = a[i] * cs[i] + sign * b[i] * sn[i];
  const uint4 res = pack8<DT>(o);
  if (head < q_heads) q[((int64_t)row * q_heads + head) * 16 + t] = res;
  else k[((int64_t)row * kv_heads + head - q_heads) * 16 + t] = res;
}

// in: [rows, 2 * inter] (gate | up), out: [rows, inter]; one 16-byte piece of the output per thread.
template <int DT>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const uint4* __restrict__ in, uint4* out, int pieces, int rows) {
  ri_pdl_enter();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * pieces) return;
  const int64_t row = i / pieces, p = i - row * pieces;
  float g[8], u[8], o[8];
  unpack8<DT>(in[row * 2 * pieces + p], g);
  unpack8<DT>(in[row * 2 * pieces + pieces + p], u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  out[i] = pack8<DT>(o);
}

}  // namespace

extern "C" int ri_rmsnorm(const void* d_x, void* d_residual, const void* d_weight, void* d_out, int32_t rows, int32_t dim,
                          float eps, int32_t dtype, void* stream) {
  RI_REQUIRE(d_x && d_weight && d_out, "ri_rmsnorm: null pointer");
  RI_REQUIRE(rows >= 1 && dim >= 8 && dim % 8 == 0 && dim <= 8 * kNormThreads * kMaxPieces,
             "ri_rmsnorm: rows=%d dim=%d unsupported (dim a multiple of 8 up to %d)", rows, dim, 8 * kNormThreads * kMaxPieces);
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)d_x | (uintptr_t)d_residual | (uintptr_t)d_weight | (uintptr_t)d_out) % 16 == 0,
             "ri_rmsnorm: pointers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto go = [&](auto kernel) {
    return ri_launch_pdl_id(8, kernel, dim3(rows), dim3(kNormThreads), 0, s, static_cast<const uint4*>(d_x),
                            static_cast<uint4*>(d_residual), static_cast<const uint4*>(d_weight), static_cast<uint4*>(d_out),
                            dim / 8, eps, 1.0f / (float)dim);
  };
  RI_CUDA_OK(dtype == RI_BF16 ? go(rmsnorm_kernel<RI_BF16>) : go(rmsnorm_kernel<RI_F16>));
  return RI_OK;
}

extern "C" int ri_rope_split(const void* d_qkv, const float* d_cos_sin, const int64_t* d_positions, void* d_q, void* d_k,
                             void* d_v, int32_t rows, int32_t q_heads, int32_t kv_heads, int64_t max_positions,
                             int32_t dtype, void* stream) {
  RI_REQUIRE(d_qkv && d_cos_sin && d_positions && d_q && d_k && d_v, "ri_rope_split: null pointer");
  RI_REQUIRE(rows >= 1 && q_heads >= 1 && kv_heads >= 1 && q_heads + 2 * kv_heads <= 65535 && max_positions >= 1,
             "ri_rope_split: bad sizes");
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)d_qkv | (uintptr_t)d_cos_sin | (uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v) % 16 == 0,
             "ri_rope_split: pointers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows, q_heads + 2 * kv_heads);
  auto go = [&](auto kernel) {
    return ri_launch_pdl_id(8, kernel, grid, dim3(16), 0, s, static_cast<const uint4*>(d_qkv),
                            reinterpret_cast<const float4*>(d_cos_sin), d_positions, static_cast<uint4*>(d_q),
                            static_cast<uint4*>(d_k), static_cast<uint4*>(d_v), q_heads, kv_heads, max_positions);
  };
  RI_CUDA_OK(dtype == RI_BF16 ? go(rope_split_kernel<RI_BF16>) : go(rope_split_kernel<RI_F16>));
  return RI_OK;
}

extern "C" int ri_silu_and_mul(const void* d_in, void* d_out, int32_t rows, int32_t inter, int32_t dtype, void* stream) {
  RI_REQUIRE(d_in && d_out, "ri_silu_and_mul: null pointer");
  RI_REQUIRE(rows >= 1 && inter >= 8 && inter % 8 == 0, "ri_silu_and_mul: rows=%d inter=%d unsupported", rows, inter);
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)d_in | (uintptr_t)d_out) % 16 == 0, "ri_silu_and_mul: pointers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int pieces = inter / 8;
  const int64_t n = (int64_t)rows * pieces;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  auto go = [&](auto kernel) {
    return ri_launch_pdl_id(8, kernel, dim3(blocks), dim3(256), 0, s, static_cast<const uint4*>(d_in),
                            static_cast<uint4*>(d_out), pieces, rows);
  };
  RI_CUDA_OK(dtype == RI_BF16 ? go(silu_and_mul_kernel<RI_BF16>) : go(silu_and_mul_kernel<RI_F16>));
  return RI_OK;
}
