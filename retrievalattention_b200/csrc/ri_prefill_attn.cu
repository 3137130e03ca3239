// Dense (causal) prefill attention, head_dim 128, grouped-query heads, 16-bit inputs, fp32 accumulation.
// Replaces the flash-attn call of attn_hub/retroinfer_attn.py:4-13 (`retroinfer_prefill_attn`:
// flash_attn_with_kvcache(q, k_cache, v_cache, causal) over the whole prompt).
//
// One CTA per (128 query rows, query head, request); it walks the key/value tiles of 128 tokens the rows may see.
//   S = Q.K^T      tcgen05.mma, M 128 x N 128 x K 128 (8 x K16), Q and K tiles staged by TMA with the 128-byte
//                  swizzle straight from the token-major tensors, fp32 accumulator in TMEM (two buffers);
//   softmax        128 threads, one per query row (= TMEM lane): a row of S comes down with tcgen05.ld, online
//                  softmax in the log2 domain with a LAZY reference maximum (the running maximum is only adopted
//                  when it has grown by more than 2^8, so the accumulator is rescaled rarely), P is stored as the
//                  16-bit A operand of the second product in shared memory, swizzled by the thread itself;
//   O += P.V       tcgen05.mma again, M 128 x N 128 (channels) x K 128 (keys); its B operand must have the keys
//                  contiguous, so V is transposed once beforehand into [request, kv head, channel, token]
//                  (a pass over V only: S*128*2 bytes per head against S^2*128*2 flops) and its tiles come in by
//                  TMA like everything else; O stays in TMEM for the whole walk and is rescaled in place
//                  (tcgen05.ld / tcgen05.st) in the rare case the reference maximum moves.
// Six warps: TMA producer, MMA issuer, four softmax/epilogue warps.  QK^T of tile j+1 is issued before P.V of tile j,
// so the tensor pipe works on the next scores while the softmax warps are busy with the current ones.
// Every mbarrier wait is bounded; on expiry the kernel records where, releases its TMEM and returns.
#include <cuda.h>

#include "ri_common.cuh"
#include "ri_tc.cuh"

namespace {

using namespace ri_tc;

constexpr int kTile = 128;                 // query rows per CTA, keys per step
constexpr int kHalf = kTile * 128;         // bytes of a 128-row x 64-element operand half-tile
constexpr int kKvStages = 2;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;        // S buffer 0 | S buffer 1 | O | (unused)
constexpr int kSmem = 1024 /*align*/ + 2 * kHalf /*Q*/ + kKvStages * 2 * kHalf /*K*/ + kKvStages * 2 * kHalf /*V^T*/ +
                      2 * kHalf /*P*/ + 256 /*barriers*/;
constexpr float kLazy = 8.0f;              // the reference maximum follows the running one in steps of more than 2^8

struct AttnArgs {
  void* out;             // [B, S, Hq, 128]
  int* error_flag;
  int S, Hq, Hk, causal;
  int s_pad;             // row length of the transposed V
  float scale2;          // log2(e) / sqrt(128)
  uint32_t idesc;
};

// V [B, S, Hk, 128] -> Vt [B, Hk, 128, s_pad], zero beyond S
__global__ void __launch_bounds__(256) transpose_v_kernel(const uint16_t* __restrict__ v, uint16_t* __restrict__ vt, int S,
                                                          int Hk, int s_pad) {
  typedef uint16_t T;
  __shared__ T tile[64][128 + 2];
  const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 64 * 128; i += 256) {
    const int t = i >> 7, c = i & 127;
    tile[t][c] = t0 + t < S ? v[(((int64_t)b * S + t0 + t) * Hk + h) * 128 + c] : T(0);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 128; i += 256) {
    const int c = i >> 6, t = i & 63;
    if (t0 + t < s_pad) vt[(((int64_t)b * Hk + h) * 128 + c) * s_pad + t0 + t] = tile[t][c];
  }
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = sQ + 2 * kHalf, sV = sK + kKvStages * 2 * kHalf, sP = sV + kKvStages * 2 * kHalf;
  const uint32_t bars = sP + 2 * kHalf;
  uint8_t* sP_ptr = smem_raw + (sP - smem_u32(smem_raw));
  const uint32_t bar_q = bars;
  auto bar_k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_k_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto bar_v_full = [&](int s) { return bars + 8u * (5 + s); };
  auto bar_v_empty = [&](int s) { return bars + 8u * (7 + s); };
  auto bar_s_full = [&](int b) { return bars + 8u * (9 + b); };
  auto bar_s_empty = [&](int b) { return bars + 8u * (11 + b); };
  const uint32_t bar_p_full = bars + 8u * 13, bar_pv_done = bars + 8u * 14;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_skip;

  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(a.error_flag);
  __syncthreads();
  if (s_skip) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;      // long walks (late query tiles) are scheduled first
  const int h = blockIdx.y, b = blockIdx.z, hk = h / (a.Hq / a.Hk);
  const int q_row0 = qt * kTile;
  const int n_kv = a.causal ? min(qt + 1, (a.S + kTile - 1) / kTile) : (a.S + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(bar_k_full(s), 1); mbar_init(bar_k_empty(s), 1);
      mbar_init(bar_v_full(s), 1); mbar_init(bar_v_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_s_full(i), 1); mbar_init(bar_s_empty(i), 4); }
    mbar_init(bar_p_full, 4);
    mbar_init(bar_pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tmem_o = tmem + 2 * kTile;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q, 2 * kHalf);
      tma_load_2d(sQ, &map_q, bar_q, h * 128, b * a.S + q_row0);
      tma_load_2d(sQ + kHalf, &map_q, bar_q, h * 128 + 64, b * a.S + q_row0);
      bool ok = true;
      int issued = 0;
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j % kKvStages;
        const uint32_t par = ((j / kKvStages) & 1) ^ 1;
        ok = mbar_wait(bar_k_empty(s), par, abort_flag, 21);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_k_full(s), 2 * kHalf);
        tma_load_2d(sK + s * 2 * kHalf, &map_k, bar_k_full(s), hk * 128, b * a.S + j * kTile);
        tma_load_2d(sK + s * 2 * kHalf + kHalf, &map_k, bar_k_full(s), hk * 128 + 64, b * a.S + j * kTile);
        ok = mbar_wait(bar_v_empty(s), par, abort_flag, 22);
        if (!ok) { issued = j + 1; break; }
        mbar_arrive_expect_tx(bar_v_full(s), 2 * kHalf);
        tma_load_2d(sV + s * 2 * kHalf, &map_vt, bar_v_full(s), j * kTile, (b * a.Hk + hk) * 128);
        tma_load_2d(sV + s * 2 * kHalf + kHalf, &map_vt, bar_v_full(s), j * kTile + 64, (b * a.Hk + hk) * 128);
        issued = j + 1;
      }
      if (*abort_flag) {     // give the copies still in flight a bounded chance to land before the CTA exits
        mbar_wait(bar_q, 0, abort_flag, 26);
        for (int j = max(0, issued - kKvStages); j < issued; ++j) {
          mbar_wait(bar_k_full(j % kKvStages), (j / kKvStages) & 1, abort_flag, 27);
          mbar_wait(bar_v_full(j % kKvStages), (j / kKvStages) & 1, abort_flag, 28);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = mbar_wait(bar_q, 0, abort_flag, 23);
      auto issue_pv = [&](int t) {
        const int s = t % kKvStages;
        if (!mbar_wait(bar_p_full, t & 1, abort_flag, 24)) return false;
        if (!mbar_wait(bar_v_full(s), (t / kKvStages) & 1, abort_flag, 25)) return false;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = umma_desc_sw128(sP + kb * kHalf), db = umma_desc_sw128(sV + s * 2 * kHalf + kb * kHalf);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(tmem_o, da + 2 * k, db + 2 * k, a.idesc, (t | kb | k) != 0);
        }
        tc_commit(bar_v_empty(s));
        tc_commit(bar_pv_done);
        return true;
      };
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j % kKvStages, buf = j & 1;
        ok = mbar_wait(bar_k_full(s), (j / kKvStages) & 1, abort_flag, 29) &&
             mbar_wait(bar_s_empty(buf), ((j >> 1) & 1) ^ 1, abort_flag, 30);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = umma_desc_sw128(sQ + kb * kHalf), db = umma_desc_sw128(sK + s * 2 * kHalf + kb * kHalf);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(tmem + buf * kTile, da + 2 * k, db + 2 * k, a.idesc, (kb | k) != 0);
        }
        tc_commit(bar_k_empty(s));
        tc_commit(bar_s_full(buf));
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) issue_pv(n_kv - 1);
    }
  } else {
    // ---------------- softmax and epilogue: thread = query row = TMEM lane ----------------
    const int lane_group = warp & 3;                       // a warp may touch only its quarter of the TMEM lanes
    const int row = lane_group * 32 + lane;                // row of the tile
    const int q_row = q_row0 + row;                        // position of the query in its request
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < n_kv; ++j) {
      const int buf = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full(buf), (j >> 1) & 1, abort_flag, 31));
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld32(tmem + t_lane + buf * kTile + c * 32, sr[c]);
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld_landed(sr[c]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_s_empty(buf));        // this warp's quarter of the scores is in registers

      // scaled, masked scores and their maximum
      const int col0 = j * kTile;
      const bool edge = col0 + kTile > a.S || (a.causal && col0 + kTile - 1 > q_row);
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(sr[c][i]) * a.scale2;
          if (edge) {
            const int col = col0 + c * 32 + i;
            if (col >= a.S || (a.causal && col > q_row)) x = -INFINITY;
          }
          sr[c][i] = __float_as_uint(x);
          m_tile = fmaxf(m_tile, x);
        }
      // lazy reference maximum: adopt the running maximum only when it has grown by more than kLazy
      const bool move = m_tile > m_ref + kLazy;            // also true for the first tile (m_ref = -inf)
      const float m_new = move ? m_tile : m_ref;
      const float factor = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_new);      // 1 when the maximum stays
      // probabilities, packed as the 16-bit operand of the second product
      uint32_t pk[64];
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2f(__uint_as_float(sr[c][i]) - m_new), p1 = exp2f(__uint_as_float(sr[c][i + 1]) - m_new);
          lsum += p0 + p1;
          pk[c * 16 + i / 2] = Elem<DT>::pack2(p0, p1);
        }
      l_run = l_run * factor + lsum;
      m_ref = m_new;

      // P's buffer and the accumulator are free once the previous tile's second product has completed
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_pv_done, (j - 1) & 1, abort_flag, 32));
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, move)) {               // rare: bring this warp's rows of O to the new reference
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t orow[32];
            tc_ld32(tmem_o + t_lane + c * 32, orow);
            tc_wait_ld();
            tc_ld_landed(orow);
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * factor);
            tc_st32(tmem_o + t_lane + c * 32, orow);
          }
          tc_wait_st();
        }
      }
      // P into shared memory: row `row` of two K-major half-tiles (keys 0..63 | 64..127), 128-byte swizzle
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint32_t off = hf * kHalf + (row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(sP_ptr + off) =
              make_uint4(pk[hf * 32 + ch * 4], pk[hf * 32 + ch * 4 + 1], pk[hf * 32 + ch * 4 + 2], pk[hf * 32 + ch * 4 + 3]);
        }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> the MMA's async reads
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full);
    }
    // ---- epilogue: O / l, one row per thread ----
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_pv_done, (n_kv - 1) & 1, abort_flag, 33));
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + (((int64_t)b * a.S + q_row) * a.Hq + h) * 128);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t orow[32];
        tc_ld32(tmem_o + t_lane + c * 32, orow);
        tc_wait_ld();
        tc_ld_landed(orow);
        if (q_row < a.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = Elem<DT>::pack2(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv);
            w.y = Elem<DT>::pack2(__uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
            w.z = Elem<DT>::pack2(__uint_as_float(orow[i + 4]) * inv, __uint_as_float(orow[i + 5]) * inv);
            w.w = Elem<DT>::pack2(__uint_as_float(orow[i + 6]) * inv, __uint_as_float(orow[i + 7]) * inv);
            dst[c * 4 + i / 8] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) *a.error_flag = s_abort;
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

template <int DT>
int launch(const void* q, const void* k, const void* v, void* out, void* scratch, int32_t* error, int B, int S, int Hq,
           int Hk, int causal, cudaStream_t s) {
  const int s_pad = (S + kTile - 1) / kTile * kTile;
  uint16_t* vt = static_cast<uint16_t*>(scratch);
  transpose_v_kernel<<<dim3((s_pad + 63) / 64, Hk, B), 256, 0, s>>>(static_cast<const uint16_t*>(v), vt, S, Hk, s_pad);
  RI_LAUNCH_OK("transpose_v_kernel");
  CUtensorMap map_q, map_k, map_vt;
  int rc;
  if ((rc = make_map_2d(&map_q, q, (int64_t)Hq * 128, (int64_t)B * S, (int64_t)Hq * 256, DT)) != RI_OK) return rc;
  if ((rc = make_map_2d(&map_k, k, (int64_t)Hk * 128, (int64_t)B * S, (int64_t)Hk * 256, DT)) != RI_OK) return rc;
  if ((rc = make_map_2d(&map_vt, vt, s_pad, (int64_t)B * Hk * 128, (int64_t)s_pad * 2, DT)) != RI_OK) return rc;
  AttnArgs a;
  a.out = out; a.error_flag = error; a.S = S; a.Hq = Hq; a.Hk = Hk; a.causal = causal; a.s_pad = s_pad;
  a.scale2 = RI_LOG2E * 0.08838834764831845f;
  a.idesc = idesc_f16(DT, kTile, kTile);
  RI_CUDA_OK(cudaFuncSetAttribute(prefill_attn_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  prefill_attn_kernel<DT><<<dim3((S + kTile - 1) / kTile, Hq, B), kThreads, kSmem, s>>>(map_q, map_k, map_vt, a);
  RI_LAUNCH_OK("prefill_attn_kernel");
  return RI_OK;
}

}  // namespace

extern "C" int64_t ri_prefill_attn_scratch_bytes(int32_t batch, int32_t seq_len, int32_t kv_heads) {
  if (batch < 1 || seq_len < 1 || kv_heads < 1) return RI_ERR_INVALID;
  const int64_t s_pad = ((int64_t)seq_len + kTile - 1) / kTile * kTile;
  return (int64_t)batch * kv_heads * 128 * s_pad * 2;
}

extern "C" int ri_prefill_attn(const void* d_q, const void* d_k, const void* d_v, void* d_out, void* d_scratch,
                               int32_t* d_error, int32_t batch, int32_t seq_len, int32_t q_heads, int32_t kv_heads,
                               int32_t causal, int32_t dtype, void* stream) {
  RI_REQUIRE(d_q && d_k && d_v && d_out && d_scratch && d_error, "ri_prefill_attn: null pointer");
  RI_REQUIRE(batch >= 1 && seq_len >= 1 && kv_heads >= 1 && q_heads >= kv_heads && q_heads % kv_heads == 0,
             "ri_prefill_attn: bad sizes (batch %d, seq_len %d, %d q heads, %d kv heads)", batch, seq_len, q_heads, kv_heads);
  RI_REQUIRE((int64_t)batch * seq_len < (1ll << 31) && (int64_t)batch * kv_heads * 128 < (1ll << 31), "ri_prefill_attn: too large");
  RI_REQUIRE(dtype == RI_BF16 || dtype == RI_F16, "dtype=%d unsupported", dtype);
  RI_REQUIRE(((uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v | (uintptr_t)d_out | (uintptr_t)d_scratch) % 16 == 0,
             "ri_prefill_attn: tensors must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == RI_BF16 ? launch<RI_BF16>(d_q, d_k, d_v, d_out, d_scratch, d_error, batch, seq_len, q_heads, kv_heads, causal, s)
                          : launch<RI_F16>(d_q, d_k, d_v, d_out, d_scratch, d_error, batch, seq_len, q_heads, kv_heads, causal, s);
}
