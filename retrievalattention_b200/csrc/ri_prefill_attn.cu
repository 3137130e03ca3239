// Dense (causal) prefill attention, head_dim 128, grouped-query heads, 16-bit inputs, fp32 accumulation.
// Replaces the flash-attn call of attn_hub/retroinfer_attn.py:4-13 (`retroinfer_prefill_attn`:
// flash_attn_with_kvcache(q, k_cache, v_cache, causal) over the whole prompt).
//
// One CTA per (128 query rows, query head, request); it walks the key/value tiles of 128 tokens the rows may see.
//   S = Q.K^T      tcgen05.mma, M 128 x N 128 x K 128 (8 x K16), Q and K tiles staged by TMA with the 128-byte
//                  swizzle straight from the token-major tensors, fp32 accumulator in TMEM (two buffers);
//   softmax        TWO groups of 128 threads, one thread per query row (= TMEM lane); group g takes the tiles
//                  j = g, g + 2, ... and keeps its own running (maximum, sum) and its own accumulator, so the
//                  exponentials of two tiles are computed side by side while the tensor pipe multiplies.  A row of
//                  S comes down with tcgen05.ld; online softmax in the log2 domain with a LAZY reference maximum
//                  (the running maximum is only adopted when it has grown by more than 2^8, so an accumulator is
//                  rescaled rarely); P is stored as the 16-bit A operand of the second product in shared memory,
//                  swizzled by the thread itself;
//   O_g += P.V     tcgen05.mma again, M 128 x N 128 (channels) x K 128 (keys); its B operand must have the keys
//                  contiguous, so V is transposed once beforehand into [request, kv head, channel, token]
//                  (a pass over V only: S*128*2 bytes per head against S^2*128*2 flops) and its tiles come in by
//                  TMA like everything else; O_0 and O_1 stay in TMEM for the whole walk (S_0 | S_1 | O_0 | O_1 =
//                  all 512 columns), are rescaled in place (tcgen05.ld / tcgen05.st) in the rare case a reference
//                  maximum moves, and are merged by log-sum-exp at the end.
// Ten warps: TMA producer, MMA issuer, eight softmax/epilogue warps.  QK^T of tile j+1 is issued before P.V of tile j.
// Every mbarrier wait is bounded; on expiry the kernel records where, releases its TMEM and returns.
#include <cuda.h>

#include "ri_common.cuh"
#include "ri_tc.cuh"

namespace {

using namespace ri_tc;

constexpr int kTile = 128;                 // query rows per CTA, keys per step
constexpr int kHalf = kTile * 128;         // bytes of a 128-row x 64-element operand half-tile
constexpr int kKvStages = 2;
constexpr int kThreads = 320;
constexpr uint32_t kTmemCols = 512;        // S_0 | S_1 | O_0 | O_1, 128 columns each
constexpr int kSmem = 1024 /*align*/ + 2 * kHalf /*Q*/ + kKvStages * 2 * kHalf /*K*/ + kKvStages * 2 * kHalf /*V^T*/ +
                      2 * 2 * kHalf /*P_0, P_1*/ + 256 /*barriers*/;
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
  const uint32_t bars = sP + 2 * 2 * kHalf;
  uint8_t* sP_ptr = smem_raw + (sP - smem_u32(smem_raw));
  const uint32_t bar_q = bars;
  auto bar_k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_k_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto bar_v_full = [&](int s) { return bars + 8u * (5 + s); };
  auto bar_v_empty = [&](int s) { return bars + 8u * (7 + s); };
  auto bar_s_full = [&](int b) { return bars + 8u * (9 + b); };
  auto bar_s_empty = [&](int b) { return bars + 8u * (11 + b); };
  auto bar_p_full = [&](int g) { return bars + 8u * (13 + g); };
  auto bar_pv_done = [&](int g) { return bars + 8u * (15 + g); };
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_skip;
  __shared__ float s_m1[kTile], s_l1[kTile];      // group 1's running (maximum, sum) per row, for the final merge

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
    for (int i = 0; i < 2; ++i) { mbar_init(bar_p_full(i), 4); mbar_init(bar_pv_done(i), 1); }
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
      auto issue_pv = [&](int t) {          // tile t belongs to softmax group t & 1: its P buffer, its accumulator
        const int s = t % kKvStages, g = t & 1;
        if (!mbar_wait(bar_p_full(g), (t >> 1) & 1, abort_flag, 24)) return false;
        if (!mbar_wait(bar_v_full(s), (t / kKvStages) & 1, abort_flag, 25)) return false;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = umma_desc_sw128(sP + (g * 2 + kb) * kHalf), db = umma_desc_sw128(sV + s * 2 * kHalf + kb * kHalf);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(tmem + (2 + g) * kTile, da + 2 * k, db + 2 * k, a.idesc, ((t >> 1) | kb | k) != 0);
        }
        tc_commit(bar_v_empty(s));
        tc_commit(bar_pv_done(g));
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
    // ---------------- softmax and epilogue: thread = query row = TMEM lane; group g owns tiles g, g+2, ... ----------------
    const int grp = (warp - 2) >> 2;                       // 0 or 1
    const int lane_group = warp & 3;                       // a warp may touch only its quarter of the TMEM lanes
    const int row = lane_group * 32 + lane;                // row of the tile
    const int q_row = q_row0 + row;                        // position of the query in its request
    const uint32_t t_lane = (uint32_t)(lane_group * 32) << 16;
    const uint32_t tmem_s = tmem + grp * kTile, tmem_o = tmem + (2 + grp) * kTile;
    uint8_t* my_p = sP_ptr + grp * 2 * kHalf;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    int k = 0;                                             // this group's tiles done
    for (int j = grp; ok && j < n_kv; j += 2, ++k) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full(grp), k & 1, abort_flag, 31));
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld32(tmem_s + t_lane + c * 32, sr[c]);
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld_landed(sr[c]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_s_empty(grp));        // this warp's quarter of the scores is in registers

      // masked scores (edge tiles only) and the row maximum, on the raw products (the scale is positive)
      const int col0 = j * kTile;
      const bool edge = col0 + kTile > a.S || (a.causal && col0 + kTile - 1 > q_row);
      float m_raw = -INFINITY;
      if (edge) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + c * 32 + i;
            if (col >= a.S || (a.causal && col > q_row)) sr[c][i] = 0xff800000u;     // -inf
          }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) m_raw = fmaxf(m_raw, __uint_as_float(sr[c][i]));
      const float m_tile = m_raw * a.scale2;
      // lazy reference maximum: adopt the running maximum only when it has grown by more than kLazy
      const bool move = m_tile > m_ref + kLazy;            // also true for the group's first tile (m_ref = -inf)
      const float m_new = move ? m_tile : m_ref;
      const float factor = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_new);      // 1 when the maximum stays
      // probabilities p = 2^(s * scale - m), packed in place as the 16-bit operand of the second product:
      // word w of the row = columns 2w, 2w+1 (it overwrites the scores already consumed)
      float lsum = 0.f;
      const float neg_m = -m_new;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(sr[c][i]), a.scale2, neg_m));
          const float p1 = exp2f(fmaf(__uint_as_float(sr[c][i + 1]), a.scale2, neg_m));
          lsum += p0 + p1;
          sr[c][i / 2] = Elem<DT>::pack2(p0, p1);
        }
      l_run = l_run * factor + lsum;
      m_ref = m_new;

      // this group's P buffer and accumulator are free once its previous tile's second product has completed
      if (k > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_pv_done(grp), (k - 1) & 1, abort_flag, 32));
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
          const int c = hf * 2 + (ch >> 2), w = (ch & 3) * 4;     // columns hf*64 + ch*8 .. +7 = words w..w+3 of chunk c
          *reinterpret_cast<uint4*>(my_p + off) = make_uint4(sr[c][w], sr[c][w + 1], sr[c][w + 2], sr[c][w + 3]);
        }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> the MMA's async reads
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full(grp));
    }
    // ---- epilogue: wait for the group's last product; group 1 hands its (maximum, sum) over; group 0 merges the two
    //      accumulators by log-sum-exp, divides and stores, one row per thread ----
    if (ok && k > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_pv_done(grp), (k - 1) & 1, abort_flag, 33));
    if (grp == 1) { s_m1[row] = m_ref; s_l1[row] = l_run; }
    tc_fence_before();
    asm volatile("bar.sync 1, 256;" ::: "memory");         // the eight softmax warps, always reached (also after a give-up)
    tc_fence_after();
    if (grp == 0 && ok && !*abort_flag) {
      const float m1 = s_m1[row], l1 = s_l1[row];
      const float M = fmaxf(m_ref, m1);                    // group 0 always has a tile: finite
      const float f0 = exp2f(m_ref - M), f1 = m1 == -INFINITY ? 0.f : exp2f(m1 - M);
      const float l = l_run * f0 + l1 * f1;
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      const float w0 = f0 * inv, w1 = f1 * inv;
      const bool two = n_kv > 1;                           // O_1 holds nothing when group 1 had no tile
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + (((int64_t)b * a.S + q_row) * a.Hq + h) * 128);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o0[32], o1[32];
        tc_ld32(tmem + 2 * kTile + t_lane + c * 32, o0);
        if (two) tc_ld32(tmem + 3 * kTile + t_lane + c * 32, o1);
        tc_wait_ld();
        tc_ld_landed(o0);
        if (two) tc_ld_landed(o1);
        if (q_row < a.S) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o0[i]) * w0 + (two ? __uint_as_float(o1[i]) * w1 : 0.f);
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            dst[c * 4 + i / 8] = make_uint4(Elem<DT>::pack2(v[i], v[i + 1]), Elem<DT>::pack2(v[i + 2], v[i + 3]),
                                            Elem<DT>::pack2(v[i + 4], v[i + 5]), Elem<DT>::pack2(v[i + 6], v[i + 7]));
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
