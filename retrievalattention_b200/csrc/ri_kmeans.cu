// Prefill clustering: segmented inner-product Lloyd k-means, per-cluster value sums and the
// cluster-contiguous KV layout.
//
//   centre   mean key per group (fp32 sums in a fixed order), centred = round(key - mean)
//   assign   argmax_c <x, c> for every token of every problem: tcgen05 MMA (M = 128 tokens,
//            N = 128 centroids, K = 128 channels as 8 x K16) with operands staged by TMA
//            (128-byte swizzle) and fp32 accumulators in TMEM; a warp-specialised CTA
//            (TMA producer / MMA issuer / epilogue warps) overlaps the running arg-max of one
//            accumulator buffer with the MMAs into the other: 256 tokens per block, persistent
//            over blocks, eight epilogue warps.
//   bucket   stable counting sort of the tokens of a problem by cluster: counts, offsets and
//            the member list in ascending token order (deterministic, no global atomics).
//   update   one warp per cluster sums its member rows in list order (fp32), forms the mean,
//            optionally L2-normalises, and stores the centroid in the key dtype if the cluster
//            is non-empty.  On the last iteration the same pass also produces the value sums
//            and writes the cluster-contiguous copy of K and V.
//
// A "problem" is one (group, segment) pair during the segmented iterations and one group
// during the last, global iteration (reference: cache_hub/kmeans.py:240-250).
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "ri_common.cuh"
#include "ri_tc.cuh"

namespace {

using namespace ri_tc;

constexpr int kTileM = 128;       // tokens per CTA tile
constexpr int kTileN = 128;       // centroids per MMA tile
constexpr int kHalfBytes = kTileM * 128;   // one K-block (64 channels) of a 128-row tile: 16 KB

// ---- assign ---------------------------------------------------------------------------------
struct AssignArgs {
  int32_t* assign;       // [total tokens] local centroid index of each token within its problem
  int* error_flag;       // set to 1 if a bounded wait ran out
  int n_tok;             // tokens per problem
  int n_cen;             // centroids per problem
  int seg_per_group;     // problems per group
  int64_t group_stride;  // token rows per group (N)
  uint32_t idesc;
};

// ---- assign kernel --------------------------------------------------------------------------------
// A CTA works through consecutive 256-token blocks of one problem.  Per block
// two 128-row token tiles (A, double-buffered per block) meet every centroid tile (B, streamed
// through three stages) in two MMAs, so a centroid tile fetched into shared memory serves 256 tokens
// and the CTA's set-up is paid once for many blocks; the accumulators fill all 512 TMEM columns
// (2 buffers x 2 token tiles x 128 centroids).  Ten warps: TMA producer, MMA issuer, and eight
// epilogue warps (four per token tile, one per TMEM lane quarter) that keep the running arg-max
// of their 32 tokens: per 32 columns a max tree, then the first column equal to the max (ties ->
// lowest index, the rule of torch.argmax), so nothing in the epilogue is a serial chain.
// Every mbarrier wait has a time and an iteration limit; on expiry the CTA records where it gave up, releases its
// TMEM and returns.
constexpr int kWideThreads = 320;
constexpr int kWideBStages = 3;
constexpr uint32_t kWideTmemCols = 512;
constexpr int kWideSmem = 1024 /*align*/ + 2 * 4 * kHalfBytes /*A: 2 blocks x 2 tiles*/ +
                          kWideBStages * 2 * kHalfBytes /*B*/ + 256 /*barriers*/;

struct WideArgs {
  AssignArgs a;
  int blocks_per_cta;    // 256-token blocks a CTA works through
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));   // three-input maximum (sm_100)
  return d;
}

// arg-max of 32 accumulator columns against the running (best, best_idx).  FULL: all 32 columns exist.
template <bool FULL>
__device__ __forceinline__ void argmax32(const uint32_t (&r)[32], int col_base, int valid, float& best, int& best_idx) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = FULL || i < valid ? __uint_as_float(r[i]) : -INFINITY;
  float m11[11];
#pragma unroll
  for (int i = 0; i < 10; ++i) m11[i] = max3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
  m11[10] = fmaxf(v[30], v[31]);
  const float a0 = max3(m11[0], m11[1], m11[2]), a1 = max3(m11[3], m11[4], m11[5]), a2 = max3(m11[6], m11[7], m11[8]);
  const float m = max3(max3(a0, a1, a2), m11[9], m11[10]);
  if (m > best) {          // strict: an equal value in a later column never replaces an earlier one
    // First column equal to the maximum, found on the FMA pipe (the compare-and-mask form of this search kept the
    // ALU pipe, which also does every maximum, busier than the tensor pipe whenever a problem has few centroid
    // tiles): v - m is exactly 0 for the maxima and negative elsewhere, so fma(v - m, 2^120, -i) is -i for them and
    // far below -32 for the others (differences under 2^-115 do not occur between scores of ordinary magnitude);
    // the maximum of those is minus the first index.
    float w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = fmaf(v[i] - m, 0x1p120f, -(float)i);
    float t11[11];
#pragma unroll
    for (int i = 0; i < 10; ++i) t11[i] = max3(w[3 * i], w[3 * i + 1], w[3 * i + 2]);
    t11[10] = fmaxf(w[30], w[31]);
    const float b0 = max3(t11[0], t11[1], t11[2]), b1 = max3(t11[3], t11[4], t11[5]), b2 = max3(t11[6], t11[7], t11[8]);
    const float wm = max3(max3(b0, b1, b2), t11[9], t11[10]);
    best = m;
    best_idx = col_base + (int)(-wm);
  }
}

__global__ void __launch_bounds__(kWideThreads, 1)
kmeans_assign_wide_kernel(const __grid_constant__ CUtensorMap map_keys, const __grid_constant__ CUtensorMap map_cent,
                          WideArgs w) {
  const AssignArgs& a = w.a;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;     // SW128 tiles need 1024-byte alignment
  const uint32_t sA = base;                                         // [block parity][tile][K half]
  const uint32_t sB = base + 2 * 4 * kHalfBytes;                    // [stage][K half]
  const uint32_t bars = sB + kWideBStages * 2 * kHalfBytes;
  auto bar_a_full = [&](int s) { return bars + 8u * s; };
  auto bar_a_empty = [&](int s) { return bars + 8u * (2 + s); };
  auto bar_b_full = [&](int s) { return bars + 8u * (4 + s); };
  auto bar_b_empty = [&](int s) { return bars + 8u * (4 + kWideBStages + s); };
  auto bar_acc_full = [&](int b) { return bars + 8u * (4 + 2 * kWideBStages + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (6 + 2 * kWideBStages + b); };
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_skip;

  // once any CTA of this launch has given up, the rest leave at once (uniformly per CTA)
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(a.error_flag);
  __syncthreads();
  if (s_skip) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int problem = blockIdx.y;
  const int n_blocks_total = (a.n_tok + 2 * kTileM - 1) / (2 * kTileM);
  const int first_block = blockIdx.x * w.blocks_per_cta;
  const int nb = min(w.blocks_per_cta, n_blocks_total - first_block);       // > 0 by the grid's construction
  const int64_t tok_row0 = (int64_t)(problem / a.seg_per_group) * a.group_stride +
                           (int64_t)(problem % a.seg_per_group) * a.n_tok + (int64_t)first_block * 2 * kTileM;
  const int cen_row0 = problem * a.n_cen;
  const int n_tiles = (a.n_cen + kTileN - 1) / kTileN;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < 2; ++s) { mbar_init(bar_a_full(s), 1); mbar_init(bar_a_empty(s), 1); }
    for (int s = 0; s < kWideBStages; ++s) { mbar_init(bar_b_full(s), 1); mbar_init(bar_b_empty(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kWideTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int a_issued = 0, b_issued = 0;
      auto load_a = [&](int blk) {          // both token tiles of a block: 4 boxes of 128 rows x 64 channels
        const int sa = blk & 1;
        if (!mbar_wait(bar_a_empty(sa), ((blk >> 1) & 1) ^ 1, abort_flag, 11)) return false;
        mbar_arrive_expect_tx(bar_a_full(sa), 4 * kHalfBytes);
        const int row = (int)(tok_row0 + (int64_t)blk * 2 * kTileM);
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
          tma_load_2d(sA + (sa * 4 + tile * 2) * kHalfBytes, &map_keys, bar_a_full(sa), 0, row + tile * kTileM);
          tma_load_2d(sA + (sa * 4 + tile * 2 + 1) * kHalfBytes, &map_keys, bar_a_full(sa), 64, row + tile * kTileM);
        }
        a_issued = blk + 1;
        return true;
      };
      bool ok = load_a(0);
      for (int blk = 0; ok && blk < nb; ++blk) {
        for (int t = 0; ok && t < n_tiles; ++t) {
          const int s = b_issued % kWideBStages;
          ok = mbar_wait(bar_b_empty(s), ((b_issued / kWideBStages) & 1) ^ 1, abort_flag, 12);
          if (!ok) break;
          mbar_arrive_expect_tx(bar_b_full(s), 2 * kHalfBytes);
          tma_load_2d(sB + s * 2 * kHalfBytes, &map_cent, bar_b_full(s), 0, cen_row0 + t * kTileN);
          tma_load_2d(sB + s * 2 * kHalfBytes + kHalfBytes, &map_cent, bar_b_full(s), 64, cen_row0 + t * kTileN);
          ++b_issued;
          if (t == 0 && blk + 1 < nb) ok = load_a(blk + 1);   // the next block's tokens, well ahead of their use
        }
      }
      if (*abort_flag) {
        // give our own copies still in flight a bounded chance to land before the CTA exits
        for (int blk = max(0, a_issued - 2); blk < a_issued; ++blk)
          mbar_wait(bar_a_full(blk & 1), (blk >> 1) & 1, abort_flag, 16);
        for (int j = max(0, b_issued - kWideBStages); j < b_issued; ++j)
          mbar_wait(bar_b_full(j % kWideBStages), (j / kWideBStages) & 1, abort_flag, 17);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int j = 0;                       // centroid tiles issued so far (accumulator buffer = j & 1, B stage = j % 3)
      bool ok = true;
      for (int blk = 0; ok && blk < nb; ++blk) {
        const int sa = blk & 1;
        ok = mbar_wait(bar_a_full(sa), (blk >> 1) & 1, abort_flag, 13);
        for (int t = 0; ok && t < n_tiles; ++t, ++j) {
          const int s = j % kWideBStages, buf = j & 1;
          ok = mbar_wait(bar_b_full(s), (j / kWideBStages) & 1, abort_flag, 14) &&
               mbar_wait(bar_acc_empty(buf), ((j >> 1) & 1) ^ 1, abort_flag, 15);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int tile = 0; tile < 2; ++tile) {
            const uint32_t d_tmem = tmem_base + buf * 2 * kTileN + tile * kTileN;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
              const uint64_t da = umma_desc_sw128(sA + (sa * 4 + tile * 2 + kb) * kHalfBytes);
              const uint64_t db = umma_desc_sw128(sB + s * 2 * kHalfBytes + kb * kHalfBytes);
#pragma unroll
              for (int k = 0; k < 4; ++k)   // K16 steps: 32 bytes along the swizzled row = +2 in the address field
                tc_mma_f16(d_tmem, da + 2 * k, db + 2 * k, a.idesc, (kb | k) != 0);
            }
          }
          tc_commit(bar_b_empty(s));     // the stage is free once these MMAs have read it
          tc_commit(bar_acc_full(buf));  // and both accumulators of the buffer are complete
        }
        if (ok) tc_commit(bar_a_empty(sa));   // the block's token tiles are free once all its MMAs have read them
      }
    }
  } else {
    // ---------------- epilogue: running arg-max over the centroid tiles ----------------
    const int tile = (warp - 2) >> 2;                // which token tile of the block
    const int lane_group = warp & 3;                 // TMEM lanes 32*lane_group .. +31 (a warp may touch only its quarter)
    int j = 0;
    bool ok = true;
    for (int blk = 0; ok && blk < nb; ++blk) {
      float best = -INFINITY;
      int best_idx = 0;
      for (int t = 0; ok && t < n_tiles; ++t, ++j) {
        const int buf = j & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full(buf), (j >> 1) & 1, abort_flag, 18));   // warp-uniform
        if (!ok) break;
        tc_fence_after();
        const int col0 = t * kTileN;
        const int valid = min(kTileN, a.n_cen - col0);
        const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * 2 * kTileN + tile * kTileN;
        // the second half of the columns is on its way from TMEM while the first is being reduced
        uint32_t r0[32], r1[32], r2[32], r3[32];
        tc_ld32(taddr, r0);
        tc_ld32(taddr + 32, r1);
        tc_wait_ld();
        tc_ld_landed(r0);
        tc_ld_landed(r1);
        tc_ld32(taddr + 64, r2);
        tc_ld32(taddr + 96, r3);
        if (valid == kTileN) {
          argmax32<true>(r0, col0, 32, best, best_idx);
          argmax32<true>(r1, col0 + 32, 32, best, best_idx);
          tc_wait_ld();
          tc_ld_landed(r2);
          tc_ld_landed(r3);
          argmax32<true>(r2, col0 + 64, 32, best, best_idx);
          argmax32<true>(r3, col0 + 96, 32, best, best_idx);
        } else {
          argmax32<false>(r0, col0, valid, best, best_idx);
          argmax32<false>(r1, col0 + 32, valid - 32, best, best_idx);
          tc_wait_ld();
          tc_ld_landed(r2);
          tc_ld_landed(r3);
          argmax32<false>(r2, col0 + 64, valid - 64, best, best_idx);
          argmax32<false>(r3, col0 + 96, valid - 96, best, best_idx);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty(buf));
      }
      const int local_tok = (first_block + blk) * 2 * kTileM + tile * kTileM + lane_group * 32 + lane;
      if (ok && local_tok < a.n_tok)
        a.assign[tok_row0 + (int64_t)blk * 2 * kTileM + tile * kTileM + lane_group * 32 + lane] = best_idx;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) *a.error_flag = s_abort;   // which wait gave up (see mbar_wait call sites)
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kWideTmemCols));
  }
}

// ---- assign kernel, centroids resident ----------------------------------------------------------------
// Problems of at most 512 centroids (the segmented iterations of the reference's schedule, the re-index build): the
// problem's centroid tiles (up to four, 128 KB) are fetched ONCE per CTA and stay in shared memory, and only the
// tokens stream, as single 128-row tiles through a three-slot ring (the wide kernel above re-fetches the centroid
// tiles for every 256 tokens).  Per token tile two rounds of two centroid tiles each (accumulators: 2 buffers x
// 2 centroid tiles x 128 columns); the eight epilogue warps are four lane quarters x the two centroid tiles of a
// round, so a token's running arg-max lives in two warps, which meet through shared memory once per token tile
// (equal maxima: the lower index wins, as within a warp).  Every warp runs a fixed number of token tiles and rounds
// whatever its waits return, so the named barrier of that merge is always reached.
// Measured on a segmented launch of configuration 2 (ncu): 580 us and the tensor pipe 48 % active, against 610 us /
// 45 % for the wide kernel; with the epilogue's tcgen05.ld removed 388 us / 70 %, with a single 32-column load per
// warp and round left 527 us / 52 % — the loads themselves, not the arithmetic behind them, hold the MMAs up; four
// accumulator buffers of one centroid tile (the issuer three rounds ahead) were slower still (647 us).
constexpr int kResSlots = 3;
constexpr int kResSmem = 1024 /*align*/ + 4 * 2 * kHalfBytes /*B: 4 tiles*/ + kResSlots * 2 * kHalfBytes /*A ring*/ + 256;

__global__ void __launch_bounds__(kWideThreads, 1)
kmeans_assign_resident_kernel(const __grid_constant__ CUtensorMap map_keys, const __grid_constant__ CUtensorMap map_cent,
                              WideArgs w) {
  const AssignArgs& a = w.a;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sB = base;                                         // [centroid tile][K half]
  const uint32_t sA = base + 4 * 2 * kHalfBytes;                    // [slot][K half]
  const uint32_t bars = sA + kResSlots * 2 * kHalfBytes;
  auto bar_a_full = [&](int s) { return bars + 8u * s; };
  auto bar_a_empty = [&](int s) { return bars + 8u * (kResSlots + s); };
  const uint32_t bar_b_full = bars + 8u * (2 * kResSlots);
  auto bar_acc_full = [&](int b) { return bars + 8u * (2 * kResSlots + 1 + b); };
  auto bar_acc_empty = [&](int b) { return bars + 8u * (2 * kResSlots + 3 + b); };
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_skip;
  __shared__ float s_best[2][kTileM];      // the merge of a token's two warps (indices fit 16 bits: <= 512 centroids)
  __shared__ uint16_t s_idx[2][kTileM];

  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(a.error_flag);
  __syncthreads();
  if (s_skip) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int problem = blockIdx.y;
  const int units_total = (a.n_tok + kTileM - 1) / kTileM;
  const int first_unit = blockIdx.x * w.blocks_per_cta * 2;
  const int nu = min(w.blocks_per_cta * 2, units_total - first_unit);       // > 0 by the grid's construction
  const int64_t tok_row0 = (int64_t)(problem / a.seg_per_group) * a.group_stride +
                           (int64_t)(problem % a.seg_per_group) * a.n_tok + (int64_t)first_unit * kTileM;
  const int cen_row0 = problem * a.n_cen;
  const int n_tiles = (a.n_cen + kTileN - 1) / kTileN;              // 1 .. 4
  const int rounds = (n_tiles + 1) / 2;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kResSlots; ++s) { mbar_init(bar_a_full(s), 1); mbar_init(bar_a_empty(s), 1); }
    mbar_init(bar_b_full, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kWideTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_b_full, n_tiles * 2 * kHalfBytes);
      for (int t = 0; t < n_tiles; ++t) {
        tma_load_2d(sB + t * 2 * kHalfBytes, &map_cent, bar_b_full, 0, cen_row0 + t * kTileN);
        tma_load_2d(sB + t * 2 * kHalfBytes + kHalfBytes, &map_cent, bar_b_full, 64, cen_row0 + t * kTileN);
      }
      int issued = 0;
      bool ok = true;
      for (int u = 0; ok && u < nu; ++u) {
        const int s = u % kResSlots;
        ok = mbar_wait(bar_a_empty(s), ((u / kResSlots) & 1) ^ 1, abort_flag, 21);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_a_full(s), 2 * kHalfBytes);
        const int row = (int)(tok_row0 + (int64_t)u * kTileM);
        tma_load_2d(sA + s * 2 * kHalfBytes, &map_keys, bar_a_full(s), 0, row);
        tma_load_2d(sA + s * 2 * kHalfBytes + kHalfBytes, &map_keys, bar_a_full(s), 64, row);
        issued = u + 1;
      }
      if (*abort_flag) {
        // give our own copies still in flight a bounded chance to land before the CTA exits
        mbar_wait(bar_b_full, 0, abort_flag, 26);
        for (int u = max(0, issued - kResSlots); u < issued; ++u)
          mbar_wait(bar_a_full(u % kResSlots), (u / kResSlots) & 1, abort_flag, 27);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = mbar_wait(bar_b_full, 0, abort_flag, 22);
      int j = 0;                       // rounds issued so far (accumulator buffer = j & 1)
      for (int u = 0; ok && u < nu; ++u) {
        const int s = u % kResSlots;
        ok = mbar_wait(bar_a_full(s), (u / kResSlots) & 1, abort_flag, 23);
        for (int r = 0; ok && r < rounds; ++r, ++j) {
          const int buf = j & 1;
          ok = mbar_wait(bar_acc_empty(buf), ((j >> 1) & 1) ^ 1, abort_flag, 24);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int ct = 2 * r + h;
            if (ct < n_tiles) {
              const uint32_t d_tmem = tmem_base + buf * 2 * kTileN + h * kTileN;
#pragma unroll
              for (int kb = 0; kb < 2; ++kb) {
                const uint64_t da = umma_desc_sw128(sA + (s * 2 + kb) * kHalfBytes);
                const uint64_t db = umma_desc_sw128(sB + (ct * 2 + kb) * kHalfBytes);
#pragma unroll
                for (int k = 0; k < 4; ++k) tc_mma_f16(d_tmem, da + 2 * k, db + 2 * k, a.idesc, (kb | k) != 0);
              }
            }
          }
          tc_commit(bar_acc_full(buf));
        }
        if (ok) tc_commit(bar_a_empty(s));   // the token tile is free once all its MMAs have read it
      }
    }
  } else {
    // ---------------- epilogue: running arg-max, two warps per token ----------------
    const int half = (warp - 2) >> 2;                // which centroid tile of a round
    const int lane_group = warp & 3;                 // TMEM lanes 32*lane_group .. +31 (a warp may touch only its quarter)
    const int row = lane_group * 32 + lane;          // this lane's token within the tile
    int j = 0;
    bool ok = true;
    for (int u = 0; u < nu; ++u) {                   // fixed trip counts: the barrier below must be reached by all
      float best = -INFINITY;
      int best_idx = 0;
      for (int r = 0; r < rounds; ++r, ++j) {
        const int buf = j & 1;
        ok = ok && __all_sync(0xffffffffu, mbar_wait(bar_acc_full(buf), (j >> 1) & 1, abort_flag, 25));   // warp-uniform
        const int ct = 2 * r + half;
        if (ok && ct < n_tiles) {
          tc_fence_after();
          const int col0 = ct * kTileN;
          const int valid = min(kTileN, a.n_cen - col0);
          const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * 2 * kTileN + half * kTileN;
          uint32_t r0[32], r1[32], r2[32], r3[32];
          tc_ld32(taddr, r0);
          tc_ld32(taddr + 32, r1);
          tc_wait_ld();
          tc_ld_landed(r0);
          tc_ld_landed(r1);
          tc_ld32(taddr + 64, r2);
          tc_ld32(taddr + 96, r3);
          if (valid == kTileN) {
            argmax32<true>(r0, col0, 32, best, best_idx);
            argmax32<true>(r1, col0 + 32, 32, best, best_idx);
            tc_wait_ld();
            tc_ld_landed(r2);
            tc_ld_landed(r3);
            argmax32<true>(r2, col0 + 64, 32, best, best_idx);
            argmax32<true>(r3, col0 + 96, 32, best, best_idx);
          } else {
            argmax32<false>(r0, col0, valid, best, best_idx);
            argmax32<false>(r1, col0 + 32, valid - 32, best, best_idx);
            tc_wait_ld();
            tc_ld_landed(r2);
            tc_ld_landed(r3);
            argmax32<false>(r2, col0 + 64, valid - 64, best, best_idx);
            argmax32<false>(r3, col0 + 96, valid - 96, best, best_idx);
          }
          tc_fence_before();
        }
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(bar_acc_empty(buf));
      }
      // the two warps of a token meet (buffers alternate per token tile, so one barrier per tile is enough)
      const int par = u & 1;
      if (half == 1) { s_best[par][row] = best; s_idx[par][row] = (uint16_t)best_idx; }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0) {
        const float ob = s_best[par][row];
        const int oi = (int)s_idx[par][row];
        if (ob > best || (ob == best && oi < best_idx)) best_idx = oi;
        const int local_tok = (first_unit + u) * kTileM + row;
        if (ok && local_tok < a.n_tok) a.assign[tok_row0 + (int64_t)u * kTileM + row] = best_idx;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) *a.error_flag = s_abort;   // which wait gave up (see mbar_wait call sites)
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kWideTmemCols));
  }
}

// ---- centre ---------------------------------------------------------------------------------
constexpr int kMeanRows = 2048;   // rows per partial-sum CTA

template <int DT>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const uint4* __restrict__ keys, float* __restrict__ partial,
                                                             int n_tok, int chunks) {
  const int z = blockIdx.y, chunk = blockIdx.x;
  const int piece = threadIdx.x & 15, rl = threadIdx.x >> 4;   // 16 pieces of 8 channels x 16 row lanes
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int r0 = chunk * kMeanRows, r1 = min(n_tok, r0 + kMeanRows);
  for (int r = r0 + rl; r < r1; r += 16) {
    const uint4 v = ri_ldg16(keys + ((int64_t)z * n_tok + r) * 16 + piece);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += Elem<DT>::from_bits((uint16_t)(w[i] & 0xffffu));
      acc[2 * i + 1] += Elem<DT>::from_bits((uint16_t)(w[i] >> 16));
    }
  }
  __shared__ float red[16][128];
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][piece * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 128) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) s += red[k][threadIdx.x];
    partial[((int64_t)z * chunks + chunk) * 128 + threadIdx.x] = s;
  }
}

template <int DT>
__global__ void colmean_final_kernel(const float* __restrict__ partial, uint16_t* __restrict__ mean, int n_tok, int chunks) {
  const int z = blockIdx.x, c = threadIdx.x;
  float s = 0.f;
  for (int k = 0; k < chunks; ++k) s += partial[((int64_t)z * chunks + k) * 128 + c];
  mean[z * 128 + c] = Elem<DT>::bits(s / (float)n_tok);
}

template <int DT>
__global__ void __launch_bounds__(256) centre_apply_kernel(const uint4* __restrict__ keys, const uint16_t* __restrict__ mean,
                                                           uint4* __restrict__ out, int64_t pieces_per_group) {
  const int z = blockIdx.y;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces_per_group) return;
  const int piece = (int)(i & 15);
  const uint4 v = ri_ldg16(keys + (int64_t)z * pieces_per_group + i);
  const uint4 m = *reinterpret_cast<const uint4*>(mean + z * 128 + piece * 8);
  const uint32_t vw[4] = {v.x, v.y, v.z, v.w}, mw[4] = {m.x, m.y, m.z, m.w};
  uint32_t ow[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float lo = Elem<DT>::from_bits((uint16_t)(vw[k] & 0xffffu)) - Elem<DT>::from_bits((uint16_t)(mw[k] & 0xffffu));
    const float hi = Elem<DT>::from_bits((uint16_t)(vw[k] >> 16)) - Elem<DT>::from_bits((uint16_t)(mw[k] >> 16));
    ow[k] = Elem<DT>::pack2(lo, hi);
  }
  out[(int64_t)z * pieces_per_group + i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// ---- initial centroids (cache_hub/kmeans.py:234-237: index arithmetic in float32) -------------
__global__ void init_centroids_kernel(const uint4* __restrict__ centred, uint4* __restrict__ cent, int n_tok, int n_cen,
                                      float step, float half) {
  const int z = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece
  if (i >= n_cen * 16) return;
  const int c = i >> 4, piece = i & 15;
  const long long idx = (long long)__fadd_rn(__fmul_rn((float)c, step), half);
  const long long row = idx < 0 ? 0 : (idx >= n_tok ? n_tok - 1 : idx);
  cent[((int64_t)z * n_cen + c) * 16 + piece] = ri_ldg16(centred + ((int64_t)z * n_tok + row) * 16 + piece);
}

// ---- bucket ---------------------------------------------------------------------------------
struct BucketArgs {
  const int32_t* assign;   // [total tokens] local centroid ids
  int32_t* order;          // [total tokens] local token ids, cluster-major, ascending inside a cluster
  int32_t* count;          // [problems, n_cen]
  int32_t* offset;         // [problems, n_cen + 1]
  int n_tok, n_cen, seg_per_group;
  int64_t group_stride;
};

// One CTA per problem.  The tokens are cut into `workers` contiguous ranges; a table [workers][n_cen] first holds
// how many tokens of each range fall into each cluster, then (after the scan of the totals) where each range
// starts writing inside each cluster, so that `workers` warps can scatter their ranges side by side and the
// order inside a cluster is still ascending in the token id.
__global__ void __launch_bounds__(1024) kmeans_bucket_kernel(BucketArgs a, int workers) {
  extern __shared__ int32_t bucket_smem[];
  int32_t* cursor = bucket_smem;                 // [n_cen]: counts, then first positions
  int32_t* table = workers == 1 ? bucket_smem : bucket_smem + a.n_cen;   // [workers][n_cen]; one range: the same array
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_carry;
  const int problem = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t tok0 = (int64_t)(problem / a.seg_per_group) * a.group_stride + (int64_t)(problem % a.seg_per_group) * a.n_tok;
  const int32_t* asg = a.assign + tok0;
  const int chunk = ((a.n_tok + workers - 1) / workers + 31) & ~31;     // tokens per range, whole warp steps
  for (int i = tid; i < a.n_cen * (workers == 1 ? 1 : workers + 1); i += 1024) bucket_smem[i] = 0;
  if (tid == 0) s_carry = 0;
  __syncthreads();
  auto clamp_id = [&](int32_t c) { return min(max(c, 0), a.n_cen - 1); };   // never index outside the table
  for (int t = tid; t < a.n_tok; t += 1024) {
    const int c = clamp_id(asg[t]);
    atomicAdd(&table[(t / chunk) * a.n_cen + c], 1);
  }
  __syncthreads();
  for (int c = tid; c < a.n_cen; c += 1024) {
    int total = 0;
    for (int w = 0; w < workers; ++w) total += table[w * a.n_cen + c];
    cursor[c] = total;
  }
  __syncthreads();
  // exclusive scan of the counts, 1024 at a time
  for (int c0 = 0; c0 < a.n_cen; c0 += 1024) {
    const int c = c0 + tid;
    const uint32_t v = c < a.n_cen ? (uint32_t)cursor[c] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    uint32_t ws = warp_sums[lane], winc = ws;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    const uint32_t carry = s_carry;
    const uint32_t excl = carry + __shfl_sync(0xffffffffu, winc - ws, warp) + inc - v;
    if (c < a.n_cen) {
      a.count[(int64_t)problem * a.n_cen + c] = (int32_t)v;
      a.offset[(int64_t)problem * (a.n_cen + 1) + c] = (int32_t)excl;
      // where each range starts inside this cluster
      uint32_t running = excl;
      for (int w = 0; w < workers; ++w) {
        const int32_t n_w = table[w * a.n_cen + c];
        table[w * a.n_cen + c] = (int32_t)running;
        running += (uint32_t)n_w;
      }
    }
    const uint32_t chunk_total = __shfl_sync(0xffffffffu, winc, 31);   // every lane takes part in the shuffle
    __syncthreads();
    if (tid == 1023) s_carry = carry + chunk_total;
    __syncthreads();
  }
  if (tid == 0) a.offset[(int64_t)problem * (a.n_cen + 1) + a.n_cen] = (int32_t)s_carry;
  __syncthreads();
  // stable scatter: warp w takes range w, 32 tokens at a time in token order
  if (warp >= workers) return;
  int32_t* ord = a.order + tok0;
  int32_t* my_cursor = table + warp * a.n_cen;
  const int t_begin = warp * chunk, t_end = min(a.n_tok, t_begin + chunk);
  constexpr int kAhead = 8;
  for (int t0 = t_begin; t0 < t_end; t0 += 32 * kAhead) {
    int32_t cl[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int t = t0 + u * 32 + lane;
      cl[u] = t < t_end ? clamp_id(asg[t]) : -1;
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int t = t0 + u * 32 + lane;
      const unsigned active = __ballot_sync(0xffffffffu, cl[u] >= 0);
      if (cl[u] >= 0) {
        const unsigned peers = __match_any_sync(active, cl[u]);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int pos = my_cursor[cl[u]] + rank;
        ord[pos] = t;
        __syncwarp(active);
        if (lane == 31 - __clz(peers)) my_cursor[cl[u]] = pos + 1;
      }
      __syncwarp();
    }
  }
}

// ---- update ---------------------------------------------------------------------------------
struct UpdateArgs {
  const uint2* centred;      // [Z, N, 128] centred keys
  const uint2* raw_keys;     // optional: uncentred keys for the cluster-contiguous copy
  const uint2* values;       // optional: V rows (value sums + copy)
  const int32_t* order;
  const int32_t* count;
  const int32_t* offset;
  uint2* centroids;          // [problems, n_cen, 128] in/out (centred)
  uint2* out_centroids;      // optional final: centroid + mean
  const uint16_t* mean;      // optional [Z, 128]
  uint2* value_sum;          // optional [Z, C, 128]
  uint16_t* size_dt;         // optional [Z, C]
  uint2* keys_out;           // optional [Z, N, 128]
  uint2* values_out;
  int n_tok, n_cen, seg_per_group, normalize;
  int64_t group_stride;
};

template <int DT>
__device__ __forceinline__ void add_row(float (&acc)[4], uint2 v) {
  acc[0] += Elem<DT>::from_bits((uint16_t)(v.x & 0xffffu));
  acc[1] += Elem<DT>::from_bits((uint16_t)(v.x >> 16));
  acc[2] += Elem<DT>::from_bits((uint16_t)(v.y & 0xffffu));
  acc[3] += Elem<DT>::from_bits((uint16_t)(v.y >> 16));
}

// LAST: the pass that also sums the values and writes the cluster-contiguous copy (three rows per member).
// Cluster sizes are very uneven (median of a few members, a tail of thousands).  With one short-lived CTA per
// eight clusters most CTAs had next to nothing to do and the kernel was bound by CTA turnover (about 220 CTAs
// per SM in a row), so the warps are persistent instead: a few CTAs per SM, warp w of the grid takes clusters
// w, w + W, w + 2W, ... of all problems, which also evens out the large clusters.
template <int DT, bool LAST>
__global__ void __launch_bounds__(256) kmeans_update_kernel(UpdateArgs a, int n_problems) {
  const int lane = threadIdx.x & 31;
  // most clusters hold a handful of rows, so the per-cluster index arithmetic counts: 32-bit, and (problem, c)
  // advance by a fixed step instead of being divided out of the running index (the launcher checks the range)
  const int n_total = n_problems * a.n_cen;
  const int n_warps = (int)gridDim.x * 8;
  const int step_p = n_warps / a.n_cen, step_c = n_warps - step_p * a.n_cen;
  const int idx0 = (int)blockIdx.x * 8 + (int)(threadIdx.x >> 5);
  int problem = idx0 / a.n_cen, c = idx0 - problem * a.n_cen;
  for (int idx = idx0; idx < n_total; idx += n_warps, problem += step_p, c += step_c) {
  if (c >= a.n_cen) { c -= a.n_cen; ++problem; }
  const int z = (int)((unsigned)problem / (unsigned)a.seg_per_group);
  const int64_t tok0 = (int64_t)z * a.group_stride + (int64_t)(problem - z * a.seg_per_group) * a.n_tok;
  const int cnt = a.count[(int64_t)problem * a.n_cen + c];
  const int off = a.offset[(int64_t)problem * (a.n_cen + 1) + c];
  const int32_t* ord = a.order + tok0 + off;
  const int64_t crow = ((int64_t)problem * a.n_cen + c) * 32 + lane;    // uint2 index of this lane's 4 channels
  if (a.size_dt) a.size_dt[(int64_t)problem * a.n_cen + c] = Elem<DT>::bits((float)cnt);

  float ks[4] = {0, 0, 0, 0}, vs[4] = {0, 0, 0, 0};
  constexpr int kUnroll = LAST ? 8 : 4;
  for (int b0 = 0; b0 < cnt; b0 += 32) {
    // the member list of up to 32 rows in one coalesced load; the rows are then fetched kUnroll at a time
    const int my_row = b0 + lane < cnt ? ord[b0 + lane] : -1;
    const int n_here = min(32, cnt - b0);
    for (int j0 = 0; j0 < n_here; j0 += kUnroll) {
      int rows[kUnroll];
      uint2 kv[kUnroll], vv[kUnroll], rk[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) rows[u] = __shfl_sync(0xffffffffu, my_row, (j0 + u) & 31);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (j0 + u < n_here) {
          const int64_t r = (tok0 + rows[u]) * 32 + lane;
          kv[u] = __ldg(a.centred + r);
          if (LAST && a.values) vv[u] = __ldg(a.values + r);
          if (LAST && a.raw_keys) rk[u] = __ldg(a.raw_keys + r);
        }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (j0 + u < n_here) {
          add_row<DT>(ks, kv[u]);           // sequential in list order: bit-identical to a serial sum
          if (LAST && a.values) add_row<DT>(vs, vv[u]);
          if (LAST && a.keys_out) {
            const int64_t o = ((int64_t)z * a.group_stride + off + b0 + j0 + u) * 32 + lane;
            a.keys_out[o] = rk[u];
            a.values_out[o] = vv[u];
          }
        }
    }
  }
  if (a.value_sum) {
    uint2 o;
    o.x = Elem<DT>::pack2(vs[0], vs[1]);
    o.y = Elem<DT>::pack2(vs[2], vs[3]);
    a.value_sum[crow] = o;
  }
  float x[4];
  if (cnt > 0) {
    const float fc = (float)cnt;
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = ks[i] / fc;
    if (a.normalize) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float nrm = sqrtf(ss);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = x[i] / nrm;
    }
    uint2 o;
    o.x = Elem<DT>::pack2(x[0], x[1]);
    o.y = Elem<DT>::pack2(x[2], x[3]);
    a.centroids[crow] = o;
  }
  if (a.out_centroids) {
    // stored centroid = round(centroid_dt + mean_dt), both already in the key dtype
    // (cache_hub/retroinfer_cache.py:429)
    const uint2 cd = a.centroids[crow];
    const uint2 m = *reinterpret_cast<const uint2*>(a.mean + z * 128 + lane * 4);
    uint2 o;
    o.x = Elem<DT>::pack2(Elem<DT>::from_bits((uint16_t)(cd.x & 0xffffu)) + Elem<DT>::from_bits((uint16_t)(m.x & 0xffffu)),
                          Elem<DT>::from_bits((uint16_t)(cd.x >> 16)) + Elem<DT>::from_bits((uint16_t)(m.x >> 16)));
    o.y = Elem<DT>::pack2(Elem<DT>::from_bits((uint16_t)(cd.y & 0xffffu)) + Elem<DT>::from_bits((uint16_t)(m.y & 0xffffu)),
                          Elem<DT>::from_bits((uint16_t)(cd.y >> 16)) + Elem<DT>::from_bits((uint16_t)(m.y >> 16)));
    a.out_centroids[crow] = o;
  }
  }   // next cluster of this warp
}

// ---- host side --------------------------------------------------------------------------------
// rows x 128 channels, 16-bit elements, box = 128 rows x 64 channels, 128-byte swizzle
int make_row_map(CUtensorMap* map, const void* base, int64_t rows, int dtype) {
  return make_map_2d(map, base, 128, rows, 256, dtype);
}

struct FitLayout {
  int64_t cent_work, assign, order, count, offset, centred, mean, partial, error, total;
  int chunks;
};

FitLayout fit_layout(const ri_kmeans* p, bool with_centring) {
  FitLayout L;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = ri_align_up(off + bytes, 1024); return o; };
  const int64_t Z = p->groups, N = p->n_tokens, C = p->n_centroids;
  L.chunks = (int)((N + kMeanRows - 1) / kMeanRows);
  L.error = take(4);
  L.cent_work = take(Z * C * 256);
  L.assign = take(Z * N * 4);
  L.order = take(Z * N * 4);
  L.count = take(Z * C * 4);
  L.offset = take((Z * C + Z * (int64_t)p->n_segments) * 4 + 4);
  L.centred = with_centring ? take(Z * N * 256) : 0;
  L.mean = with_centring ? take(Z * 256) : 0;
  L.partial = with_centring ? take(Z * L.chunks * 512) : 0;
  L.total = off;
  return L;
}

int validate_fit(const ri_kmeans* p) {
  RI_REQUIRE(p != nullptr, "ri_kmeans is null");
  RI_REQUIRE(p->groups > 0 && p->n_tokens > 0 && p->n_centroids > 0, "groups/n_tokens/n_centroids must be positive");
  RI_REQUIRE(p->n_segments >= 1 && p->n_centroids % p->n_segments == 0, "n_centroids must be a multiple of n_segments");
  RI_REQUIRE((p->n_centroids / p->n_segments) % 32 == 0,
             "centroids per segment (%d) must be a multiple of 32", p->n_centroids / p->n_segments);
  RI_REQUIRE(p->n_centroids <= 49152, "n_centroids=%d too large (limit 49152)", p->n_centroids);
  RI_REQUIRE(p->n_iters >= 1, "n_iters must be at least 1");
  RI_REQUIRE(p->dtype == RI_BF16 || p->dtype == RI_F16, "dtype=%d unsupported", p->dtype);
  RI_REQUIRE((int64_t)p->groups * p->n_tokens < (1ll << 31), "groups*n_tokens must stay below 2^31 rows");
  RI_REQUIRE(p->n_tokens / p->n_segments >= 1, "fewer tokens than segments");
  return RI_OK;
}

template <int DT>
int run_fit(const ri_kmeans* p, const FitLayout& L, const void* centred, cudaStream_t s) {
  uint8_t* sc = static_cast<uint8_t*>(p->d_scratch);
  const int Z = p->groups, N = p->n_tokens, C = p->n_centroids, S = p->n_segments;
  int* err = reinterpret_cast<int*>(sc + L.error);
  void* cent = sc + L.cent_work;
  int32_t* assign = p->d_assign ? p->d_assign : reinterpret_cast<int32_t*>(sc + L.assign);
  int32_t* order = p->d_order ? p->d_order : reinterpret_cast<int32_t*>(sc + L.order);
  int32_t* count_work = reinterpret_cast<int32_t*>(sc + L.count);
  int32_t* offset_work = reinterpret_cast<int32_t*>(sc + L.offset);

  RI_CUDA_OK(cudaMemsetAsync(err, 0, 4, s));
  {
    const float step = (float)((double)N / (double)C);
    const float half = (float)((double)N / (double)C / 2.0);
    dim3 grid((C * 16 + 255) / 256, Z);
    init_centroids_kernel<<<grid, 256, 0, s>>>(static_cast<const uint4*>(centred), static_cast<uint4*>(cent), N, C, step, half);
    RI_LAUNCH_OK("init_centroids_kernel");
  }
  CUtensorMap map_keys, map_cent;
  int rc = make_row_map(&map_keys, centred, (int64_t)Z * N, DT);
  if (rc != RI_OK) return rc;
  rc = make_row_map(&map_cent, cent, (int64_t)Z * C, DT);
  if (rc != RI_OK) return rc;
  RI_CUDA_OK(cudaFuncSetAttribute(kmeans_assign_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideSmem));
  RI_CUDA_OK(cudaFuncSetAttribute(kmeans_assign_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kResSmem));

  for (int it = 0; it < p->n_iters; ++it) {
    const bool last = it == p->n_iters - 1;
    const int seg = last ? 1 : S;
    const int n_tok = last ? N : N / S;
    const int n_cen = C / seg;
    const int problems = Z * seg;
    AssignArgs aa;
    aa.assign = assign; aa.error_flag = err; aa.n_tok = n_tok; aa.n_cen = n_cen; aa.seg_per_group = seg;
    aa.group_stride = N;
    aa.idesc = idesc_f16(DT, kTileM, kTileN);
    {
      // blocks per CTA: enough CTAs for about six waves over the SMs, at most 16 blocks each (config 2: 16 blocks in
      // both the segmented and the last iteration, an even split of 32 and 512 blocks; 9 blocks per CTA with a dozen
      // waves left one CTA in four with 5 blocks and cost 2 % of the build)
      WideArgs wa;
      wa.a = aa;
      const int n_blocks = (n_tok + 2 * kTileM - 1) / (2 * kTileM);
      int per = (int)(((int64_t)n_blocks * problems) / (148 * 6));
      per = per < 1 ? 1 : (per > 16 ? 16 : per);
      wa.blocks_per_cta = per;
      dim3 wgrid((n_blocks + per - 1) / per, problems);
      if (n_cen <= 4 * kTileN) {        // the problem's centroids fit shared memory: they stay there
        kmeans_assign_resident_kernel<<<wgrid, kWideThreads, kResSmem, s>>>(map_keys, map_cent, wa);
        RI_LAUNCH_OK("kmeans_assign_resident_kernel");
      } else {
        kmeans_assign_wide_kernel<<<wgrid, kWideThreads, kWideSmem, s>>>(map_keys, map_cent, wa);
        RI_LAUNCH_OK("kmeans_assign_wide_kernel");
      }
    }

    BucketArgs ba;
    ba.assign = assign; ba.order = order;
    ba.count = last && p->d_cluster_count ? p->d_cluster_count : count_work;
    ba.offset = last && p->d_cluster_offset ? p->d_cluster_offset : offset_work;
    ba.n_tok = n_tok; ba.n_cen = n_cen; ba.seg_per_group = seg; ba.group_stride = N;
    // as many token ranges (scattering warps) as fit the shared memory: a table of [ranges + 1][n_cen] words
    int workers = 32;
    while (workers > 1 && (size_t)(workers + 1) * n_cen * 4 > 200 * 1024) workers >>= 1;
    const size_t bsmem = (size_t)(workers == 1 ? 1 : workers + 1) * n_cen * 4;
    RI_REQUIRE(bsmem <= 227 * 1024, "n_centroids per problem = %d too large for the bucket pass", n_cen);
    if (bsmem > 48 * 1024)
      RI_CUDA_OK(cudaFuncSetAttribute(kmeans_bucket_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bsmem));
    kmeans_bucket_kernel<<<problems, 1024, bsmem, s>>>(ba, workers);
    RI_LAUNCH_OK("kmeans_bucket_kernel");

    UpdateArgs ua = {};
    ua.centred = static_cast<const uint2*>(centred);
    ua.order = order; ua.count = ba.count; ua.offset = ba.offset;
    ua.centroids = static_cast<uint2*>(cent);
    ua.n_tok = n_tok; ua.n_cen = n_cen; ua.seg_per_group = seg; ua.normalize = last ? 0 : 1; ua.group_stride = N;
    if (last) {
      ua.values = static_cast<const uint2*>(p->d_values);
      ua.value_sum = static_cast<uint2*>(p->d_value_sum);
      ua.size_dt = static_cast<uint16_t*>(p->d_cluster_size);
      if (p->d_keys_out) {
        ua.raw_keys = static_cast<const uint2*>(p->d_keys);
        ua.keys_out = static_cast<uint2*>(p->d_keys_out);
        ua.values_out = static_cast<uint2*>(p->d_values_out);
      }
      if (p->center) {
        ua.mean = reinterpret_cast<const uint16_t*>(sc + L.mean);
        ua.out_centroids = static_cast<uint2*>(p->d_centroids);
      }
    }
    // persistent warps: as many CTAs as are resident at once
    static int resident[2] = {0, 0};
    const int form = ua.values ? 1 : 0;
    if (resident[form] == 0) {
      int per_sm = 0, sms = 0, dev = 0;
      RI_CUDA_OK(cudaGetDevice(&dev));
      RI_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      if (form) RI_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kmeans_update_kernel<DT, true>, 256, 0));
      else RI_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kmeans_update_kernel<DT, false>, 256, 0));
      resident[form] = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 148);
    }
    RI_REQUIRE((int64_t)n_cen * problems < (1ll << 30), "too many clusters in one launch (%d x %d)", n_cen, problems);
    const int64_t ctas_needed = ((int64_t)n_cen * problems + 7) / 8;
    const int ugrid = (int)(ctas_needed < resident[form] ? ctas_needed : resident[form]);
    if (form) kmeans_update_kernel<DT, true><<<ugrid, 256, 0, s>>>(ua, problems);
    else kmeans_update_kernel<DT, false><<<ugrid, 256, 0, s>>>(ua, problems);
    RI_LAUNCH_OK("kmeans_update_kernel");
  }
  if (!p->center)
    RI_CUDA_OK(cudaMemcpyAsync(p->d_centroids, cent, (size_t)Z * C * 256, cudaMemcpyDeviceToDevice, s));
  if (p->d_error) RI_CUDA_OK(cudaMemcpyAsync(p->d_error, err, 4, cudaMemcpyDeviceToDevice, s));
  return RI_OK;
}

template <int DT>
int run_build(const ri_kmeans* p, cudaStream_t s) {
  const FitLayout L = fit_layout(p, p->center != 0);
  uint8_t* sc = static_cast<uint8_t*>(p->d_scratch);
  const void* centred = p->d_keys;
  if (p->center) {
    const int Z = p->groups, N = p->n_tokens;
    float* partial = reinterpret_cast<float*>(sc + L.partial);
    uint16_t* mean = reinterpret_cast<uint16_t*>(sc + L.mean);
    colsum_partial_kernel<DT><<<dim3(L.chunks, Z), 256, 0, s>>>(static_cast<const uint4*>(p->d_keys), partial, N, L.chunks);
    RI_LAUNCH_OK("colsum_partial_kernel");
    colmean_final_kernel<DT><<<Z, 128, 0, s>>>(partial, mean, N, L.chunks);
    RI_LAUNCH_OK("colmean_final_kernel");
    const int64_t pieces = (int64_t)N * 16;
    centre_apply_kernel<DT><<<dim3((unsigned)((pieces + 255) / 256), Z), 256, 0, s>>>(
        static_cast<const uint4*>(p->d_keys), mean, reinterpret_cast<uint4*>(sc + L.centred), pieces);
    RI_LAUNCH_OK("centre_apply_kernel");
    centred = sc + L.centred;
    if (p->d_mean_key) RI_CUDA_OK(cudaMemcpyAsync(p->d_mean_key, mean, (size_t)Z * 256, cudaMemcpyDeviceToDevice, s));
  }
  return run_fit<DT>(p, L, centred, s);
}

}  // namespace

extern "C" int64_t ri_kmeans_scratch_bytes(const ri_kmeans* p) {
  if (validate_fit(p) != RI_OK) return RI_ERR_INVALID;
  return fit_layout(p, p->center != 0).total;
}

extern "C" int ri_kmeans_build(const ri_kmeans* p, void* stream) {
  int rc = validate_fit(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(p->d_keys && p->d_values && p->d_centroids && p->d_value_sum && p->d_cluster_size && p->d_scratch,
             "ri_kmeans: a required pointer is null");
  RI_REQUIRE((p->d_keys_out == nullptr) == (p->d_values_out == nullptr), "keys_out and values_out go together");
  RI_REQUIRE(((uintptr_t)p->d_keys | (uintptr_t)p->d_values | (uintptr_t)p->d_centroids | (uintptr_t)p->d_value_sum |
              (uintptr_t)p->d_scratch | (uintptr_t)p->d_keys_out | (uintptr_t)p->d_values_out) % 16 == 0,
             "tensor pointers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return p->dtype == RI_BF16 ? run_build<RI_BF16>(p, s) : run_build<RI_F16>(p, s);
}
