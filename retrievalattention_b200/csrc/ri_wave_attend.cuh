// attend: split-K weighted flash decoding over (a) the estimation set — every estimated cluster is
// one row: score from the scan, value = the cluster's value sum, weight = cluster size in the
// softmax denominator — and (b) the exact set — steady zone followed by the retrieved clusters, read
// in place from the cluster-contiguous KV store through the row list.
// (reference: the two weighted_flash_decoding calls, cache_hub/retroinfer_cache.py:611-617 and
// :666-674, with gather_copy_vectors :601-605 and gather_copy_and_concat :642-648 in between).
//
// Work decomposition: a fixed, SM-filling grid of 8-CTA clusters (2 CTAs per SM, 4 warps each); a
// cluster works on one group at a time.  Inside a group the 16-row steps (ceil(E/16) estimation steps, then
// ceil((steady + retrieved rows)/16) exact steps) are cut into equal-cost contiguous ranges, one
// per warp (an exact step moves twice the bytes of an estimation step).  A warp streams its steps
// through a lane-private three-stage cp.async ring in shared memory (256 bytes per lane and step;
// the row ids of the next step to issue are prefetched into registers) and keeps running
// (max, sum, O).  The four warps of a CTA merge in shared memory into one partial result; the 8 CTAs
// of a group form a thread-block cluster and merge their partials by log-sum-exp through
// distributed shared memory, each CTA finishing one eighth of the output values.
//
// Tensor-core use: m16n8k16 MMA.  QK^T has the GQA group in M and 8 rows in N, with the same
// channel permutation on both operands as in the scan.  PV is computed transposed (16 channels in
// M, the 8 heads in N, 16 rows in K): lane (r, t) owns rows tt = {2t, 2t+1, 8+2t, 9+2t} of the step
// and, of each, the 16-byte pieces r and r+8 (channels 8r..8r+7 and 64+8r..64+8r+7).  O^T tile x
// takes channel word x of those pieces: low halves are MMA rows r, high halves rows r+8, so tile x,
// row r is channel ch(x) = (x<4 ? 8r+2x : 64+8r+2(x-4)) and row r+8 is ch(x)+1.  The probabilities
// come straight from the QK^T accumulators as the B fragment.
//
// The per-group body is a device function shared by the stand-alone kernel and the single-kernel
// decode path.
#pragma once

#include <cooperative_groups.h>

#include "ri_wave_internal.cuh"

namespace ri_wave {

namespace cg = cooperative_groups;


#ifndef RI_ATTEND_STAGES
#define RI_ATTEND_STAGES 3
#endif
constexpr int kStages = RI_ATTEND_STAGES;
constexpr int kCtasPerSm = RI_ATTEND_STAGES == 2 ? 3 : 2;
constexpr int kAttendCluster = 8;   // CTAs per group
#ifndef RI_COST_EST
#define RI_COST_EST 2
#define RI_COST_EXACT 3
#endif
// relative cost of a step when the steps of a group are shared out (an estimation step moves half the bytes of an
// exact one); RI_COST_EST / RI_COST_EXACT in the environment override them (tuning)
constexpr int kStageBytes = 16 * 32 * 16;       // 16 pieces x 32 lanes x 16 bytes = 8 KB per warp and stage
constexpr int kRingBytes = 4 * kStages * kStageBytes;

struct AttendArgs {
  const uint4* q;
  const uint4* keys;
  const uint4* values;
  const uint4* steady_k;
  const uint4* steady_v;
  const uint4* value_sum;
  const int32_t* static_len;
  const int32_t* rows;       // null: exact row i is row i of keys/values (execution-buffer mode)
  const int32_t* n_exact;
  const int32_t* est_ids;
  const float* est_w;
  const float* est_s2;
  void* out;
  int64_t N;
  int G, C, gs, E, e_pad, e_steps, steady_stride, max_rows;
  float scale2;        // log2(e) / sqrt(d)
  int cost_est, cost_exact;   // relative cost of an estimation / exact step when the steps are shared out
  uint16_t* const* copies;    // device array of n_copies more destinations of the output (other GPUs' gather buffers)
  int n_copies;
  // operator form (ri_weighted_flash_decoding), all optional: a weight per exact row in the softmax denominator,
  // a previous partial result to merge with, and the log-sum-exp of the result
  const uint16_t* row_w;      // [G, N] in the 16-bit type
  const uint16_t* prev_out;   // [G, gs, 128]
  const float* prev_lse;      // [G, gs] natural log
  float* lse_out;             // [G, gs] natural log
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DT>
__device__ __forceinline__ void pv_step(float (&acc)[8][4], const uint4 (&v)[4][2], uint32_t b0, uint32_t b1) {
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int piece = x >> 2, w = x & 3;
    const uint32_t t0 = (&v[0][piece].x)[w], t1 = (&v[1][piece].x)[w];
    const uint32_t t2 = (&v[2][piece].x)[w], t3 = (&v[3][piece].x)[w];
    const uint32_t a0 = __byte_perm(t0, t1, 0x5410), a1 = __byte_perm(t0, t1, 0x7632);
    const uint32_t a2 = __byte_perm(t2, t3, 0x5410), a3 = __byte_perm(t2, t3, 0x7632);
    Elem<DT>::mma16816(acc[x], a0, a1, a2, a3, b0, b1);
  }
}

struct RowIds { int k[2]; int v[4]; };   // >= 0: row of the KV store / cluster id; < 0: steady row -1-id

// Shared-memory lists of the single-kernel path (LOCAL mode of attend_group): this CTA's own estimation
// entries and its range of the group's exact steps, the retrieved rows given by the kept clusters.
struct LocalLists {
  const uint16_t* est_idx;   // [n_est] centroid index inside this CTA's slice, ascending
  const float* est_wt;       // [n_est] weight (cluster size)
  const float* est_sc;       // [gs][cap] log2-domain scores
  int cap, n_est, slice_lo;
  const uint32_t* dstart;    // [keep + 1] first position of each kept cluster in the retrieved-row list; [keep] = total
  const uint32_t* doff;      // [keep] its first row in the KV store
  int keep, n_rows;          // kept clusters, retrieved rows kept
  int x_lo, x_hi;            // this CTA's exact steps [x_lo, x_hi) of ceil((steady + n_rows) / 16)
};

// The value-sum rows of one estimation step (pieces 8..15 of a ring stage), ids = this lane's four clusters.
__device__ __forceinline__ void issue_value_sums(const uint4* value_sum, int64_t g, int C, uint32_t dst, const int (&ids)[4], int r) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4* p = value_sum + (g * C + ids[i]) * 16;
    cp_async16(dst + (8 + 2 * i) * 512, p + r);
    cp_async16(dst + (9 + 2 * i) * 512, p + r + 8);
  }
}

// One group's attention by one cluster of CPG CTAs of WARPS warps each (CTA `cl` of it).  `ring`:
// WARPS * kStages * kStageBytes of 16-byte aligned dynamic shared memory.  `n_exact_known` >= 0: the group's retrieved-row count, when the caller has it at
// hand (otherwise it is read from a.n_exact).  Ends with a cluster barrier after the last remote read, so the shared
// memory may be reused (or the CTA may exit) when it returns.
template <int DT, bool LOCAL = false, int WARPS = 4, int CPG = kAttendCluster>
__device__ __forceinline__ void attend_group(const AttendArgs& a, const int g, const int cl, uint8_t* ring,
                                             const LocalLists* ll = nullptr) {
  __shared__ float sm_m[WARPS][kMaxHeads], sm_l[WARPS][kMaxHeads];
  __shared__ float cta_m[kMaxHeads], cta_l[kMaxHeads];   // this CTA's partial result: (max, sum) here, O in the ring
  float (*cta_o)[RI_HEAD_DIM] = reinterpret_cast<float (*)[RI_HEAD_DIM]>(ring + WARPS * kStageBytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int gs = a.gs, es = LOCAL ? (ll->n_est + 15) / 16 : a.e_steps;
  const int static_len = a.static_len ? *a.static_len : 0;   // null: the exact rows already contain the steady zone
  cg::cluster_group cluster = cg::this_cluster();
  constexpr int cpg = CPG;                               // CTAs per group
  constexpr int kThreads = WARPS * 32;
  // ring: stage-major, slot (stage, warp) at (stage * WARPS + warp) * kStageBytes
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring) + warp * kStageBytes + lane * 16;
  const uint8_t* my_ring_ptr = ring + warp * kStageBytes + lane * 16;
  constexpr int kStageStride = WARPS * kStageBytes;
  auto warp_o = [&](int w) { return reinterpret_cast<float*>(ring + w * kStageBytes); };   // stage 0 of warp w

  const int te = static_len + (LOCAL ? ll->n_rows : __ldcg(a.n_exact + g));           // steady + retrieved rows
  // The step sequence this CTA's warps share: LOCAL: its own estimation steps, then its exact steps
  // [x_lo, x_hi); otherwise the whole group's estimation steps, then all exact steps, shared by all 32 warps.
  const int x_first = LOCAL ? ll->x_lo : 0;
  const int xs = LOCAL ? ll->x_hi - ll->x_lo : (te + 15) / 16;
  const int n_est_rows = LOCAL ? ll->n_est : a.E;
  // cost units: kCostEst per estimation step, kCostExact per exact step; a step belongs to the warp holding
  // its first unit (an estimation step moves half the bytes but costs about two thirds of the time, measured)
  const int kCostEst = a.cost_est, kCostExact = a.cost_exact;
  const int units = kCostEst * es + kCostExact * xs;
  const int n_w = LOCAL ? WARPS : cpg * WARPS, wl = LOCAL ? warp : cl * WARPS + warp;
  const int per = max(kCostExact, (units + n_w - 1) / n_w);
  auto steps_before_unit = [&](int u) {
    return u < kCostEst * es ? (u + kCostEst - 1) / kCostEst : es + (u - kCostEst * es + kCostExact - 1) / kCostExact;
  };
  const int lu = min(units, wl * per), hu = min(units, lu + per);
  const int lo = steps_before_unit(lu), hi = steps_before_unit(hu);
  // This warp's steps, numbered j = 0 .. n_steps - 1.  Shared sequence (not LOCAL): steps lo .. hi - 1 of it.
  // LOCAL: the CTA's estimation steps go round the warps (warp w: steps w, w + WARPS, ...), then a contiguous range
  // of the CTA's exact steps, sized so that every warp ends up with the same number of steps (+-1).
  int n_steps = hi - lo, e_w = 0, xa = 0;
  if (LOCAL) {
    const int S = es + xs;
    e_w = es / WARPS + (warp < es % WARPS ? 1 : 0);
    n_steps = S / WARPS + (warp < S % WARPS ? 1 : 0);
    xa = x_first + (warp * (S / WARPS) + min(warp, S % WARPS)) - (warp * (es / WARPS) + min(warp, es % WARPS));
  }
  auto locate = [&](int j, bool& est, int& base) {
    if (LOCAL) { est = j < e_w; base = (est ? warp + j * WARPS : xa + j - e_w) * 16; }
    else { const int s = lo + j; est = s < es; base = (est ? s : s - es) * 16; }
  };

  // ids of the rows this lane touches in step j (called by whole warps, in increasing j)
  int hint = -1;               // LOCAL: kept cluster holding the first retrieved row of the step being resolved
  auto load_ids = [&](int j) {
    RowIds id;
    bool est;
    int base;
    locate(j, est, base);
    const int last = (est ? n_est_rows : te) - 1;
    const int tt[4] = {2 * t, 2 * t + 1, 8 + 2 * t, 9 + 2 * t};
    if (LOCAL && !est) {
      // lanes 0..15 resolve row base+lane through the kept-cluster list, then the warp shares them out
      const int i = min(base + (lane & 15), last);
      int myrow = -1 - i, myci = hint;
      if (hint < 0 && base + 15 >= static_len) {     // first step of this warp that reaches the retrieved rows
        const int ri0 = max(base - static_len, 0);
        int lo_c = 0, hi_c = ll->keep;               // largest c with dstart[c] <= ri0 (dstart[0] = 0)
        while (hi_c - lo_c > 1) {
          const int mid = (lo_c + hi_c) >> 1;
          if ((int)ll->dstart[mid] <= ri0) lo_c = mid; else hi_c = mid;
        }
        hint = lo_c;
        myci = lo_c;
      }
      if (i >= static_len) {
        const int ri = i - static_len;
        while (myci + 1 < ll->keep && ri >= (int)ll->dstart[myci + 1]) ++myci;   // dstart[keep] = n_rows > ri
        myrow = (int)ll->doff[myci] + ri - (int)ll->dstart[myci];
      }
      hint = __shfl_sync(0xffffffffu, myci, 15);
#pragma unroll
      for (int i2 = 0; i2 < 4; ++i2) id.v[i2] = __shfl_sync(0xffffffffu, myrow, tt[i2]);
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) id.k[jj] = __shfl_sync(0xffffffffu, myrow, jj * 8 + r);
      return id;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = min(base + tt[i], last);
      if (est) id.v[i] = LOCAL ? ll->slice_lo + (int)ll->est_idx[row] : __ldcg(a.est_ids + (int64_t)g * a.e_pad + row);
      else id.v[i] = row < static_len ? -1 - row : (a.rows ? __ldcg(a.rows + (int64_t)g * a.max_rows + row - static_len) : row - static_len);
    }
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int row = min(base + jj * 8 + r, last);
      id.k[jj] = est ? 0 : (row < static_len ? -1 - row : (a.rows ? __ldcg(a.rows + (int64_t)g * a.max_rows + row - static_len) : row - static_len));
    }
    return id;
  };
  // start the copies of step j into ring stage `stage`
  auto issue = [&](int j, int stage, const RowIds& id) {
    const uint32_t dst = my_ring + stage * kStageStride;
    bool est;
    int base;
    locate(j, est, base);
    if (est) {
      // pieces 0/1: this lane's scores and weights of the step (LOCAL: read from the lists when the step
      // is consumed); pieces 8..15: value-sum rows
      if (!LOCAL) {
        const int i0 = base + 2 * t;
        if (r < gs) {
          const float* sp = a.est_s2 + ((int64_t)g * kMaxHeads + r) * a.e_pad + i0;
          cp_async8(dst, sp);
          cp_async8(dst + 8, sp + 8);
        }
        const float* wp = a.est_w + (int64_t)g * a.e_pad + i0;
        cp_async8(dst + 512, wp);
        cp_async8(dst + 512 + 8, wp + 8);
      }
      issue_value_sums(a.value_sum, g, a.C, dst, id.v, r);
    } else {
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int x = id.k[jj];
        const uint4* p = x < 0 ? a.steady_k + ((int64_t)g * a.steady_stride + (-1 - x)) * 16
                               : a.keys + ((int64_t)g * a.N + x) * 16;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) cp_async16(dst + (4 * jj + kk) * 512, p + t + kk * 4);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int x = id.v[i];
        const uint4* p = x < 0 ? a.steady_v + ((int64_t)g * a.steady_stride + (-1 - x)) * 16
                               : a.values + ((int64_t)g * a.N + x) * 16;
        cp_async16(dst + (8 + 2 * i) * 512, p + r);
        cp_async16(dst + (9 + 2 * i) * 512, p + r + 8);
      }
    }
  };

  // ---- prologue: fill the ring (the ids of all its steps are fetched before the first copy is issued,
  //      so their latencies overlap) ----
  int j_issue = min(kStages, n_steps);
  RowIds nid;
  {
    RowIds pid[kStages];
#pragma unroll
    for (int st = 0; st < kStages; ++st)
      if (st < n_steps) pid[st] = load_ids(st);
#pragma unroll
    for (int st = 0; st < kStages; ++st) {
      if (st < n_steps) issue(st, st, pid[st]);
      cp_async_commit();
    }
    if (j_issue < n_steps) nid = load_ids(j_issue);
  }
  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < gs ? ri_ldg16(a.q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);
  float acc[8][4];
#pragma unroll
  for (int x = 0; x < 8; ++x)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[x][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;   // head r (l: this lane's share, reduced over the quad at the end)
  int stage = 0;
#pragma unroll 1
  for (int j = 0; j < n_steps; ++j) {
    bool is_est;
    int base;
    locate(j, is_est, base);
    float rw[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if (!LOCAL && a.row_w != nullptr && !is_est) {   // operator form: weights of this lane's four exact rows
      const int b0 = base + 2 * t;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int row = min(b0 + jj * 8 + e, te - 1);
          rw[jj][e] = Elem<DT>::from_bits(a.row_w[(int64_t)g * a.N + row]);
        }
    }
    cp_async_wait<kStages - 1>();           // the group of step s has landed (lane-private slots: no barrier)
    if (j == 0) RI_FT(10);
    const uint8_t* src = my_ring_ptr + stage * kStageStride;
    const int rows_end = is_est ? n_est_rows : te;

    float s2[2][2];
    float w[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if (is_est) {
      float4 sv, wv;
      if (LOCAL) {
        const int j0 = base + 2 * t;                 // < cap: cap is a multiple of 16 and n_est <= cap
        const float2 a0 = *reinterpret_cast<const float2*>(ll->est_sc + (r < gs ? r : 0) * ll->cap + j0);
        const float2 a1 = *reinterpret_cast<const float2*>(ll->est_sc + (r < gs ? r : 0) * ll->cap + j0 + 8);
        const float2 w0 = *reinterpret_cast<const float2*>(ll->est_wt + j0);
        const float2 w1 = *reinterpret_cast<const float2*>(ll->est_wt + j0 + 8);
        sv = make_float4(a0.x, a0.y, a1.x, a1.y);
        wv = make_float4(w0.x, w0.y, w1.x, w1.y);
      } else {
        sv = *reinterpret_cast<const float4*>(src);
        wv = *reinterpret_cast<const float4*>(src + 512);
      }
      const bool head = r < gs;
      s2[0][0] = head ? sv.x : -INFINITY; s2[0][1] = head ? sv.y : -INFINITY;
      s2[1][0] = head ? sv.z : -INFINITY; s2[1][1] = head ? sv.w : -INFINITY;
      w[0][0] = wv.x; w[0][1] = wv.y; w[1][0] = wv.z; w[1][1] = wv.w;
    } else {
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        // two independent accumulation chains of four MMAs each instead of one of eight
        float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint4 kb = *reinterpret_cast<const uint4*>(src + (4 * jj + kk) * 512);
          Elem<DT>::mma16816(c, qa[kk].x, 0u, qa[kk].y, 0u, kb.x, kb.y);
          Elem<DT>::mma16816(c2, qa[kk].z, 0u, qa[kk].w, 0u, kb.z, kb.w);
        }
        s2[jj][0] = (c[0] + c2[0]) * a.scale2;
        s2[jj][1] = (c[1] + c2[1]) * a.scale2;
        w[jj][0] = rw[jj][0];
        w[jj][1] = rw[jj][1];
      }
    }
#pragma unroll
    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (base + jj * 8 + 2 * t + e >= rows_end) { s2[jj][e] = -INFINITY; w[jj][e] = 0.f; }

    // online softmax for head r
    float mx = fmaxf(fmaxf(s2[0][0], s2[0][1]), fmaxf(s2[1][0], s2[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_safe);   // m_run = -inf -> 0
    float p[2][2];
    float psum = 0.f;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[jj][e] = exp2f(s2[jj][e] - m_safe);
        psum += p[jj][e] * w[jj][e];
      }
    l_run = l_run * alpha + psum;
    m_run = m_new;
    // the accumulators hold heads 2t and 2t+1: fetch their rescale factors from the quads that own them
    const float f0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4);
    const float f1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
    for (int x = 0; x < 8; ++x) { acc[x][0] *= f0; acc[x][1] *= f1; acc[x][2] *= f0; acc[x][3] *= f1; }
    uint4 v[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i][0] = *reinterpret_cast<const uint4*>(src + (8 + 2 * i) * 512);
      v[i][1] = *reinterpret_cast<const uint4*>(src + (9 + 2 * i) * 512);
    }
    pv_step<DT>(acc, v, Elem<DT>::pack2(p[0][0], p[0][1]), Elem<DT>::pack2(p[1][0], p[1][1]));

    // refill the stage just consumed (the same lane wrote and read it), then fetch the ids after that
    if (j_issue < n_steps) {
      issue(j_issue, stage, nid);
      ++j_issue;
      if (j_issue < n_steps) nid = load_ids(j_issue);
    }
    cp_async_commit();
    stage = stage + 1 == kStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();
  RI_FT(11);

  // ---- merge the warps of this CTA (each parks its 8 x 128 accumulator in its own idle ring region) ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (t == 0) { sm_m[warp][r] = m_run; sm_l[warp][r] = l_run; }
  {
    float* my_o = warp_o(warp);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const int ch = (x < 4) ? 8 * r + 2 * x : 64 + 8 * r + 2 * (x - 4);
      my_o[(2 * t) * RI_HEAD_DIM + ch] = acc[x][0];
      my_o[(2 * t + 1) * RI_HEAD_DIM + ch] = acc[x][1];
      my_o[(2 * t) * RI_HEAD_DIM + ch + 1] = acc[x][2];
      my_o[(2 * t + 1) * RI_HEAD_DIM + ch + 1] = acc[x][3];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gs * RI_HEAD_DIM; idx += kThreads) {
    const int h = idx >> 7, ch = idx & (RI_HEAD_DIM - 1);
    float M = -INFINITY;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) M = fmaxf(M, sm_m[wi][h]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) {
      const float f = exp2f(sm_m[wi][h] - Ms);
      L += sm_l[wi][h] * f;
      O += warp_o(wi)[h * RI_HEAD_DIM + ch] * f;
    }
    cta_o[h][ch] = O;
    if (ch == 0) { cta_m[h] = M; cta_l[h] = L; }
  }
  cluster.sync();
  RI_FT(12);

  // ---- merge the partial results of the group's CTAs through distributed shared memory: this CTA
  //      finishes values [cl * share, (cl+1) * share) of the gs*128 outputs ----
  const int share = (gs * RI_HEAD_DIM + cpg - 1) / cpg;
  for (int tv = tid; tv < share; tv += kThreads) {
    const int v = cl * share + tv, h = v >> 7, ch = v & 127;
    if (v >= gs * RI_HEAD_DIM) break;      // cluster sizes that do not divide the outputs: the last CTA's share is short
    float mc[cpg], lc[cpg], oc[cpg];
#pragma unroll
    for (int c = 0; c < cpg; ++c) {
      mc[c] = cluster.map_shared_rank(cta_m, c)[h];
      lc[c] = cluster.map_shared_rank(cta_l, c)[h];
      oc[c] = cluster.map_shared_rank(&cta_o[0][0], c)[h * RI_HEAD_DIM + ch];
    }
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < cpg; ++c) M = fmaxf(M, mc[c]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int c = 0; c < cpg; ++c) {
      const float f = exp2f(mc[c] - Ms);
      L += lc[c] * f;
      O += oc[c] * f;
    }
    const int64_t idx = ((int64_t)g * gs + h) * RI_HEAD_DIM + ch;
    float Mt = Ms;                         // log2-domain reference of L and O
    if (a.prev_lse != nullptr) {           // operator form: merge with a previous partial result
      const float mp = a.prev_lse[(int64_t)g * gs + h] * RI_LOG2E;
      const float op = Elem<DT>::from_bits(a.prev_out[idx]);
      const float Mn = fmaxf(M, mp);
      Mt = Mn == -INFINITY ? 0.f : Mn;
      const float fa = M == -INFINITY ? 0.f : exp2f(M - Mt), fb = mp == -INFINITY ? 0.f : exp2f(mp - Mt);
      L = L * fa + fb;
      O = O * fa + op * fb;
    }
    if (a.lse_out != nullptr && ch == 0)
      a.lse_out[(int64_t)g * gs + h] = L > 0.f ? (Mt + log2f(L)) * 0.6931471805599453f : -INFINITY;
    const uint16_t bits = Elem<DT>::bits(L > 0.f ? O / L : 0.f);
    reinterpret_cast<uint16_t*>(a.out)[idx] = bits;
    for (int c = 0; c < a.n_copies; ++c) a.copies[c][idx] = bits;   // several GPUs: the other ranks' gather buffers
  }
  cluster.sync();                        // remote reads done: the partials and the ring may be reused
}

inline void fill_attend_args(const ri_wave_layer& p, const Layout& L, const ExecBuffer* eb, AttendArgs& a) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  a.q = static_cast<const uint4*>(p.d_q);
  a.keys = static_cast<const uint4*>(p.d_keys);
  a.values = static_cast<const uint4*>(p.d_values);
  a.steady_k = static_cast<const uint4*>(p.d_steady_keys);
  a.steady_v = static_cast<const uint4*>(p.d_steady_values);
  a.value_sum = static_cast<const uint4*>(p.d_value_sum);
  a.static_len = p.d_static_len;
  a.rows = reinterpret_cast<const int32_t*>(sc + L.rows);
  a.n_exact = reinterpret_cast<const int32_t*>(sc + L.n_exact);
  a.est_ids = reinterpret_cast<const int32_t*>(sc + L.est_ids);
  a.est_w = reinterpret_cast<const float*>(sc + L.est_w);
  a.est_s2 = reinterpret_cast<const float*>(sc + L.est_s2);
  a.out = p.d_out;
  a.N = p.tokens_per_group;
  a.G = p.groups; a.C = p.n_centroids; a.gs = p.group_size; a.E = p.n_estimate; a.e_pad = L.e_pad;
  a.e_steps = (p.n_estimate + 15) / 16;
  a.steady_stride = p.steady_stride; a.max_rows = p.max_exact_rows;
  a.scale2 = RI_LOG2E * 0.08838834764831845f;
  a.copies = nullptr;
  a.n_copies = 0;
  a.row_w = nullptr; a.prev_out = nullptr; a.prev_lse = nullptr; a.lse_out = nullptr;
  static const int cost_est = getenv("RI_COST_EST") ? atoi(getenv("RI_COST_EST")) : RI_COST_EST;
  static const int cost_exact = getenv("RI_COST_EXACT") ? atoi(getenv("RI_COST_EXACT")) : RI_COST_EXACT;
  a.cost_est = cost_est > 0 ? cost_est : 1;
  a.cost_exact = cost_exact > 0 ? cost_exact : 1;
  if (eb) {   // exact rows = the first lengths[g] rows of a dense buffer that already starts with the steady zone
    a.keys = static_cast<const uint4*>(eb->keys);
    a.values = static_cast<const uint4*>(eb->values);
    a.N = eb->stride;
    a.n_exact = eb->lengths;
    a.static_len = nullptr;
    a.rows = nullptr;
    a.lse_out = eb->lse_out;
  }
}

}  // namespace ri_wave
