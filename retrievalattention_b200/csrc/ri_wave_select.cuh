// select: per group, turn the centroid scores into the retrieval set (top P, ranked), the
// estimation set (next E) and the row list of the retrieved clusters.
//
// One thread-block cluster of 8 CTAs works on one group; every CTA owns a contiguous slice of the
// centroids and the CTAs exchange histograms, counts and the P retrieval candidates through
// distributed shared memory.  Steps (reference arithmetic: cache_hub/retroinfer_cache.py:569-575):
//   1. (caller) softmax statistics per head: maximum and 1/sum of exponentials of the rounded scores;
//   2. dist = round(sum_h round(exp(round(s_h) - max_h) / sum_h)), empty clusters forced to the most
//      negative value, mapped to order-preserving 16-bit keys;
//   3. exact two-level radix select (high byte, then low byte) of the P-th and (P+E)-th largest
//      key; ties at a cut are taken in ascending cluster id;
//   4. ordered compaction: estimation entries (id, weight = cluster size, log2-domain scores) to
//      global memory, retrieval candidates to CTA 0;
//   5. CTA 0 ranks the P candidates (descending key, ascending id), applies the page-budget prefix
//      rule (wave_buffer_cpu.cpp:207-216) and computes each kept cluster's place in the row list;
//   6. all CTAs expand the kept clusters into row indices.
//
// The body is a device function so that the stand-alone selection kernel (256 threads) and the
// single-kernel decode path (128 threads, selection between its scan and attend phases) share it.
#pragma once

#include <cooperative_groups.h>

#include "ri_wave_internal.cuh"

namespace ri_wave {

namespace cg = cooperative_groups;

struct SelectArgs {
  const float* scores;
  const float* tile_max;
  const float* tile_sum;
  const uint16_t* size_dt;
  const int32_t* count;
  const int32_t* offset;
  uint16_t* dist_keys;
  int32_t* est_ids;
  float* est_w;
  float* est_s2;
  int32_t* rows;
  int32_t* n_exact;
  int64_t* retrieved_ids;
  int32_t* retrieved_kept;
  int64_t* estimated_ids;
  int C, gs, P, E, e_pad, page, buffer_pages, max_rows, n_tiles, slice, p_pad;
};

// Dynamic shared memory the body needs: the slice's keys and seven arrays of p_pad words.
inline size_t select_dyn_bytes(const SelectArgs& a) { return ri_align16((size_t)a.slice * 2) + (size_t)a.p_pad * 28; }

inline int fill_select_args(const ri_wave_layer& p, const Layout& L, SelectArgs& a) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  a.scores = reinterpret_cast<const float*>(sc + L.scores);
  a.tile_max = reinterpret_cast<const float*>(sc + L.tile_max);
  a.tile_sum = reinterpret_cast<const float*>(sc + L.tile_sum);
  a.size_dt = static_cast<const uint16_t*>(p.d_cluster_size);
  a.count = p.d_cluster_count;
  a.offset = p.d_cluster_offset;
  a.dist_keys = reinterpret_cast<uint16_t*>(sc + L.dist_keys);
  a.est_ids = reinterpret_cast<int32_t*>(sc + L.est_ids);
  a.est_w = reinterpret_cast<float*>(sc + L.est_w);
  a.est_s2 = reinterpret_cast<float*>(sc + L.est_s2);
  a.rows = reinterpret_cast<int32_t*>(sc + L.rows);
  a.n_exact = reinterpret_cast<int32_t*>(sc + L.n_exact);
  a.retrieved_ids = p.d_retrieved_ids;
  a.retrieved_kept = p.d_retrieved_kept;
  a.estimated_ids = p.d_estimated_ids;
  a.C = p.n_centroids; a.gs = p.group_size; a.P = p.nprobe; a.E = p.n_estimate; a.e_pad = L.e_pad;
  a.page = p.page_size; a.buffer_pages = p.buffer_pages; a.max_rows = p.max_exact_rows; a.n_tiles = L.n_tiles;
  a.slice = ((p.n_centroids / 8 + kSelectCluster - 1) / kSelectCluster) * 8;
  a.p_pad = (int)ri_align_up(p.nprobe, 4);
  RI_REQUIRE(p.max_exact_rows < (1 << 20), "max_exact_rows=%d too large (limit 2^20 - 1)", p.max_exact_rows);
  return RI_OK;
}

// Exclusive scan of one value per thread over the block.  `total` = block sum.
template <int THREADS, typename T>
__device__ __forceinline__ T block_scan(T v, T* warp_sums, T& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();   // protects warp_sums from its previous use
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  T base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) {
    const T x = warp_sums[w];
    if (w < warp) base += x;
    tot += x;
  }
  total = tot;
  return base + inc - v;
}

__device__ __forceinline__ void cluster_arrive() {
  __syncwarp();   // .aligned: the whole warp must execute the instruction together
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  __syncwarp();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Two histograms of 256 bins (bin 255 = largest keys), each given as the cluster-wide sum (ga, gb)
// and this CTA's own counts (la, lb); counts fit 16 bits.  For histogram a find the bin where the
// count from the top first reaches ka (>= 1), likewise b/kb, with ONE packed scan; a thread looks
// after 256/THREADS consecutive bins.
// out?[0] = bin, out?[1] = cluster-wide count above it, out?[2] = this CTA's count above it.
template <int THREADS>
__device__ __forceinline__ void find_bins(const int* ga, const int* la, int ka, int* outa, const int* gb,
                                          const int* lb, int kb, int* outb, uint64_t* warp_sums) {
  constexpr int BPT = 256 / THREADS;
  uint64_t v[BPT], sum = 0;
#pragma unroll
  for (int j = 0; j < BPT; ++j) {
    const int bin = 255 - ((int)threadIdx.x * BPT + j);
    v[j] = (uint64_t)ga[bin] | ((uint64_t)la[bin] << 16) | ((uint64_t)gb[bin] << 32) | ((uint64_t)lb[bin] << 48);
    sum += v[j];
  }
  uint64_t total;
  uint64_t pre = block_scan<THREADS, uint64_t>(sum, warp_sums, total);
#pragma unroll
  for (int j = 0; j < BPT; ++j) {
    const int bin = 255 - ((int)threadIdx.x * BPT + j);
    const int ca = (int)(v[j] & 0xffffu), cb = (int)((v[j] >> 32) & 0xffffu);
    const int above_a = (int)(pre & 0xffffu), above_la = (int)((pre >> 16) & 0xffffu);
    const int above_b = (int)((pre >> 32) & 0xffffu), above_lb = (int)(pre >> 48);
    if (above_a < ka && above_a + ca >= ka) { outa[0] = bin; outa[1] = above_a; outa[2] = above_la; }
    if (above_b < kb && above_b + cb >= kb) { outb[0] = bin; outb[1] = above_b; outb[2] = above_lb; }
    pre += v[j];
  }
  __syncthreads();
}

// The same search with the counts of a thread's two bins (255-2*tid, then 254-2*tid) given in registers.
template <int THREADS>
__device__ __forceinline__ void find_bins_regs(const int (&ga)[2], const int (&la)[2], int ka, int* outa,
                                               const int (&gb)[2], const int (&lb)[2], int kb, int* outb,
                                               uint64_t* warp_sums) {
  static_assert(THREADS == 128, "two bins per thread");
  uint64_t v[2], sum = 0;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    v[j] = (uint64_t)ga[j] | ((uint64_t)la[j] << 16) | ((uint64_t)gb[j] << 32) | ((uint64_t)lb[j] << 48);
    sum += v[j];
  }
  uint64_t total;
  uint64_t pre = block_scan<THREADS, uint64_t>(sum, warp_sums, total);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int bin = 255 - ((int)threadIdx.x * 2 + j);
    const int above_a = (int)(pre & 0xffffu), above_la = (int)((pre >> 16) & 0xffffu);
    const int above_b = (int)((pre >> 32) & 0xffffu), above_lb = (int)(pre >> 48);
    if (above_a < ka && above_a + ga[j] >= ka) { outa[0] = bin; outa[1] = above_a; outa[2] = above_la; }
    if (above_b < kb && above_b + gb[j] >= kb) { outb[0] = bin; outb[1] = above_b; outb[2] = above_lb; }
    pre += v[j];
  }
  __syncthreads();
}

// Steps 2-6 for group `g`.  `dyn`: select_dyn_bytes() of 16-byte aligned shared memory; `s_max`,
// `s_inv`: the per-head softmax statistics in shared memory (a block barrier inside orders the
// caller's writes before their first use).  LATE_ARRIVE = false: the last cluster barrier is
// armed before the row list is stored, so that its release does not wait for those stores (nothing
// in the same kernel reads them).  LATE_ARRIVE = true: it is armed after them, behind a fence, so
// that the other CTAs of the cluster may read every global result of this function afterwards.
template <int DT, int THREADS, bool LATE_ARRIVE>
__device__ __forceinline__ void select_body(const SelectArgs& a, uint8_t* dyn, int g, const float* s_max,
                                            const float* s_inv) {
  static_assert(THREADS == 128 || THREADS == 256, "select_body: 128 or 256 threads");
  constexpr int kWarps = THREADS / 32;
  cg::cluster_group cluster = cg::this_cluster();
  uint16_t* keys = reinterpret_cast<uint16_t*>(dyn);                                   // [slice]
  uint32_t* cand = reinterpret_cast<uint32_t*>(dyn + ri_align16((size_t)a.slice * 2)); // [p_pad] (used in CTA 0)
  uint32_t* cand_cnt = cand + a.p_pad;      // size and first row of each candidate, written by its owner
  uint32_t* cand_off = cand_cnt + a.p_pad;
  uint32_t* ranked = cand_off + a.p_pad;    // the same three, in rank order, plus the place in the row list
  uint32_t* rcnt = ranked + a.p_pad;
  uint32_t* roff = rcnt + a.p_pad;
  uint32_t* rstart = roff + a.p_pad;

  __shared__ int hist1[256], hist2a[256], hist2b[256], hsum[256], hsum2[256];
  __shared__ int s_pub[2];          // this CTA's (clusters in top P+E, clusters in top P)
  __shared__ int fk[3], fp[3], lk[3], lp[3];
  __shared__ uint32_t warp_sums[kWarps];
  __shared__ uint64_t warp_sums64[kWarps];
  __shared__ int s_keep, s_rows;

  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = a.C, gs = a.gs;
  const float* sc = a.scores + (int64_t)g * gs * C;
  const int lo = min(C, rank * a.slice), hi = min(C, lo + a.slice), n_loc = hi - lo;

  for (int i = tid; i < 256; i += THREADS) { hist1[i] = 0; hist2a[i] = 0; hist2b[i] = 0; }
  if (tid < 3) { fk[tid] = 0; fp[tid] = 0; lk[tid] = 0; lp[tid] = 0; }
  __syncthreads();

  // ---- 2. distance keys of this CTA's slice, first-level histogram ----
  for (int e = tid * 4; e < n_loc; e += THREADS * 4) {
    const int c = lo + e;
    float dist[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) {
        const float4 s4 = *reinterpret_cast<const float4*>(sc + (int64_t)h * C + c);
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dist[i] += Elem<DT>::round(exp2f((Elem<DT>::round(sv[i]) - s_max[h]) * RI_LOG2E) * s_inv[h]);
      }
    const int4 cnt4 = *reinterpret_cast<const int4*>(a.count + (int64_t)g * C + c);
    const int cv[4] = {cnt4.x, cnt4.y, cnt4.z, cnt4.w};
    uint16_t k4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint16_t b = Elem<DT>::bits(dist[i]);
      if (cv[i] == 0) b = DT == RI_BF16 ? 0xFF7Fu : 0xFBFFu;   // most negative finite value
      k4[i] = ri_ordered_key(b);
      keys[e + i] = k4[i];
      atomicAdd(&hist1[k4[i] >> 8], 1);
    }
  }
  __syncthreads();
  RI_FT(3);
  cluster.sync();
  RI_FT(4);

  // ---- 3a. high byte of the two cuts ----
  const int K = a.P + a.E;
  for (int i = tid; i < 256; i += THREADS) {
    int s = 0;
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) s += cluster.map_shared_rank(hist1, rr)[i];
    hsum[i] = s;
  }
  __syncthreads();
  find_bins<THREADS>(hsum, hist1, K, fk, hsum, hist1, a.P, fp, warp_sums64);
  const int binK = fk[0], binP = fp[0];

  // ---- 3b. low byte ----
  for (int e = tid; e < n_loc; e += THREADS) {
    const uint16_t k = keys[e];
    if ((k >> 8) == binK) atomicAdd(&hist2a[k & 255], 1);
    if ((k >> 8) == binP) atomicAdd(&hist2b[k & 255], 1);
  }
  __syncthreads();
  cluster.sync();
  RI_FT(5);
  for (int i = tid; i < 256; i += THREADS) {
    int sa = 0, sb = 0;
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) {
      sa += cluster.map_shared_rank(hist2a, rr)[i];
      sb += cluster.map_shared_rank(hist2b, rr)[i];
    }
    hsum[i] = sa;
    hsum2[i] = sb;
  }
  __syncthreads();
  find_bins<THREADS>(hsum, hist2a, K - fk[1], lk, hsum2, hist2b, a.P - fp[1], lp, warp_sums64);
  const uint16_t TK = (uint16_t)((binK << 8) | lk[0]), TP = (uint16_t)((binP << 8) | lp[0]);
  const int needK = K - fk[1] - lk[1];      // how many keys equal to TK are taken (cluster-wide)
  const int needP = a.P - fp[1] - lp[1];
  // ties are taken in ascending id, i.e. lower cluster ranks first
  int tieK_base = 0, tieP_base = 0;
  for (int rr = 0; rr < rank; ++rr) {
    tieK_base += cluster.map_shared_rank(hist2a, rr)[lk[0]];
    tieP_base += cluster.map_shared_rank(hist2b, rr)[lp[0]];
  }
  if (tid == 0) {
    const int takenK = min(max(needK - tieK_base, 0), hist2a[lk[0]]);
    const int takenP = min(max(needP - tieP_base, 0), hist2b[lp[0]]);
    s_pub[0] = fk[2] + lk[2] + takenK;     // this CTA's clusters among the top P+E
    s_pub[1] = fp[2] + lp[2] + takenP;     // ... among the top P
  }
  __syncthreads();
  cluster.sync();
  RI_FT(6);
  int est_base = 0, ret_base = 0;
  for (int rr = 0; rr < rank; ++rr) {
    const int* pub = cluster.map_shared_rank(s_pub, rr);
    est_base += pub[0] - pub[1];
    ret_base += pub[1];
  }

  // ---- 4. ordered compaction ----
  uint32_t* cand0 = cluster.map_shared_rank(cand, 0);
  uint32_t* cand_cnt0 = cluster.map_shared_rank(cand_cnt, 0);
  uint32_t* cand_off0 = cluster.map_shared_rank(cand_off, 0);
  for (int e0 = 0; e0 < n_loc; e0 += THREADS * 4) {
    const int e = e0 + tid * 4;
    const bool quad = e < n_loc;            // slices are multiples of 4: a quad is entirely in or out
    // what an estimation entry needs, fetched coalesced up front (the scans below hide the latency)
    float4 s4[kMaxHeads];
    uint2 sz = make_uint2(0u, 0u);
    if (quad) {
#pragma unroll
      for (int h = 0; h < kMaxHeads; ++h)
        if (h < gs) s4[h] = *reinterpret_cast<const float4*>(sc + (int64_t)h * C + lo + e);
      sz = *reinterpret_cast<const uint2*>(a.size_dt + (int64_t)g * C + lo + e);
    }
    uint16_t k4[4];
    uint32_t eq = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      k4[i] = quad ? keys[e + i] : (uint16_t)0;
      if (quad) eq += (k4[i] == TK ? 1u : 0u) | (k4[i] == TP ? 0x10000u : 0u);
    }
    uint32_t eq_total;
    const uint32_t eq_pre = block_scan<THREADS, uint32_t>(eq, warp_sums, eq_total);
    int rkK = tieK_base + (int)(eq_pre & 0xffffu), rkP = tieP_base + (int)(eq_pre >> 16);
    bool isEst[4], isRet[4];
    int rcount[4] = {0, 0, 0, 0}, roffset[4] = {0, 0, 0, 0};
    uint32_t sel = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool inK = quad && (k4[i] > TK || (k4[i] == TK && rkK < needK));
      const bool inP = quad && (k4[i] > TP || (k4[i] == TP && rkP < needP));
      if (quad && k4[i] == TK) ++rkK;
      if (quad && k4[i] == TP) ++rkP;
      isRet[i] = inP;
      isEst[i] = inK && !inP;
      sel += (isEst[i] ? 1u : 0u) | (isRet[i] ? 0x10000u : 0u);
      if (inP) {                            // travels with the candidate: no gather later
        rcount[i] = a.count[(int64_t)g * C + lo + e + i];
        roffset[i] = a.offset[(int64_t)g * (C + 1) + lo + e + i];
      }
    }
    tieK_base += (int)(eq_total & 0xffffu);
    tieP_base += (int)(eq_total >> 16);
    uint32_t sel_total;
    const uint32_t sel_pre = block_scan<THREADS, uint32_t>(sel, warp_sums, sel_total);
    int pe = est_base + (int)(sel_pre & 0xffffu), pr = ret_base + (int)(sel_pre >> 16);
    // retrieval candidates first (shared memory of CTA 0) ...
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (isRet[i]) {
        if (pr < a.P) {
          cand0[pr] = ((uint32_t)k4[i] << 16) | (uint32_t)(0xffff - (lo + e + i));
          cand_cnt0[pr] = (uint32_t)rcount[i];
          cand_off0[pr] = (uint32_t)roffset[i];
        }
        ++pr;
      }
    est_base += (int)(sel_total & 0xffffu);
    ret_base += (int)(sel_total >> 16);
    const bool last_round = e0 + THREADS * 4 >= n_loc;
    if (last_round) cluster_arrive();   // ... so the barrier's release does not wait for the global stores below
    const uint32_t szw[2] = {sz.x, sz.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (isEst[i]) {
        if (pe < a.E) {
          a.est_ids[(int64_t)g * a.e_pad + pe] = lo + e + i;
          a.est_w[(int64_t)g * a.e_pad + pe] = Elem<DT>::from_bits((uint16_t)(szw[i >> 1] >> (16 * (i & 1))));
#pragma unroll
          for (int h = 0; h < kMaxHeads; ++h)
            if (h < gs) a.est_s2[((int64_t)g * kMaxHeads + h) * a.e_pad + pe] = (&s4[h].x)[i] * RI_LOG2E;
          if (a.estimated_ids) a.estimated_ids[(int64_t)g * a.E + pe] = lo + e + i;
        }
        ++pe;
      }
    }
  }
  if (n_loc <= 0) cluster_arrive();     // a CTA with an empty slice never entered the loop
  cluster_wait();
  RI_FT(7);

  // ---- 5. CTA 0: rank the candidates, page budget, place of each kept cluster in the row list ----
  if (rank == 0) {
    for (int i = tid; i < a.P; i += THREADS) {
      const uint32_t mine = cand[i];
      int rk = 0;
      for (int j = 0; j < a.P; ++j) rk += cand[j] > mine;   // distinct values: distinct ranks
      ranked[rk] = mine;
      rcnt[rk] = cand_cnt[i];
      roff[rk] = cand_off[i];
    }
    __syncthreads();
    constexpr int kPer = 1024 / THREADS;    // P <= 1024
    int cnt[kPer], pages[kPer];
    uint32_t psum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      cnt[u] = i < a.P ? (int)rcnt[i] : 0;
      pages[u] = (cnt[u] + a.page - 1) / a.page;
      psum += (uint32_t)pages[u];
    }
    uint32_t total;
    uint32_t before = block_scan<THREADS, uint32_t>(psum, warp_sums, total);
    // pages are non-negative, so the clusters that fit the budget form a prefix of the ranking
    bool fits[kPer];
    uint32_t nfit = 0, rsum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      before += (uint32_t)pages[u];
      fits[u] = tid * kPer + u < a.P && (int)before <= a.buffer_pages;
      nfit += fits[u] ? 1u : 0u;
      rsum += fits[u] ? (uint32_t)cnt[u] : 0u;
    }
    // kept count (<= 1024) in the high 12 bits, kept rows (< 2^20) in the low 20
    uint32_t both_total;
    const uint32_t both_pre = block_scan<THREADS, uint32_t>((nfit << 20) | rsum, warp_sums, both_total);
    uint32_t row_start = both_pre & 0xfffffu;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      if (i < a.P) rstart[i] = row_start;
      row_start += fits[u] ? (uint32_t)cnt[u] : 0u;
    }
    if (tid == 0) { s_keep = (int)(both_total >> 20); s_rows = (int)(both_total & 0xfffffu); }
    __syncthreads();
  }
  cluster.sync();
  RI_FT(8);

  // ---- 6. all CTAs expand the kept clusters into row indices ----
  // Lane l of a warp fetches the descriptor of the warp's l-th cluster from CTA 0.
  const int keep = *cluster.map_shared_rank(&s_keep, 0);
  constexpr int kWarpsTotal = kSelectCluster * kWarps;
  static_assert(kWarpsTotal * 32 >= 1024, "one descriptor per lane must cover P <= 1024");
  const int my_i = rank * kWarps + warp + kWarpsTotal * lane;
  int d_off = 0, d_cnt = 0, d_start = 0;
  if (my_i < keep) {
    d_off = (int)cluster.map_shared_rank(roff, 0)[my_i];
    d_cnt = (int)cluster.map_shared_rank(rcnt, 0)[my_i];
    d_start = (int)cluster.map_shared_rank(rstart, 0)[my_i];
  }
  if (!LATE_ARRIVE) cluster_arrive();
  const int n_mine = (keep - (rank * kWarps + warp) + kWarpsTotal - 1) / kWarpsTotal;
  for (int l = 0; l < n_mine; ++l) {
    const int off = __shfl_sync(0xffffffffu, d_off, l), cnt = __shfl_sync(0xffffffffu, d_cnt, l);
    const int start = __shfl_sync(0xffffffffu, d_start, l);
    for (int j = lane; j < cnt; j += 32)
      if (start + j < a.max_rows) a.rows[(int64_t)g * a.max_rows + start + j] = off + j;
  }
  for (int e = tid * 4; e < n_loc; e += THREADS * 4) {   // the 16-bit distance keys (a view for tests)
    uint2 kw;
    kw.x = (uint32_t)keys[e] | ((uint32_t)keys[e + 1] << 16);
    kw.y = (uint32_t)keys[e + 2] | ((uint32_t)keys[e + 3] << 16);
    *reinterpret_cast<uint2*>(a.dist_keys + (int64_t)g * C + lo + e) = kw;
  }
  if (rank == 0) {
    if (tid == 0) {
      a.n_exact[g] = s_rows;
      if (a.retrieved_kept) a.retrieved_kept[g] = s_keep;
    }
    if (a.retrieved_ids)
      for (int i = tid; i < a.P; i += THREADS) a.retrieved_ids[(int64_t)g * a.P + i] = 0xffff - (int)(ranked[i] & 0xffffu);
  }
  if (LATE_ARRIVE) {
    __threadfence();
    cluster_arrive();
  }
  cluster_wait();   // CTA 0's shared memory must outlive the remote reads above
}

}  // namespace ri_wave
