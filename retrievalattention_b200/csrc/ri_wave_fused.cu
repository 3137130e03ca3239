// The whole decode step of one layer in ONE kernel: an 8-CTA thread-block cluster per group runs
//   phase 1  scan    s = alpha * q.C^T over the group's centroids (each CTA one slice, streamed
//                    through the lane-private cp.async ring), per-CTA softmax partials exchanged
//                    through distributed shared memory;
//   phase 2  select  the selection of ri_wave_select.cuh reorganised for scores that never leave
//                    shared memory (select_in_cluster below);
//   phase 3  attend  the shared attention body (ri_wave_attend.cuh) over the group's estimation
//                    and exact rows.
// Groups are independent, so nothing crosses a cluster: the two kernel boundaries of the staged
// path (drain, launch, ramp-up, and the scores' trip through the per-tile partials) disappear, and
// clusters drift apart in time so that one group's selection overlaps another group's streaming.
// Reference path: cache_hub/retroinfer_cache.py:549-697 (compute).
#include "ri_wave_attend.cuh"
#include "ri_wave_select.cuh"

namespace ri_wave {
namespace {

constexpr int kFusedThreads = 128;
constexpr int kKeysPerThread = 8;                                   // a CTA's slice holds at most 1024 centroids
constexpr int kMaxSlice = kFusedThreads * kKeysPerThread;
constexpr int kScoreStride = kMaxSlice + 8;                          // floats per head in shared memory (bank spread)
constexpr int kScanStages = 2;                                       // the third ring stage holds the scores instead
constexpr int kScoreOffset = 4 * kScanStages * kStageBytes;          // 64 KB
static_assert(kAttendCluster == kSelectCluster, "one cluster shape for all phases");

struct FusedArgs {
  SelectArgs sel;
  AttendArgs att;
  const uint4* cent;
  float* scores;     // global copy of the scores (a view for tests), written only when `views`
  float alpha;
  int views;         // also fill the global lists and views (tests, callers that asked for the id outputs)
  // this step's key/value rows [G, 128] to append to the steady zone (row static_len - 1) first; null: already there
  const uint4* new_k;
  const uint4* new_v;
  uint4* steady_k_w;
  uint4* steady_v_w;
  int persist_off;   // byte offset, behind the ring and the scores, of the lists that outlive the selection
  int cap;           // estimation entries a CTA can keep in shared memory (multiple of 16)
};

// Phase 1 for this CTA's slice [lo, hi) of group g: scores into shared memory (s_sc[h * kScoreStride + e]),
// and the slice's per-head (max, sum of exponentials) of the rounded scores into part_m/part_s.
template <int DT>
__device__ __forceinline__ void scan_slice(const FusedArgs& f, int g, int lo, int hi, uint8_t* ring, float* s_sc,
                                           float* part_m, float* part_s) {
  __shared__ float w_m[4][kMaxHeads], w_s[4][kMaxHeads];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int C = f.sel.C, gs = f.sel.gs;
  // stage-major ring as in the attend phase; only stages 0 and 1 are used here
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring) + warp * kStageBytes + lane * 16;
  const uint8_t* my_ring_ptr = ring + warp * kStageBytes + lane * 16;
  constexpr int kStageStride = 4 * kStageBytes;
  const int n_steps = (hi - lo + 31) / 32;            // 32 centroids per warp step

  // piece j*4+kk of a stage: row j*8+r of the step, bytes 16*(t+4kk) — the fragment layout of the scan kernel
  auto issue = [&](int step, int stage) {
    const uint32_t dst = my_ring + stage * kStageStride;
    const int base = lo + step * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = min(base + j * 8 + r, hi - 1);   // rows past the slice are masked below
      const uint4* p = f.cent + ((int64_t)g * C + row) * 16 + t;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) cp_async16(dst + (j * 4 + kk) * 512, p + kk * 4);
    }
  };

  int s_issue = warp;                                  // a warp takes steps warp, warp+4, ...
#pragma unroll
  for (int st = 0; st < kScanStages; ++st) {
    if (s_issue < n_steps) { issue(s_issue, st); s_issue += 4; }
    cp_async_commit();
  }
  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < gs ? ri_ldg16(f.att.q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

  float m_run = -INFINITY, s_run = 0.f;   // softmax statistics of head r over this warp's centroids
  int stage = 0;
#pragma unroll 1
  for (int step = warp; step < n_steps; step += 4) {
    cp_async_wait<kScanStages - 1>();
    const uint8_t* src = my_ring_ptr + stage * kStageStride;
    const int base = lo + step * 32;
    float rv[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint4 kb = *reinterpret_cast<const uint4*>(src + (j * 4 + kk) * 512);
        Elem<DT>::mma16816(acc, qa[kk].x, 0u, qa[kk].y, 0u, kb.x, kb.y);
        Elem<DT>::mma16816(acc, qa[kk].z, 0u, qa[kk].w, 0u, kb.z, kb.w);
      }
      const int c0 = base + j * 8 + 2 * t;
      const float v0 = f.alpha * acc[0], v1 = f.alpha * acc[1];
      const bool ok = r < gs && c0 < hi;               // slices are multiples of 8: a tile is entirely in or out
      if (ok) {
        *reinterpret_cast<float2*>(s_sc + r * kScoreStride + (c0 - lo)) = make_float2(v0, v1);
        if (f.views) *reinterpret_cast<float2*>(f.scores + ((int64_t)g * gs + r) * C + c0) = make_float2(v0, v1);
      }
      rv[j][0] = ok ? Elem<DT>::round(v0) : -INFINITY;
      rv[j][1] = ok ? Elem<DT>::round(v1) : -INFINITY;
    }
    if (s_issue < n_steps) { issue(s_issue, stage); s_issue += 4; }
    cp_async_commit();
    stage ^= 1;

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
  cp_async_wait<0>();
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 1);
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 2);
  if (t == 0) { w_m[warp][r] = m_run; w_s[warp][r] = s_run; }
  __syncthreads();
  if (tid < kMaxHeads) {
    const int h = tid;
    const float M = fmaxf(fmaxf(w_m[0][h], w_m[1][h]), fmaxf(w_m[2][h], w_m[3][h]));
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (w_m[w][h] > -INFINITY) S += w_s[w][h] * exp2f((w_m[w][h] - M) * RI_LOG2E);
    part_m[h] = M;
    part_s[h] = S;
  }
}

// Phase 2.  The arithmetic and the tie rules are those of the selection body in ri_wave_select.cuh;
// the organisation differs: a thread keeps its eight keys in registers, the scores come from shared
// memory, the positions in the compacted lists follow from ONE packed block scan plus closed forms
// (the counts of the lower-ranked CTAs are summed from their histograms, ties are taken in id
// order, so "ties taken before me" = min(ties before me, ties to take)), the P retrieval
// candidates stay with their owners until every CTA pulls a copy, and every CTA ranks them and applies the
// page budget on its own copy.  Four cluster barriers instead of six.
// What the attend phase needs stays in shared memory (`ll`): this CTA's own estimation entries, the kept
// clusters' row ranges and this CTA's share of the exact steps (balanced against the estimation work
// every CTA has).  Returns true when that form is usable; false (some CTA holds more estimation entries
// than its list takes) after writing the global lists that the stand-alone attend body reads instead.
template <int DT>
__device__ __forceinline__ bool select_in_cluster(const FusedArgs& f, int g, int rank, int lo, int n_loc, uint8_t* dyn,
                                                  const float* s_sc, const float* s_max, const float* s_inv,
                                                  int static_len, LocalLists& ll) {
  constexpr int T = kFusedThreads;
  const SelectArgs& a = f.sel;
  cg::cluster_group cluster = cg::this_cluster();
  uint4* own = reinterpret_cast<uint4*>(dyn);           // [p_pad] this CTA's retrieval candidates, in id order:
                                                       //   key<<16 | (0xffff - id), cluster size, first row, unused
  uint32_t* cand = reinterpret_cast<uint32_t*>(own + a.p_pad);   // [p_pad] all P candidates of the group (pulled)
  uint32_t* cand_cnt = cand + a.p_pad;
  uint32_t* cand_off = cand_cnt + a.p_pad;
  uint32_t* ranked = cand_off + a.p_pad;               // the same three in rank order, plus the place in the row list
  uint32_t* rcnt = ranked + a.p_pad;
  uint32_t* roff = rcnt + a.p_pad;
  uint32_t* rstart = roff + a.p_pad;

  // lists that outlive this phase (behind the ring and the scores)
  uint32_t* dstart = reinterpret_cast<uint32_t*>(dyn + f.persist_off);   // [p_pad + 4]
  uint32_t* doff = dstart + a.p_pad + 4;                                 // [p_pad]
  float* est_wt = reinterpret_cast<float*>(doff + a.p_pad);              // [cap]
  float* est_sc = est_wt + f.cap;                                        // [gs][cap]
  uint16_t* est_idx = reinterpret_cast<uint16_t*>(est_sc + (size_t)a.gs * f.cap);   // [cap]

  // histograms of 256 bins, two 16-bit counters per word (bin 2w low, bin 2w+1 high; a slice holds <= 1024 keys)
  __shared__ uint32_t hist1[128], hist2a[128], hist2b[128];
  __shared__ __align__(16) int s_cnt[4];          // this CTA's keys above the K cut | above the P cut | on the K cut | on the P cut
  __shared__ int s_before[4];       // the same four, summed over the CTAs of lower rank
  __shared__ int s_share[4];        // this CTA's exact steps [lo, hi), its estimation entries, whether the lists fit
  __shared__ int s_nret[kSelectCluster], s_nest[kSelectCluster];   // every CTA's candidates / estimation entries
  __shared__ int fk[3], fp[3], lk[3], lp[3];
  __shared__ uint32_t warp_sums[T / 32];
  __shared__ uint64_t warp_sums64[T / 32];
  __shared__ __align__(16) int s_keep, s_rows;
  __shared__ __align__(8) int s_pub[2];   // this CTA's retrieval candidates, estimation entries

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = a.C, gs = a.gs;
  if (tid < 128) { hist1[tid] = 0; hist2a[tid] = 0; hist2b[tid] = 0; }
  if (tid < 3) { fk[tid] = 0; fp[tid] = 0; lk[tid] = 0; lp[tid] = 0; }
  __syncthreads();

  // ---- keys of this thread's eight centroids (ids lo + 8*tid ..), first-level histogram ----
  const int e0 = tid * kKeysPerThread;
  const bool live = e0 < n_loc;                  // slices are multiples of 8: all eight or none
  const int64_t gc = (int64_t)g * C + lo + e0;
  uint16_t key[kKeysPerThread];
  int cnt[kKeysPerThread], off[kKeysPerThread];
  uint4 sz = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int i = 0; i < kKeysPerThread; ++i) { key[i] = 0; cnt[i] = 0; off[i] = 0; }
  if (live) {
    const int4 c0 = *reinterpret_cast<const int4*>(a.count + gc), c1 = *reinterpret_cast<const int4*>(a.count + gc + 4);
    cnt[0] = c0.x; cnt[1] = c0.y; cnt[2] = c0.z; cnt[3] = c0.w; cnt[4] = c1.x; cnt[5] = c1.y; cnt[6] = c1.z; cnt[7] = c1.w;
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i) off[i] = a.offset[(int64_t)g * (C + 1) + lo + e0 + i];
    sz = *reinterpret_cast<const uint4*>(a.size_dt + gc);
    float dist[kKeysPerThread];
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i) dist[i] = 0.f;
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) {
        const float4 s0 = *reinterpret_cast<const float4*>(s_sc + h * kScoreStride + e0);
        const float4 s1 = *reinterpret_cast<const float4*>(s_sc + h * kScoreStride + e0 + 4);
        const float sv[kKeysPerThread] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < kKeysPerThread; ++i)
          dist[i] += Elem<DT>::round(exp2f((Elem<DT>::round(sv[i]) - s_max[h]) * RI_LOG2E) * s_inv[h]);
      }
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i) {
      uint16_t b = Elem<DT>::bits(dist[i]);
      if (cnt[i] == 0) b = DT == RI_BF16 ? 0xFF7Fu : 0xFBFFu;   // most negative finite value
      key[i] = ri_ordered_key(b);
      atomicAdd(&hist1[key[i] >> 9], 1u << (16 * ((key[i] >> 8) & 1)));
    }
    if (f.views) {
      uint4 kw;
      kw.x = key[0] | ((uint32_t)key[1] << 16); kw.y = key[2] | ((uint32_t)key[3] << 16);
      kw.z = key[4] | ((uint32_t)key[5] << 16); kw.w = key[6] | ((uint32_t)key[7] << 16);
      *reinterpret_cast<uint4*>(a.dist_keys + gc) = kw;
    }
  }
  __syncthreads();
  RI_FT(3);
  cluster.sync();
  RI_FT(4);

  // ---- high byte of the two cuts ----
  // Thread tid looks after bins 255-2*tid and 254-2*tid, i.e. word 127-tid of the packed histograms:
  // cluster-wide sums straight from the eight CTAs' words into registers, one packed scan to find the bins.
  const int K = a.P + a.E;
  const int my_word = 127 - tid;
  {
    uint32_t w[kSelectCluster];
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) w[rr] = cluster.map_shared_rank(hist1, rr)[my_word];
    uint32_t sum = 0;                       // no carry between the halves: a group holds < 65536 keys
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) sum += w[rr];
    const uint32_t mine = hist1[my_word];
    const int g2[2] = {(int)(sum >> 16), (int)(sum & 0xffffu)}, l2[2] = {(int)(mine >> 16), (int)(mine & 0xffffu)};
    find_bins_regs<T>(g2, l2, K, fk, g2, l2, a.P, fp, warp_sums64);
  }
  const int binK = fk[0], binP = fp[0];

  // ---- low byte ----
  if (live) {
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i) {
      const uint32_t inc = 1u << (16 * (key[i] & 1));
      if ((key[i] >> 8) == binK) atomicAdd(&hist2a[(key[i] & 255) >> 1], inc);
      if ((key[i] >> 8) == binP) atomicAdd(&hist2b[(key[i] & 255) >> 1], inc);
    }
  }
  __syncthreads();
  cluster.sync();
  RI_FT(5);
  {
    uint32_t wa[kSelectCluster], wb[kSelectCluster];
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) {
      wa[rr] = cluster.map_shared_rank(hist2a, rr)[my_word];
      wb[rr] = cluster.map_shared_rank(hist2b, rr)[my_word];
    }
    uint32_t sa = 0, sb = 0;
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) { sa += wa[rr]; sb += wb[rr]; }
    const uint32_t ma = hist2a[my_word], mb = hist2b[my_word];
    const int ga[2] = {(int)(sa >> 16), (int)(sa & 0xffffu)}, la[2] = {(int)(ma >> 16), (int)(ma & 0xffffu)};
    const int gb[2] = {(int)(sb >> 16), (int)(sb & 0xffffu)}, lb[2] = {(int)(mb >> 16), (int)(mb & 0xffffu)};
    find_bins_regs<T>(ga, la, K - fk[1], lk, gb, lb, a.P - fp[1], lp, warp_sums64);
  }
  const int lowK = lk[0], lowP = lp[0];
  RI_FT(14);
  const uint16_t TK = (uint16_t)((binK << 8) | lowK), TP = (uint16_t)((binP << 8) | lowP);
  const int needK = K - fk[1] - lk[1];      // how many keys equal to TK are taken (cluster-wide)
  const int needP = a.P - fp[1] - lp[1];

  // keys above the cuts, and keys on them, in the CTAs of lower rank (they hold the lower ids): every CTA
  // publishes its own four counts, eight lanes fetch them, the warp adds up those of lower rank
  if (tid == 0) {
    s_cnt[0] = fk[2] + lk[2];
    s_cnt[1] = fp[2] + lp[2];
    s_cnt[2] = (int)((hist2a[lowK >> 1] >> (16 * (lowK & 1))) & 0xffffu);
    s_cnt[3] = (int)((hist2b[lowP >> 1] >> (16 * (lowP & 1))) & 0xffffu);
  }
  __syncthreads();
  cluster.sync();
  if (warp == 0) {
    int4 c = make_int4(0, 0, 0, 0);
    if (lane < rank) c = *reinterpret_cast<const int4*>(cluster.map_shared_rank(s_cnt, lane));   // rank <= 7
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      c.x += __shfl_xor_sync(0xffffffffu, c.x, o); c.y += __shfl_xor_sync(0xffffffffu, c.y, o);
      c.z += __shfl_xor_sync(0xffffffffu, c.z, o); c.w += __shfl_xor_sync(0xffffffffu, c.w, o);
    }
    if (lane == 0) { s_before[0] = c.x; s_before[1] = c.y; s_before[2] = c.z; s_before[3] = c.w; }
  }
  __syncthreads();
  RI_FT(15);
  const int tieK_before = s_before[2], tieP_before = s_before[3];
  const int inK_before = s_before[0] + min(needK, tieK_before);
  const int inP_before = s_before[1] + min(needP, tieP_before);
  const int remK = max(needK - tieK_before, 0), remP = max(needP - tieP_before, 0);   // ties this CTA and later ones take

  // ---- ordered compaction ----
  uint64_t c4 = 0;     // 16-bit counters: above K cut | on K cut | above P cut | on P cut
  if (live) {
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i)
      c4 += (key[i] > TK ? 1ull : 0ull) | (key[i] == TK ? 1ull << 16 : 0ull) | (key[i] > TP ? 1ull << 32 : 0ull) |
            (key[i] == TP ? 1ull << 48 : 0ull);
  }
  uint64_t c4_total;
  const uint64_t pre = block_scan<T, uint64_t>(c4, warp_sums64, c4_total);
  int gtK = (int)(pre & 0xffffu), eqK = (int)((pre >> 16) & 0xffffu);
  int gtP = (int)((pre >> 32) & 0xffffu), eqP = (int)(pre >> 48);
  RI_FT(6);
  uint32_t est_mask = 0;     // which of the eight are estimation entries, and their positions in this CTA's list
  int est_lp[kKeysPerThread];
  if (live) {
    const uint32_t szw[4] = {sz.x, sz.y, sz.z, sz.w};
#pragma unroll
    for (int i = 0; i < kKeysPerThread; ++i) {
      const bool inK = key[i] > TK || (key[i] == TK && eqK < remK);
      const bool inP = key[i] > TP || (key[i] == TP && eqP < remP);
      const int posK = gtK + min(eqK, remK), posP = gtP + min(eqP, remP);   // taken keys before this one, in this CTA
      est_lp[i] = posK - posP;
      if (inP) {
        own[posP] = make_uint4(((uint32_t)key[i] << 16) | (uint32_t)(0xffff - (lo + e0 + i)), (uint32_t)cnt[i],
                               (uint32_t)off[i], 0u);
      } else if (inK) {
        est_mask |= 1u << i;
        const int lp = est_lp[i];
        if (lp < f.cap) {
          est_idx[lp] = (uint16_t)(e0 + i);
          est_wt[lp] = Elem<DT>::from_bits((uint16_t)(szw[i >> 1] >> (16 * (i & 1))));
#pragma unroll
          for (int h = 0; h < kMaxHeads; ++h)
            if (h < gs) est_sc[h * f.cap + lp] = s_sc[h * kScoreStride + e0 + i] * RI_LOG2E;
        }
      }
      gtK += key[i] > TK; eqK += key[i] == TK; gtP += key[i] > TP; eqP += key[i] == TP;
    }
  }
  if (tid == 0) {
    const int n_ret = (int)((c4_total >> 32) & 0xffffu) + min((int)(c4_total >> 48), remP);
    const int n_in = (int)(c4_total & 0xffffu) + min((int)((c4_total >> 16) & 0xffffu), remK);
    s_pub[0] = n_ret;
    s_pub[1] = n_in - n_ret;
  }
  __syncthreads();
  cluster.sync();       // every CTA's candidate list, estimation list and counts are complete
  RI_FT(7);

  // ---- every CTA: pull the P candidates of the group, rank them, page budget, place in the row list ----
  if (tid < kSelectCluster) {
    const int2 pub = *reinterpret_cast<const int2*>(cluster.map_shared_rank(s_pub, tid));
    s_nret[tid] = pub.x;
    s_nest[tid] = pub.y;
  }
  __syncthreads();
  {
    int nret[kSelectCluster];
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) nret[rr] = s_nret[rr];
    for (int i = tid; i < a.p_pad; i += T) {
      int src = 0, j = i, lim = nret[0];     // candidate i of the group = candidate j of CTA src, which holds lim
#pragma unroll
      for (int rr = 0; rr < kSelectCluster - 1; ++rr)
        if (src == rr && j >= nret[rr]) { j -= nret[rr]; ++src; lim = nret[rr + 1]; }
      uint4 v = make_uint4(0u, 0u, 0u, 0u);  // padding compares below every real candidate
      if (i < a.P && j < lim) v = cluster.map_shared_rank(own, src)[j];
      cand[i] = v.x; cand_cnt[i] = v.y; cand_off[i] = v.z;
    }
  }
  __syncthreads();
  cluster_arrive();     // this CTA's remote reads of the other CTAs' `own` lists are over (awaited before the ring is reused)
  RI_FT(16);
  // Page budget (wave_buffer_cpu.cpp:207-216): the clusters are taken in rank order while their pages fit.
  // When ALL P candidates fit — the usual case — the order plays no part in what is attended, so unless the
  // caller wants the ranked ids the ranking is skipped and the rows are laid out in cluster-id order.
  constexpr int kPer = 1024 / T;    // P <= 1024
  int pc[kPer], pages[kPer];
  uint32_t psum, total, before;
  auto count_pages = [&](const uint32_t* sizes) {
    psum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      pc[u] = i < a.P ? (int)sizes[i] : 0;
      pages[u] = (pc[u] + a.page - 1) / a.page;
      psum += (uint32_t)pages[u];
    }
    before = block_scan<T, uint32_t>(psum, warp_sums, total);
  };
  count_pages(cand_cnt);
  if (f.views || (int)total > a.buffer_pages) {
    {
      // rank = number of larger candidates (distinct values: distinct ranks); four lanes share a candidate,
      // each counting over a quarter of the list
      const int quads = a.p_pad / 4, seg = tid & 3;
      const int q_lo = quads * seg / 4, q_hi = quads * (seg + 1) / 4;
      for (int base = 0; base < a.P; base += T / 4) {      // uniform trip count: the shuffles below need whole warps
        const int i = base + (tid >> 2);
        const uint32_t mine = i < a.P ? cand[i] : 0xffffffffu;
        int r0 = 0, r1 = 0;
        int q = q_lo;
        for (; q + 2 <= q_hi; q += 2) {
          const uint4 c0 = *reinterpret_cast<const uint4*>(cand + 4 * q), c1 = *reinterpret_cast<const uint4*>(cand + 4 * q + 4);
          r0 += (c0.x > mine) + (c0.y > mine) + (c0.z > mine) + (c0.w > mine);
          r1 += (c1.x > mine) + (c1.y > mine) + (c1.z > mine) + (c1.w > mine);
        }
        if (q < q_hi) {
          const uint4 c = *reinterpret_cast<const uint4*>(cand + 4 * q);
          r0 += (c.x > mine) + (c.y > mine) + (c.z > mine) + (c.w > mine);
        }
        int rk = r0 + r1;
        rk += __shfl_xor_sync(0xffffffffu, rk, 1);
        rk += __shfl_xor_sync(0xffffffffu, rk, 2);
        if (seg == 0 && i < a.P) {
          ranked[rk] = mine;
          rcnt[rk] = cand_cnt[i];
          roff[rk] = cand_off[i];
        }
      }
    }
    __syncthreads();
    count_pages(rcnt);
  } else {
    rcnt = cand_cnt;      // id order serves as the order of the row list
    roff = cand_off;
  }
  RI_FT(17);
  {
    // pages are non-negative, so the clusters that fit the budget form a prefix of the order
    bool fits[kPer];
    uint32_t nfit = 0, rsum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      before += (uint32_t)pages[u];
      fits[u] = tid * kPer + u < a.P && (int)before <= a.buffer_pages;
      nfit += fits[u] ? 1u : 0u;
      rsum += fits[u] ? (uint32_t)pc[u] : 0u;
    }
    // kept count (<= 1024) in the high 12 bits, kept rows (< 2^20) in the low 20
    uint32_t both_total;
    const uint32_t both_pre = block_scan<T, uint32_t>((nfit << 20) | rsum, warp_sums, both_total);
    uint32_t row_start = both_pre & 0xfffffu;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      if (i < a.P) rstart[i] = row_start;
      row_start += fits[u] ? (uint32_t)pc[u] : 0u;
    }
    if (tid == 0) { s_keep = (int)(both_total >> 20); s_rows = (int)(both_total & 0xfffffu); }
    __syncthreads();
  }
  RI_FT(8);
  const int keep = s_keep, rows_kept = s_rows;

  // ---- what the attend phase reads: kept clusters' row ranges, and this CTA's share of the exact steps ----
  for (int i = tid; i <= keep; i += T) {
    dstart[i] = i < keep ? rstart[i] : (uint32_t)rows_kept;
    if (i < keep) doff[i] = roff[i];
  }
  // Share out the exact steps: level the cost units (kCostEst per estimation step a CTA already has,
  // kCostExact per exact step to hand out) so that sum_c max(0, level - e_c) >= X, then cut the exact steps at the
  // running sums.  Lane c of warp 0 stands for CTA c.  Two rounds of levelling (CTAs above the first level drop
  // out of the second) are enough in practice; whatever imbalance is left only costs time.
  if (warp == 0) {
    const int xs_total = (static_len + rows_kept + 15) / 16;
    const int X = f.att.cost_exact * xs_total;
    const int n_e = lane < kSelectCluster ? s_nest[lane] : 0;
    const int e_u = f.att.cost_est * ((n_e + 15) / 16);
    bool act = lane < kSelectCluster;
    int level = 0;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      int sum_e = act ? e_u : 0;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum_e += __shfl_xor_sync(0xffffffffu, sum_e, o);   // lanes 0..7 hold the sum
      sum_e = __shfl_sync(0xffffffffu, sum_e, 0);
      const int n = __popc(__ballot_sync(0xffffffffu, act));                             // >= 1: the least loaded CTA stays
      level = (int)__fdividef((float)(X + sum_e + n - 1), (float)n);
      act = act && e_u <= level;
    }
    const int x_u = lane < kSelectCluster ? max(0, level - e_u) : 0;
    int incl = x_u;
#pragma unroll
    for (int o = 1; o < kSelectCluster; o <<= 1) {
      const int nb = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += nb;
    }
    const int b_lo = min(xs_total, (incl - x_u + f.att.cost_exact - 1) / f.att.cost_exact);
    const int b_hi = lane == kSelectCluster - 1 ? xs_total : min(xs_total, (incl + f.att.cost_exact - 1) / f.att.cost_exact);
    int est_max = n_e;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) est_max = max(est_max, __shfl_xor_sync(0xffffffffu, est_max, o));
    if (lane == rank) { s_share[0] = b_lo; s_share[1] = b_hi; s_share[2] = n_e; s_share[3] = est_max <= f.cap; }
  }
  __syncthreads();
  const bool local = s_share[3] != 0;
  ll.est_idx = est_idx; ll.est_wt = est_wt; ll.est_sc = est_sc;
  ll.cap = f.cap; ll.n_est = s_share[2]; ll.slice_lo = lo;
  ll.dstart = dstart; ll.doff = doff; ll.keep = keep; ll.n_rows = rows_kept;
  ll.x_lo = s_share[0]; ll.x_hi = s_share[1];

  RI_FT(18);
  // ---- the global lists: for callers that asked for them, and for the attend body when the lists above
  //      do not fit ----
  if (f.views || !local) {
    int est_base = inK_before - inP_before;   // estimation entries in the CTAs of lower rank
    if (est_mask) {
      const uint32_t szw[4] = {sz.x, sz.y, sz.z, sz.w};
#pragma unroll
      for (int i = 0; i < kKeysPerThread; ++i)
        if (est_mask >> i & 1u) {
          const int pe = est_base + est_lp[i];
          if (pe < a.E) {
            a.est_ids[(int64_t)g * a.e_pad + pe] = lo + e0 + i;
            a.est_w[(int64_t)g * a.e_pad + pe] = Elem<DT>::from_bits((uint16_t)(szw[i >> 1] >> (16 * (i & 1))));
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h)
              if (h < gs) a.est_s2[((int64_t)g * kMaxHeads + h) * a.e_pad + pe] = s_sc[h * kScoreStride + e0 + i] * RI_LOG2E;
            if (a.estimated_ids) a.estimated_ids[(int64_t)g * a.E + pe] = lo + e0 + i;
          }
        }
    }
    constexpr int kWarpsTotal = kSelectCluster * (T / 32);   // the cluster's 32 warps share the kept clusters out
    for (int i = rank * (T / 32) + warp; i < keep; i += kWarpsTotal) {
      const int o = (int)roff[i], n = (int)rcnt[i], start = (int)rstart[i];
      for (int j = lane; j < n; j += 32)
        if (start + j < a.max_rows) a.rows[(int64_t)g * a.max_rows + start + j] = o + j;
    }
    if (rank == 0) {
      if (tid == 0) {
        a.n_exact[g] = rows_kept;
        if (a.retrieved_kept) a.retrieved_kept[g] = keep;
      }
      if (a.retrieved_ids)
        for (int i = tid; i < a.P; i += T) a.retrieved_ids[(int64_t)g * a.P + i] = 0xffff - (int)(ranked[i] & 0xffffu);
    }
    __syncthreads();    // the arrays read above lie in a ring slot that a faster warp is about to fill
  }
  cluster_wait();       // every CTA is done reading this CTA's `own` list: the ring may be reused
  if (!local) {         // the global lists are read by the other CTAs of the cluster in the next phase
    __threadfence();
    cluster.sync();
  }
  return local;
}

template <int DT>
__global__ void __cluster_dims__(kSelectCluster, 1, 1) __launch_bounds__(kFusedThreads, kCtasPerSm)
wave_fused_kernel(FusedArgs f) {
  ri_pdl_enter();
  extern __shared__ __align__(16) uint8_t ring[];
  __shared__ float part_m[kMaxHeads], part_s[kMaxHeads], s_max[kMaxHeads], s_inv[kMaxHeads];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int g = blockIdx.y, tid = threadIdx.x;
  const int C = f.sel.C;
  const int lo = min(C, rank * f.sel.slice), hi = min(C, lo + f.sel.slice);
  float* s_sc = reinterpret_cast<float*>(ring + kScoreOffset);

  int static_len;     // fetched now (not where the compiler would sink the load to: the middle of phase 2)
  asm volatile("ld.global.b32 %0, [%1];" : "=r"(static_len) : "l"(f.att.static_len));

  // the new token's rows go into the steady zone now; the attend phase reads them several cluster barriers later
  if (f.new_k != nullptr && rank == 0 && tid < 32 && static_len >= 1 && static_len <= f.att.steady_stride) {
    const int64_t dst = ((int64_t)g * f.att.steady_stride + static_len - 1) * 16 + (tid & 15);
    if (tid < 16) f.steady_k_w[dst] = f.new_k[(int64_t)g * 16 + tid];
    else f.steady_v_w[dst] = f.new_v[(int64_t)g * 16 + (tid & 15)];
  }

  // ---- phase 1: scores of this CTA's slice ----
  RI_FT(0);
  scan_slice<DT>(f, g, lo, hi, ring, s_sc, part_m, part_s);
  RI_FT(1);
  cluster.sync();     // the partials of all slices are published
  if (tid < f.sel.gs) {
    float M = -INFINITY, S = 0.f;
#pragma unroll
    for (int rr = 0; rr < kSelectCluster; ++rr) {
      const float m = cluster.map_shared_rank(part_m, rr)[tid], sv = cluster.map_shared_rank(part_s, rr)[tid];
      const float Mn = fmaxf(M, m);
      if (Mn > -INFINITY) S = S * exp2f((M - Mn) * RI_LOG2E) + sv * exp2f((m - Mn) * RI_LOG2E);
      M = Mn;
    }
    s_max[tid] = M;
    s_inv[tid] = 1.0f / S;
  }

  // ---- phase 2: selection (its arrays live in the idle ring stages) ----
  RI_FT(2);
  LocalLists ll;
  const bool local = select_in_cluster<DT>(f, g, rank, lo, hi - lo, ring, s_sc, s_max, s_inv, static_len, ll);
  RI_FT(9);

  // ---- phase 3: attention over the estimation and exact rows selected above ----
  if (local) attend_group<DT, true>(f.att, g, rank, ring, &ll);
  else attend_group<DT, false>(f.att, g, rank, ring);
  RI_FT(13);
}

// After the decode kernel of the same stream: raise this rank's flag on every rank, then wait (bounded) until
// every rank's flag here holds this step's epoch.  Thread r looks after rank r.
__global__ void gather_signal_wait_kernel(uint32_t* const* flag_slots, const uint32_t* flags, const uint32_t* epoch,
                                          int32_t* error, int n_ranks, long long limit_ns) {
  ri_pdl_enter();
  const int r = threadIdx.x;
  if (r >= n_ranks) return;
  const uint32_t expected = *epoch;
  // the decode kernel has completed (stream order), so its stores to the other GPUs happen before this fence,
  // and the fence orders them before the flag at system scope
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag_slots[r]), "r"(expected) : "memory");
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  long long spins = 0;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
    if ((int32_t)(v - expected) >= 0) break;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if ((long long)(now - t0) > limit_ns || ++spins > (1ll << 26)) { *error = 1; break; }   // give up: time or count
    __nanosleep(64);
  }
}

// Shared memory one CTA may use when two of them share an SM, minus the kernel's static part.
template <int DT>
int dynamic_budget(int* out) {
  static int cached[64] = {0};
  int dev = 0;
  RI_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || cached[dev] == 0) {
    int per_sm = 0, reserved = 0, optin = 0;
    RI_CUDA_OK(cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
    RI_CUDA_OK(cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev));
    RI_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    RI_CUDA_OK(cudaFuncGetAttributes(&fa, wave_fused_kernel<DT>));
    int budget = per_sm / kCtasPerSm - reserved - (int)fa.sharedSizeBytes;
    if (budget > optin - (int)fa.sharedSizeBytes) budget = optin - (int)fa.sharedSizeBytes;
    budget &= ~15;
    if (dev < 0 || dev >= 64) { *out = budget; return RI_OK; }
    cached[dev] = budget;
  }
  *out = cached[dev];
  return RI_OK;
}

template <int DT>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather) {
  FusedArgs f;
  int rc = fill_select_args(p, L, f.sel);
  if (rc != RI_OK) return rc;
  fill_attend_args(p, L, nullptr, f.att);
  f.cent = static_cast<const uint4*>(p.d_centroids);
  f.scores = reinterpret_cast<float*>(static_cast<uint8_t*>(p.d_scratch) + L.scores);
  f.alpha = 0.08838834764831845f;
  f.views = p.d_retrieved_ids != nullptr;
  f.new_k = static_cast<const uint4*>(p.d_new_keys);
  f.new_v = static_cast<const uint4*>(p.d_new_values);
  f.steady_k_w = static_cast<uint4*>(const_cast<void*>(p.d_steady_keys));
  f.steady_v_w = static_cast<uint4*>(const_cast<void*>(p.d_steady_values));
  if (gather) {
    f.att.copies = reinterpret_cast<uint16_t* const*>(gather->d_out_slots);
    f.att.n_copies = gather->n_ranks;

  }
  RI_REQUIRE(fused_supported(p), "the single-kernel path needs n_centroids <= %d", kMaxSlice * kSelectCluster);
  RI_REQUIRE((size_t)f.sel.p_pad * 44 <= (size_t)kScoreOffset, "nprobe=%d too large", p.nprobe);
  // dynamic shared memory: [ring | scores (over ring stage 2 and beyond)] [kept-cluster ranges] [estimation lists]
  int budget = 0;
  if ((rc = dynamic_budget<DT>(&budget)) != RI_OK) return rc;
  const int scores_end = kScoreOffset + p.group_size * kScoreStride * (int)sizeof(float);
  f.persist_off = (int)ri_align_up(scores_end > kRingBytes ? scores_end : kRingBytes, 16);
  const int ranges = (2 * f.sel.p_pad + 4) * 4;
  const int per_entry = 4 * p.group_size + 4 + 2;
  int cap = (budget - f.persist_off - ranges) / per_entry;
  if (const char* e = getenv("RI_WAVE_LOCAL_CAP")) cap = cap < atoi(e) ? cap : atoi(e);   // tests: force the global lists
  cap = cap < 0 ? 0 : (cap > kMaxSlice ? kMaxSlice : cap) & ~15;
  f.cap = cap;
  const size_t smem = ri_align_up((size_t)f.persist_off + ranges + (size_t)cap * per_entry, 16);
  RI_REQUIRE((int)smem <= budget, "nprobe=%d needs %zu bytes of shared memory per CTA (limit %d)", p.nprobe, smem, budget);
  RI_CUDA_OK(cudaFuncSetAttribute(wave_fused_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RI_CUDA_OK(ri_launch_pdl_id(5, wave_fused_kernel<DT>, dim3(kSelectCluster, p.groups), dim3(kFusedThreads), smem, s, f));
  return RI_OK;
}

}  // namespace

#ifdef RI_FUSED_TRACE
extern "C" int ri_debug_fused_trace(unsigned long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_ftrace, sizeof(unsigned long long) * n);
}
#endif

bool fused_supported(const ri_wave_layer& p) {
  return ((p.n_centroids / 8 + kSelectCluster - 1) / kSelectCluster) * 8 <= kMaxSlice;
}

int launch_fused(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s, gather) : launch<RI_F16>(p, L, s, gather);
}

int launch_gather_wait(const ri_wave_gather& g, cudaStream_t s) {
  const long long limit_ns = (g.wait_limit_us > 0 ? (long long)g.wait_limit_us : 1000000ll) * 1000ll;
  RI_CUDA_OK(ri_launch_pdl_id(6, gather_signal_wait_kernel, dim3(1), dim3(64), 0, s, g.d_flag_slots, g.d_flags, g.d_epoch,
                              g.d_error, g.n_ranks, limit_ns));
  return RI_OK;
}

}  // namespace ri_wave
