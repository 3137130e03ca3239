// The whole decode step of one layer in ONE kernel: a thread-block cluster per group (CL = 4 .. 8 CTAs of
// 256 threads, one CTA per SM; the host picks the largest size with which all clusters are resident at once) runs
//   phase 1  scan    s = alpha * q.C^T over the group's centroids (each CTA one slice, streamed
//                    through the lane-private cp.async ring), per-CTA softmax partials exchanged
//                    through distributed shared memory;
//   phase 2  select  the selection of ri_wave_select.cuh reorganised for scores that never leave
//                    shared memory (select_in_cluster below);
//   phase 3  attend  the shared attention body (ri_wave_attend.cuh) over the group's estimation
//                    and exact rows.
// Groups are independent, so nothing crosses a cluster: the two kernel boundaries of the staged
// path (drain, launch, ramp-up, and the scores' trip through the per-tile partials) disappear.
// One CTA per SM on purpose: with two 128-thread CTAs per SM the hardware placed 256 CTAs on 142 SMs
// as 114 pairs and 28 singles, a single ran its streaming phases 1.6 times faster than a paired CTA,
// and every cluster waited for its slowest member.  The cluster size is chosen so that the grid
// fills the SMs once: 4 CTAs per group from 19 groups up, 8 below.
// Reference path: cache_hub/retroinfer_cache.py:549-697 (compute).
#include "ri_wave_attend.cuh"
#include "ri_wave_select.cuh"

namespace ri_wave {
namespace {

constexpr int kFusedThreads = 256;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr int kFusedMaxCentroids = 8192;                             // per group
constexpr int kScanStages = 2;                                       // the third ring stage holds the scores instead
constexpr int kScoreOffset = kFusedWarps * kScanStages * kStageBytes;   // 128 KB
constexpr int kFusedRingBytes = kFusedWarps * kStages * kStageBytes;    // 192 KB

template <int CL>
struct Geom {
  // centroids a CTA's slice holds at most: 1024 with 8 CTAs per group, 2048 with 4 to 7 (a slice of 8192 / 7 fills
  // 147 of the 256 threads' runs of keys; the rest hold nothing)
  static constexpr int kMaxSlice = CL >= 8 ? kFusedMaxCentroids / 8 : kFusedMaxCentroids / 4;
  static constexpr int kKeys = kMaxSlice / kFusedThreads;            // keys per thread: 8 (CL 4..7) or 4 (CL 8)
  static_assert(CL >= 4 && CL <= 8, "clusters of 4 to 8 CTAs");
  // floats per head in shared memory: four words of padding after every 32 (see score_at), eight more between heads
  static constexpr int kScoreStride = kMaxSlice + kMaxSlice / 8 + 8;
  static_assert(kKeys == 4 || kKeys == 8, "a thread's keys are loaded as one or two 16-byte pieces");
};

// Place of centroid e of the slice in a head's row of scores: a thread of the selection owns a run of 4 or 8
// consecutive centroids, so without the padding its lanes would sit 8 words apart and collide on 4 banks.
__device__ __forceinline__ int score_at(int e) { return e + ((e >> 5) << 2); }

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
  int cap_limit;     // test hook: upper limit on `cap` (< 0: none)
};

// This thread's clusters, fetched before the scan so that their latency is not on the selection's critical path:
// exact sizes, first row of the first of them, sizes in the 16-bit type.
template <int KEYS>
struct ThreadClusters {
  int cnt[KEYS];
  int off0;
  uint32_t szw[KEYS / 2];
};

// Phase 1 for this CTA's slice [lo, hi) of group g: scores into shared memory (s_sc[h * kScoreStride + e]),
// and the slice's per-head (max, sum of exponentials) of the rounded scores into part_m/part_s.
template <int DT, int CL>
__device__ __forceinline__ void scan_slice(const FusedArgs& f, int g, int lo, int hi, uint8_t* ring, float* s_sc,
                                           float* part_m, float* part_s) {
  constexpr int W = kFusedWarps, kScoreStride = Geom<CL>::kScoreStride;
  __shared__ float w_m[W][kMaxHeads], w_s[W][kMaxHeads];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int C = f.sel.C, gs = f.sel.gs;
  // stage-major ring as in the attend phase; only stages 0 and 1 are used here
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring) + warp * kStageBytes + lane * 16;
  const uint8_t* my_ring_ptr = ring + warp * kStageBytes + lane * 16;
  constexpr int kStageStride = W * kStageBytes;
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

  int s_issue = warp;                                  // a warp takes steps warp, warp+W, ...
#pragma unroll
  for (int st = 0; st < kScanStages; ++st) {
    if (s_issue < n_steps) { issue(s_issue, st); s_issue += W; }
    cp_async_commit();
  }
  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < gs ? ri_ldg16(f.att.q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

  float m_run = -INFINITY, s_run = 0.f;   // softmax statistics of head r over this warp's centroids
  int stage = 0;
#pragma unroll 1
  for (int step = warp; step < n_steps; step += W) {
    cp_async_wait<kScanStages - 1>();
    const uint8_t* src = my_ring_ptr + stage * kStageStride;
    const int base = lo + step * 32;
    // the stage goes to registers and is refilled at once (the same lane wrote it and reads it), so that two stages
    // are in flight while this one is worked on
    uint4 kb[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) kb[i] = *reinterpret_cast<const uint4*>(src + i * 512);
    if (s_issue < n_steps) { issue(s_issue, stage); s_issue += W; }
    cp_async_commit();
    stage ^= 1;
    float rv[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        Elem<DT>::mma16816(acc, qa[kk].x, 0u, qa[kk].y, 0u, kb[j * 4 + kk].x, kb[j * 4 + kk].y);
        Elem<DT>::mma16816(acc, qa[kk].z, 0u, qa[kk].w, 0u, kb[j * 4 + kk].z, kb[j * 4 + kk].w);
      }
      const int c0 = base + j * 8 + 2 * t;
      const float v0 = f.alpha * acc[0], v1 = f.alpha * acc[1];
      const bool ok = r < gs && c0 < hi;               // slices are multiples of 8: a tile is entirely in or out
      if (ok) {
        *reinterpret_cast<float2*>(s_sc + r * kScoreStride + score_at(c0 - lo)) = make_float2(v0, v1);
        if (f.views) *reinterpret_cast<float2*>(f.scores + ((int64_t)g * gs + r) * C + c0) = make_float2(v0, v1);
      }
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
  cp_async_wait<0>();
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 1);
  s_run += __shfl_xor_sync(0xffffffffu, s_run, 2);
  if (t == 0) { w_m[warp][r] = m_run; w_s[warp][r] = s_run; }
  __syncthreads();
  if (tid < kMaxHeads) {
    const int h = tid;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) M = fmaxf(M, w_m[w][h]);
    float S = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w)
      if (w_m[w][h] > -INFINITY) S += w_s[w][h] * exp2f((w_m[w][h] - M) * RI_LOG2E);
    part_m[h] = M;
    part_s[h] = S;
  }
}

// Exclusive scan of two 64-bit values per thread at once (one pair of block barriers for both).
template <int THREADS>
__device__ __forceinline__ void block_scan2(uint64_t& a, uint64_t& b, uint64_t (*warp_sums)[2]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t ia = a, ib = b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint64_t na = __shfl_up_sync(0xffffffffu, ia, o), nb = __shfl_up_sync(0xffffffffu, ib, o);
    if (lane >= o) { ia += na; ib += nb; }
  }
  __syncthreads();   // protects warp_sums from its previous use
  if (lane == 31) { warp_sums[warp][0] = ia; warp_sums[warp][1] = ib; }
  __syncthreads();
  uint64_t ba = 0, bb = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w)
    if (w < warp) { ba += warp_sums[w][0]; bb += warp_sums[w][1]; }
  a = ba + ia - a;
  b = bb + ib - b;
}

// Where a cut falls in a histogram of 256 bins scanned from the top (bin 255 = largest keys): the bin, then the
// keys above that bin and the keys in it — cluster-wide, in the CTAs of lower rank, in this CTA.
struct CutBin { int bin, above_g, above_l, above_m, at_g, at_l, at_m; };

__device__ __forceinline__ void note_cut(CutBin* out, int bin, uint64_t pre, uint64_t v, int k) {
  const int ag = (int)(pre & 0xffffu), cg_ = (int)(v & 0xffffu);
  if (ag < k && ag + cg_ >= k) {
    out->bin = bin; out->above_g = ag; out->above_l = (int)((pre >> 16) & 0xffffu); out->above_m = (int)((pre >> 32) & 0xffffu);
    out->at_g = cg_; out->at_l = (int)((v >> 16) & 0xffffu); out->at_m = (int)((v >> 32) & 0xffffu);
  }
}
// Phase 2.  The arithmetic and the tie rules are those of the selection body in ri_wave_select.cuh;
// the organisation differs: a thread keeps its keys in registers, the scores come from shared
// memory, and every histogram is scanned as packed triples (cluster-wide count | count in the CTAs of
// lower rank | count in this CTA), so that one scan per radix level yields the cut AND what this CTA
// needs to place its own entries: how many selected keys, and how many ties on each cut, the CTAs of
// lower rank hold (they hold the lower ids, and ties are taken in id order: "ties taken before me" =
// min(ties before me, ties to take)).  The positions in the compacted lists then follow from ONE more
// packed block scan plus closed forms.  The P retrieval candidates stay with their owners until every
// CTA pulls a copy, and every CTA ranks them and applies the page budget on its own copy.
// Three cluster barriers (two histogram levels, candidates) and one split barrier.
// What the attend phase needs stays in shared memory (`ll`): this CTA's own estimation entries, the kept
// clusters' row ranges and this CTA's share of the exact steps (balanced against the estimation work
// every CTA has).  Returns true when that form is usable; false (some CTA holds more estimation entries
// than its list takes) after writing the global lists that the stand-alone attend body reads instead.
template <int DT, int CL>
__device__ __forceinline__ bool select_in_cluster(const FusedArgs& f, int g, int rank, int lo, int n_loc, uint8_t* dyn,
                                                  const float* s_sc, const float* s_max, const float* s_inv,
                                                  int static_len, const ThreadClusters<Geom<CL>::kKeys>& tc,
                                                  LocalLists& ll) {
  constexpr int T = kFusedThreads, KEYS = Geom<CL>::kKeys, kScoreStride = Geom<CL>::kScoreStride;
  static_assert(T == 256, "one histogram bin per thread");
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

  __shared__ uint32_t hist1[256], hist2a[256], hist2b[256];   // bin 255 = largest keys
  __shared__ CutBin fk, fp, lk, lp;   // high byte of the K and P cuts, then their low bytes
  __shared__ int s_share[4];        // this CTA's exact steps [lo, hi), its estimation entries, whether the lists fit
  __shared__ int s_nret[CL], s_nest[CL];   // every CTA's candidates / estimation entries
  __shared__ uint32_t warp_sums[T / 32];
  __shared__ uint64_t warp_sums64[T / 32];
  __shared__ uint64_t warp_sums2[T / 32][2];
  __shared__ __align__(16) int s_keep, s_rows;
  __shared__ __align__(8) int s_pub[2];   // this CTA's retrieval candidates, estimation entries

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = a.C, gs = a.gs;
  hist1[tid] = 0; hist2a[tid] = 0; hist2b[tid] = 0;
  if (tid == 0) {
    const CutBin z = {0, 0, 0, 0, 0, 0, 0};
    fk = z; fp = z; lk = z; lp = z;
  }
  __syncthreads();

  // ---- keys of this thread's centroids (ids lo + KEYS*tid ..), first-level histogram ----
  const int e0 = tid * KEYS;
  const bool live = e0 < n_loc;                  // slices are multiples of 8: all of a thread's keys or none
  const int64_t gc = (int64_t)g * C + lo + e0;
  uint16_t key[KEYS];
  int cnt[KEYS], off[KEYS];
#pragma unroll
  for (int i = 0; i < KEYS; ++i) { key[i] = 0; cnt[i] = 0; off[i] = 0; }
  if (live) {
    int run = tc.off0;
#pragma unroll
    for (int i = 0; i < KEYS; ++i) { cnt[i] = tc.cnt[i]; off[i] = run; run += cnt[i]; }
    float dist[KEYS];
#pragma unroll
    for (int i = 0; i < KEYS; ++i) dist[i] = 0.f;
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) {
#pragma unroll
        for (int q4 = 0; q4 < KEYS / 4; ++q4) {
          const float4 s4 = *reinterpret_cast<const float4*>(s_sc + h * kScoreStride + score_at(e0 + 4 * q4));
          const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dist[4 * q4 + i] += Elem<DT>::round(exp2f((Elem<DT>::round(sv[i]) - s_max[h]) * RI_LOG2E) * s_inv[h]);
        }
      }
#pragma unroll
    for (int i = 0; i < KEYS; ++i) {
      uint16_t b = Elem<DT>::bits(dist[i]);
      if (cnt[i] == 0) b = DT == RI_BF16 ? 0xFF7Fu : 0xFBFFu;   // most negative finite value
      key[i] = ri_ordered_key(b);
      atomicAdd(&hist1[key[i] >> 8], 1u);
    }
    if (f.views) {
      uint32_t kw[KEYS / 2];
#pragma unroll
      for (int i = 0; i < KEYS / 2; ++i) kw[i] = key[2 * i] | ((uint32_t)key[2 * i + 1] << 16);
      if constexpr (KEYS == 8) *reinterpret_cast<uint4*>(a.dist_keys + gc) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
      else *reinterpret_cast<uint2*>(a.dist_keys + gc) = make_uint2(kw[0], kw[1]);
    }
  }
  __syncthreads();
  RI_FT(3);
  cluster.sync();
  RI_FT(4);

  // ---- high byte of the two cuts: thread tid looks after bin 255 - tid ----
  const int K = a.P + a.E;
  const int my_bin = 255 - tid;
  {
    uint32_t w[CL];
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) w[rr] = cluster.map_shared_rank(hist1, rr)[my_bin];
    uint32_t sum = 0, lower = 0;
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) { sum += w[rr]; lower += rr < rank ? w[rr] : 0u; }
    const uint64_t v = (uint64_t)sum | ((uint64_t)lower << 16) | ((uint64_t)hist1[my_bin] << 32);
    uint64_t total;
    const uint64_t pre = block_scan<T, uint64_t>(v, warp_sums64, total);
    note_cut(&fk, my_bin, pre, v, K);
    note_cut(&fp, my_bin, pre, v, a.P);
    __syncthreads();
  }
  const int binK = fk.bin, binP = fp.bin;

  // ---- low byte ----
  if (live) {
#pragma unroll
    for (int i = 0; i < KEYS; ++i) {
      if ((key[i] >> 8) == binK) atomicAdd(&hist2a[key[i] & 255], 1u);
      if ((key[i] >> 8) == binP) atomicAdd(&hist2b[key[i] & 255], 1u);
    }
  }
  __syncthreads();
  cluster.sync();
  RI_FT(5);
  {
    uint32_t wa[CL], wb[CL];
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) {
      wa[rr] = cluster.map_shared_rank(hist2a, rr)[my_bin];
      wb[rr] = cluster.map_shared_rank(hist2b, rr)[my_bin];
    }
    uint32_t sa = 0, sb = 0, la = 0, lb = 0;
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) {
      sa += wa[rr]; sb += wb[rr];
      la += rr < rank ? wa[rr] : 0u; lb += rr < rank ? wb[rr] : 0u;
    }
    const uint64_t va = (uint64_t)sa | ((uint64_t)la << 16) | ((uint64_t)hist2a[my_bin] << 32);
    const uint64_t vb = (uint64_t)sb | ((uint64_t)lb << 16) | ((uint64_t)hist2b[my_bin] << 32);
    uint64_t pa = va, pb = vb;
    block_scan2<T>(pa, pb, warp_sums2);
    note_cut(&lk, my_bin, pa, va, K - fk.above_g);
    note_cut(&lp, my_bin, pb, vb, a.P - fp.above_g);
    __syncthreads();
  }
  RI_FT(14);
  const uint16_t TK = (uint16_t)((binK << 8) | lk.bin), TP = (uint16_t)((binP << 8) | lp.bin);
  const int needK = K - fk.above_g - lk.above_g;      // how many keys equal to TK are taken (cluster-wide)
  const int needP = a.P - fp.above_g - lp.above_g;
  // the CTAs of lower rank: ties on each cut, and selected keys (those above the cut plus the ties they take)
  const int tieK_before = lk.at_l, tieP_before = lp.at_l;
  const int inK_before = fk.above_l + lk.above_l + min(needK, tieK_before);
  const int inP_before = fp.above_l + lp.above_l + min(needP, tieP_before);
  const int remK = max(needK - tieK_before, 0), remP = max(needP - tieP_before, 0);   // ties this CTA and later ones take

  // ---- ordered compaction ----
  uint64_t c4 = 0;     // 16-bit counters: above K cut | on K cut | above P cut | on P cut
  if (live) {
#pragma unroll
    for (int i = 0; i < KEYS; ++i)
      c4 += (key[i] > TK ? 1ull : 0ull) | (key[i] == TK ? 1ull << 16 : 0ull) | (key[i] > TP ? 1ull << 32 : 0ull) |
            (key[i] == TP ? 1ull << 48 : 0ull);
  }
  uint64_t c4_total;
  const uint64_t pre = block_scan<T, uint64_t>(c4, warp_sums64, c4_total);
  int gtK = (int)(pre & 0xffffu), eqK = (int)((pre >> 16) & 0xffffu);
  int gtP = (int)((pre >> 32) & 0xffffu), eqP = (int)(pre >> 48);
  RI_FT(6);
  uint32_t est_mask = 0;     // which of this thread's keys are estimation entries, and their positions in this CTA's list
  int est_lp[KEYS];
  if (live) {
#pragma unroll
    for (int i = 0; i < KEYS; ++i) {
      const bool inK = key[i] > TK || (key[i] == TK && eqK < remK);
      const bool inP = key[i] > TP || (key[i] == TP && eqP < remP);
      const int posK = gtK + min(eqK, remK), posP = gtP + min(eqP, remP);   // taken keys before this one, in this CTA
      est_lp[i] = posK - posP;
      if (inP) {
        own[posP] = make_uint4(((uint32_t)key[i] << 16) | (uint32_t)(0xffff - (lo + e0 + i)), (uint32_t)cnt[i],
                               (uint32_t)off[i], 0u);
      } else if (inK) {
        est_mask |= 1u << i;
        const int lpos = est_lp[i];
        if (lpos < f.cap) {      // the scores follow below, one entry per thread
          est_idx[lpos] = (uint16_t)(e0 + i);
          est_wt[lpos] = Elem<DT>::from_bits((uint16_t)(tc.szw[i >> 1] >> (16 * (i & 1))));
        }
      }
      gtK += key[i] > TK; eqK += key[i] == TK; gtP += key[i] > TP; eqP += key[i] == TP;
    }
  }
  const int my_ret = (int)((c4_total >> 32) & 0xffffu) + min((int)(c4_total >> 48), remP);
  const int my_est = (int)(c4_total & 0xffffu) + min((int)((c4_total >> 16) & 0xffffu), remK) - my_ret;
  if (tid == 0) {
    s_pub[0] = my_ret;
    s_pub[1] = my_est;
  }
  __syncthreads();
  // log2-domain scores of the estimation entries, entry by entry (uniform work, consecutive stores)
  for (int j = tid; j < min(my_est, f.cap); j += T) {
    const int e = score_at((int)est_idx[j]);
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) est_sc[h * f.cap + j] = s_sc[h * kScoreStride + e] * RI_LOG2E;
  }
  __syncthreads();
  cluster.sync();       // every CTA's candidate list, estimation list and counts are complete
  RI_FT(7);

  // ---- every CTA: pull the P candidates of the group, rank them, page budget, place in the row list ----
  if (tid < CL) {
    const int2 pub = *reinterpret_cast<const int2*>(cluster.map_shared_rank(s_pub, tid));
    s_nret[tid] = pub.x;
    s_nest[tid] = pub.y;
  }
  __syncthreads();
  {
    int nret[CL];
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) nret[rr] = s_nret[rr];
    for (int i = tid; i < a.p_pad; i += T) {
      int src = 0, j = i, lim = nret[0];     // candidate i of the group = candidate j of CTA src, which holds lim
#pragma unroll
      for (int rr = 0; rr < CL - 1; ++rr)
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
  // caller wants the ranked ids the ranking is skipped and the rows are laid out in cluster-id order: one scan.
  constexpr int kPer = 1024 / T;    // P <= 1024
  int pc[kPer], pages[kPer];
  uint32_t before;
  // pages (low half) and rows (high half) of the candidates in id order, one packed scan
  uint64_t pr = 0;
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int i = tid * kPer + u;
    pc[u] = i < a.P ? (int)cand_cnt[i] : 0;
    pages[u] = (pc[u] + a.page - 1) / a.page;
    pr += (uint64_t)(uint32_t)pages[u] | ((uint64_t)(uint32_t)pc[u] << 32);
  }
  uint64_t pr_total;
  const uint64_t pr_pre = block_scan<T, uint64_t>(pr, warp_sums64, pr_total);
  if (!f.views && (int)(uint32_t)pr_total <= a.buffer_pages) {
    // everything fits: id order serves as the order of the row list, each cluster starts at the rows before it
    rcnt = cand_cnt;
    roff = cand_off;
    uint32_t row_start = (uint32_t)(pr_pre >> 32);
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      if (i < a.P) rstart[i] = row_start;
      row_start += (uint32_t)pc[u];
    }
    if (tid == 0) { s_keep = a.P; s_rows = (int)(pr_total >> 32); }
    RI_FT(17);
    __syncthreads();
  } else {
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
    uint32_t psum = 0, total;
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int i = tid * kPer + u;
      pc[u] = i < a.P ? (int)rcnt[i] : 0;
      pages[u] = (pc[u] + a.page - 1) / a.page;
      psum += (uint32_t)pages[u];
    }
    before = block_scan<T, uint32_t>(psum, warp_sums, total);
    RI_FT(17);
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
  // running sums.  Lane c of the last warp stands for CTA c (warp 0 is busy with the loop above for longest).
  // Two rounds of levelling (CTAs above the first level drop out of the second) are enough in practice; whatever
  // imbalance is left only costs time.
  if (warp == T / 32 - 1) {
    const int xs_total = (static_len + rows_kept + 15) / 16;
    const int X = f.att.cost_exact * xs_total;
    const int n_e = lane < CL ? s_nest[lane] : 0;
    const int e_u = f.att.cost_est * ((n_e + 15) / 16);
    bool act = lane < CL;
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
    const int x_u = lane < CL ? max(0, level - e_u) : 0;
    int incl = x_u;
#pragma unroll
    for (int o = 1; o < CL; o <<= 1) {
      const int nb = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += nb;
    }
    const int b_lo = min(xs_total, (incl - x_u + f.att.cost_exact - 1) / f.att.cost_exact);
    const int b_hi = lane == CL - 1 ? xs_total : min(xs_total, (incl + f.att.cost_exact - 1) / f.att.cost_exact);
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
#pragma unroll
      for (int i = 0; i < KEYS; ++i)
        if (est_mask >> i & 1u) {
          const int pe = est_base + est_lp[i];
          if (pe < a.E) {
            a.est_ids[(int64_t)g * a.e_pad + pe] = lo + e0 + i;
            a.est_w[(int64_t)g * a.e_pad + pe] = Elem<DT>::from_bits((uint16_t)(tc.szw[i >> 1] >> (16 * (i & 1))));
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h)
              if (h < gs) a.est_s2[((int64_t)g * kMaxHeads + h) * a.e_pad + pe] = s_sc[h * kScoreStride + score_at(e0 + i)] * RI_LOG2E;
            if (a.estimated_ids) a.estimated_ids[(int64_t)g * a.E + pe] = lo + e0 + i;
          }
        }
    }
    constexpr int kWarpsTotal = CL * (T / 32);   // the cluster's warps share the kept clusters out
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

template <int DT, int CL>
__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(kFusedThreads, 1)
wave_fused_kernel(FusedArgs f) {
  ri_pdl_enter();
  constexpr int KEYS = Geom<CL>::kKeys;
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

  // this thread's clusters (sizes, first row): requested now, needed after the scan
  ThreadClusters<KEYS> tc;
  {
    const int e0 = tid * KEYS;
    const int64_t gc = (int64_t)g * C + lo + e0;
    if (e0 < hi - lo) {
#pragma unroll
      // volatile: issued here, ahead of the scan, whatever the compiler would prefer
      for (int q4 = 0; q4 < KEYS / 4; ++q4)
        asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(tc.cnt[4 * q4]), "=r"(tc.cnt[4 * q4 + 1]), "=r"(tc.cnt[4 * q4 + 2]), "=r"(tc.cnt[4 * q4 + 3])
                     : "l"(f.sel.count + gc + 4 * q4));
      asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(tc.off0) : "l"(f.sel.offset + (int64_t)g * (C + 1) + lo + e0));
      if constexpr (KEYS == 8)
        asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(tc.szw[0]), "=r"(tc.szw[1]), "=r"(tc.szw[2]), "=r"(tc.szw[3]) : "l"(f.sel.size_dt + gc));
      else
        asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(tc.szw[0]), "=r"(tc.szw[1]) : "l"(f.sel.size_dt + gc));
    } else {
#pragma unroll
      for (int i = 0; i < KEYS; ++i) tc.cnt[i] = 0;
#pragma unroll
      for (int i = 0; i < KEYS / 2; ++i) tc.szw[i] = 0u;
      tc.off0 = 0;
    }
  }

  // the new token's rows go into the steady zone now; the attend phase reads them several cluster barriers later
  if (f.new_k != nullptr && rank == 0 && tid < 32 && static_len >= 1 && static_len <= f.att.steady_stride) {
    const int64_t dst = ((int64_t)g * f.att.steady_stride + static_len - 1) * 16 + (tid & 15);
    if (tid < 16) f.steady_k_w[dst] = f.new_k[(int64_t)g * 16 + tid];
    else f.steady_v_w[dst] = f.new_v[(int64_t)g * 16 + (tid & 15)];
  }

  // ---- phase 1: scores of this CTA's slice ----
  RI_FT(0);
  scan_slice<DT, CL>(f, g, lo, hi, ring, s_sc, part_m, part_s);
  RI_FT(1);
  cluster.sync();     // the partials of all slices are published
  if (tid < f.sel.gs) {
    float M = -INFINITY, S = 0.f;
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) {
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
  const bool local = select_in_cluster<DT, CL>(f, g, rank, lo, hi - lo, ring, s_sc, s_max, s_inv, static_len, tc, ll);
  RI_FT(9);

  // ---- phase 3: attention over the estimation and exact rows selected above ----
  if (local) attend_group<DT, true, kFusedWarps, CL>(f.att, g, rank, ring, &ll);
  else attend_group<DT, false, kFusedWarps, CL>(f.att, g, rank, ring);
  RI_FT(13);
}

// After the decode kernel of the same stream: raise this rank's flag on every rank, then wait (bounded) until
// every rank's flag here holds this step's epoch.  Thread r looks after rank r.
__global__ void gather_signal_wait_kernel(uint32_t* const* flag_slots, const uint32_t* flags, const uint32_t* epoch,
                                          int32_t* error, int n_ranks, long long limit_ns, unsigned long long* stamps) {
  ri_pdl_enter();
  const int r = threadIdx.x;
  if (r >= n_ranks) return;
  unsigned long long t_in;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_in));
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
  if (stamps != nullptr) {       // entry | flags raised | last flag seen (the maximum over the threads)
    unsigned long long t_out;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_out));
    if (r == 0) { stamps[0] = t_in; stamps[1] = t0; }
    atomicMax(stamps + 2, t_out);      // the timer only grows, so the latest call's maximum wins
  }
}

// Shared memory the kernel's one CTA per SM may use, minus the kernel's static part; and the SM count.
template <int DT, int CL>
int dynamic_budget(int* out, int* sms_out) {
  static int cached[64] = {0}, cached_sms[64] = {0};
  int dev = 0;
  RI_CUDA_OK(cudaGetDevice(&dev));
  const bool track = dev >= 0 && dev < 64;
  if (!track || cached[dev] == 0) {
    int per_sm = 0, reserved = 0, optin = 0, sms = 0;
    RI_CUDA_OK(cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
    RI_CUDA_OK(cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev));
    RI_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    RI_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaFuncAttributes fa;
    RI_CUDA_OK(cudaFuncGetAttributes(&fa, wave_fused_kernel<DT, CL>));
    int budget = per_sm - reserved - (int)fa.sharedSizeBytes;
    if (budget > optin - (int)fa.sharedSizeBytes) budget = optin - (int)fa.sharedSizeBytes;
    budget &= ~15;
    if (!track) { *out = budget; *sms_out = sms; return RI_OK; }
    cached[dev] = budget;
    cached_sms[dev] = sms;
  }
  *out = cached[dev];
  *sms_out = cached_sms[dev];
  return RI_OK;
}

int g_cap_limit = -1;   // ri_wave_test_local_cap

template <int DT, int CL>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather) {
  FusedArgs f;
  int rc = fill_select_args(p, L, f.sel);
  if (rc != RI_OK) return rc;
  f.sel.slice = ((p.n_centroids / 8 + CL - 1) / CL) * 8;        // centroids per CTA of this kernel's cluster
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
  RI_REQUIRE(fused_supported(p), "the single-kernel path needs n_centroids <= %d", kFusedMaxCentroids);
  RI_REQUIRE((size_t)f.sel.p_pad * 44 <= (size_t)kScoreOffset, "nprobe=%d too large", p.nprobe);
  // dynamic shared memory: [ring | scores (over ring stage 2 and beyond)] [kept-cluster ranges] [estimation lists]
  int budget = 0, sms = 0;
  if ((rc = dynamic_budget<DT, CL>(&budget, &sms)) != RI_OK) return rc;
  const int scores_end = kScoreOffset + p.group_size * Geom<CL>::kScoreStride * (int)sizeof(float);
  f.persist_off = (int)ri_align_up(scores_end > kFusedRingBytes ? scores_end : kFusedRingBytes, 16);
  const int ranges = (2 * f.sel.p_pad + 4) * 4;
  const int per_entry = 4 * p.group_size + 4 + 2;
  int cap = (budget - f.persist_off - ranges) / per_entry;
  if (g_cap_limit >= 0 && cap > g_cap_limit) cap = g_cap_limit;
  cap = cap < 0 ? 0 : (cap > Geom<CL>::kMaxSlice ? Geom<CL>::kMaxSlice : cap) & ~15;
  f.cap = cap;
  const size_t smem = ri_align_up((size_t)f.persist_off + ranges + (size_t)cap * per_entry, 16);
  RI_REQUIRE((int)smem <= budget, "nprobe=%d needs %zu bytes of shared memory per CTA (limit %d)", p.nprobe, smem, budget);
  RI_CUDA_OK(cudaFuncSetAttribute(wave_fused_kernel<DT, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  RI_CUDA_OK(ri_launch_pdl_id(5, wave_fused_kernel<DT, CL>, dim3(CL, p.groups), dim3(kFusedThreads), smem, s, f));
  return RI_OK;
}

}  // namespace

bool fused_supported(const ri_wave_layer& p) { return p.n_centroids <= kFusedMaxCentroids; }

// Test hook: cap the estimation entries a CTA keeps in shared memory (0 forces the global lists, a small value the
// mixed case); negative restores the default.  Not part of the decode interface.
extern "C" int ri_wave_test_local_cap(int cap) {
  g_cap_limit = cap;
  return RI_OK;
}

// How many clusters of CL CTAs of this kernel the device can hold at once (asked once per device).  Clusters are placed
// inside one GPC, so this is less than SMs / CL: a B200 with 148 SMs holds 15 clusters of 8, not 18.
template <int DT, int CL>
int resident_clusters(int* out) {
  static int cached[64] = {0};
  int dev = 0;
  RI_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) { *out = cached[dev]; return RI_OK; }
  int budget = 0, sms = 0;
  const int rc = dynamic_budget<DT, CL>(&budget, &sms);
  if (rc != RI_OK) return rc;
  RI_CUDA_OK(cudaFuncSetAttribute(wave_fused_kernel<DT, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CL, 64);
  cfg.blockDim = dim3(kFusedThreads);
  cfg.dynamicSmemBytes = (size_t)budget;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, wave_fused_kernel<DT, CL>, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = sms / CL;               // the query is unavailable: the bound that ignores GPC boundaries
  }
  if (dev >= 0 && dev < 64) cached[dev] = n;
  *out = n;
  return RI_OK;
}

template <int DT>
int launch_fused_dt(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather) {
  // cluster size: the largest of 8 .. 4 CTAs per group with which all groups' clusters are resident at once (a cluster
  // that has to wait for another one to finish doubles the layer's time).  Clusters are placed inside a GPC, so the
  // counts are not SMs / size: a B200 holds 15 clusters of 8 or 7 CTAs, 22 of 6, 26 of 5, 33 of 4.
  int fit = 0, rc;
  if ((rc = resident_clusters<DT, 8>(&fit)) != RI_OK) return rc;
  if (p.groups <= fit) return launch<DT, 8>(p, L, s, gather);
  if ((rc = resident_clusters<DT, 7>(&fit)) != RI_OK) return rc;
  if (p.groups <= fit) return launch<DT, 7>(p, L, s, gather);
  if ((rc = resident_clusters<DT, 6>(&fit)) != RI_OK) return rc;
  if (p.groups <= fit) return launch<DT, 6>(p, L, s, gather);
  if ((rc = resident_clusters<DT, 5>(&fit)) != RI_OK) return rc;
  if (p.groups <= fit) return launch<DT, 5>(p, L, s, gather);
  return launch<DT, 4>(p, L, s, gather);
}

int launch_fused(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather) {
  return p.dtype == RI_BF16 ? launch_fused_dt<RI_BF16>(p, L, s, gather) : launch_fused_dt<RI_F16>(p, L, s, gather);
}

int launch_gather_wait(const ri_wave_gather& g, cudaStream_t s) {
  const long long limit_ns = (g.wait_limit_us > 0 ? (long long)g.wait_limit_us : 1000000ll) * 1000ll;
  RI_CUDA_OK(ri_launch_pdl_id(6, gather_signal_wait_kernel, dim3(1), dim3(64), 0, s, g.d_flag_slots, g.d_flags, g.d_epoch,
                              g.d_error, g.n_ranks, limit_ns, g.d_stamps));
  return RI_OK;
}

}  // namespace ri_wave
