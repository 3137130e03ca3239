// Fused wave-index decode attention for one layer: scan -> select -> attend.
//
//   scan    q.C^T over every centroid of every group (the only pass over the 2*C*d-byte
//           centroid table), scores kept in fp32.
//   select  per group: per-head softmax over the 16-bit-rounded scores, group sum, masked
//           clusters last, exact two-level radix select on 16-bit keys into the retrieval
//           set (top P, ranked) and the estimation set (next E), page-budget rule, and the
//           row list of the retrieved clusters.
//   attend  split-K weighted flash decoding that reads the retrieved clusters in place from
//           the cluster-contiguous KV store and the steady zone, treats every estimated
//           cluster as one row (score from the scan, value = value sum, denominator weight =
//           cluster size) and merges everything by log-sum-exp; the last chunk of a group to
//           finish combines the partial results.
//
// Tensor-core use: warp-level m16n8k16 MMA with the GQA group packed into the M (QK^T) or N
// (PV) dimension.  Fragments are loaded straight from global memory with 16-byte loads; the
// contraction index is permuted identically on both operands so that no shared-memory
// transpose is needed (see load notes at wave_scan_kernel and attend_step).
#include "ri_common.cuh"

namespace {

constexpr int kScanTile = 128;     // centroids per scan CTA (4 warps x 4 n-tiles of 8)
constexpr int kSelectThreads = 1024;
constexpr int kAttendChunk = 128;  // rows per attend CTA (4 warps x 2 steps of 16)
constexpr int kMaxHeads = 8;       // GQA group size limit (N dimension of the PV MMA)

struct Layout {
  int64_t scores, dist_keys, est_ids, est_w, est_s2, rows, n_exact, part_o, part_m, part_l, counters, total;
  int e_pad, n_chunks, est_chunks;
};

Layout make_layout(const ri_wave_layer& p) {
  Layout L;
  const int64_t G = p.groups;
  L.e_pad = (int)ri_align_up(p.n_estimate > 0 ? p.n_estimate : 1, 16);
  L.est_chunks = (p.n_estimate + kAttendChunk - 1) / kAttendChunk;
  const int exact_max = p.steady_stride + p.max_exact_rows;
  L.n_chunks = L.est_chunks + (exact_max + kAttendChunk - 1) / kAttendChunk;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = ri_align_up(off + bytes, 256); return o; };
  L.counters = take(G * 4);   // first: the only region that must start zeroed
  L.scores = take(G * p.group_size * (int64_t)p.n_centroids * 4);
  L.dist_keys = take(G * (int64_t)p.n_centroids * 2);
  L.est_ids = take(G * L.e_pad * 4);
  L.est_w = take(G * L.e_pad * 4);
  L.est_s2 = take(G * kMaxHeads * (int64_t)L.e_pad * 4);
  L.rows = take(G * (int64_t)p.max_exact_rows * 4);
  L.n_exact = take(G * 4);
  L.part_o = take(G * L.n_chunks * (int64_t)p.group_size * RI_HEAD_DIM * 4);
  L.part_m = take(G * L.n_chunks * kMaxHeads * 4);
  L.part_l = take(G * L.n_chunks * kMaxHeads * 4);
  L.total = off;
  return L;
}

int validate_geometry_only(const ri_wave_layer* p) {
  RI_REQUIRE(p != nullptr, "ri_wave_layer is null");
  RI_REQUIRE(p->groups > 0 && p->groups <= 65535, "groups=%d out of range", p->groups);
  RI_REQUIRE(p->group_size >= 1 && p->group_size <= kMaxHeads, "group_size=%d unsupported (1..8)", p->group_size);
  RI_REQUIRE(p->n_centroids > 0 && p->n_centroids % 8 == 0 && p->n_centroids <= 65528,
             "n_centroids=%d must be a positive multiple of 8 below 65536", p->n_centroids);
  RI_REQUIRE(p->nprobe >= 1 && p->nprobe <= 1024, "nprobe=%d unsupported (1..1024)", p->nprobe);
  RI_REQUIRE(p->n_estimate >= 0 && p->nprobe + p->n_estimate <= p->n_centroids,
             "nprobe+n_estimate=%d exceeds n_centroids=%d", p->nprobe + p->n_estimate, p->n_centroids);
  RI_REQUIRE(p->page_size >= 1 && p->buffer_pages >= 1, "page_size/buffer_pages must be positive");
  RI_REQUIRE((int64_t)p->buffer_pages * p->page_size <= p->max_exact_rows,
             "max_exact_rows=%d smaller than buffer_pages*page_size", p->max_exact_rows);
  RI_REQUIRE(p->dtype == RI_BF16 || p->dtype == RI_F16, "dtype=%d unsupported", p->dtype);
  RI_REQUIRE(p->steady_stride >= 1 && p->tokens_per_group >= 0, "bad steady_stride/tokens_per_group");
  return RI_OK;
}

int validate(const ri_wave_layer* p) {
  const int rc = validate_geometry_only(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(p->d_centroids && p->d_value_sum && p->d_cluster_size && p->d_cluster_count && p->d_cluster_offset,
             "meta-index pointer is null");
  RI_REQUIRE(p->d_keys && p->d_values && p->d_steady_keys && p->d_steady_values && p->d_static_len,
             "KV pointer is null");
  RI_REQUIRE(p->d_q && p->d_out && p->d_scratch, "q/out/scratch pointer is null");
  RI_REQUIRE(((uintptr_t)p->d_centroids | (uintptr_t)p->d_value_sum | (uintptr_t)p->d_keys | (uintptr_t)p->d_values |
              (uintptr_t)p->d_steady_keys | (uintptr_t)p->d_steady_values | (uintptr_t)p->d_q |
              (uintptr_t)p->d_scratch) % 16 == 0,
             "tensor pointers must be 16-byte aligned");
  return RI_OK;
}

// ---------------------------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------------------------
// Lane (r = lane/4, t = lane%4) loads, from row r of an 8-row tile, the four 16-byte pieces at
// byte offsets 16*t + 64*kk (kk = 0..3).  Piece kk feeds MMA k-steps 2kk and 2kk+1: its four
// 32-bit words are (b0, b1) of step 2kk and (b0, b1) of step 2kk+1.  The query row of head r is
// loaded with the very same pattern and used as (a0, a2), so both operands see the same
// permutation of the 128 channels and the dot product is unchanged.
template <int DT>
__global__ void __launch_bounds__(128) wave_scan_kernel(const uint4* __restrict__ q, const uint4* __restrict__ cent,
                                                        float* __restrict__ scores, int C, int gs, float alpha) {
  const int g = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int base = blockIdx.x * kScanTile + warp * 32;
  if (base >= C) return;

  uint4 kb[4][4];
  const uint4* crow = cent + ((int64_t)g * C + base + r) * 16 + t;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bool ok = base + j * 8 < C;   // C % 8 == 0: an 8-row tile is entirely in or out
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) kb[j][kk] = ok ? ri_ldg16(crow + j * 8 * 16 + kk * 4) : make_uint4(0, 0, 0, 0);
  }
  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = r < gs ? ri_ldg16(q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      Elem<DT>::mma16816(acc, qa[kk].x, 0u, qa[kk].y, 0u, kb[j][kk].x, kb[j][kk].y);
      Elem<DT>::mma16816(acc, qa[kk].z, 0u, qa[kk].w, 0u, kb[j][kk].z, kb[j][kk].w);
    }
    const int c0 = base + j * 8 + 2 * t;
    if (r < gs && c0 < C) {
      float2 v = make_float2(alpha * acc[0], alpha * acc[1]);
      *reinterpret_cast<float2*>(scores + ((int64_t)g * gs + r) * C + c0) = v;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// select
// ---------------------------------------------------------------------------------------------
// Exclusive scan of one 32-bit value per thread over the whole block (1024 threads).
// `warp_sums` is a 32-entry shared array.  Returns the exclusive prefix; `total` = block sum.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();   // protects warp_sums from the previous use
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  uint32_t ws = warp_sums[lane];
  uint32_t winc = ws;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += n;
  }
  total = __shfl_sync(0xffffffffu, winc, 31);
  const uint32_t warp_base = __shfl_sync(0xffffffffu, winc - ws, warp);
  return warp_base + inc - v;
}

// Among 256 histogram bins (highest bin = largest keys) find, for each of two targets k, the
// bin where the count from the top first reaches k.  out[2*i] = bin, out[2*i+1] = count
// strictly above that bin.  Executed by threads 0..255; all threads must call.
__device__ __forceinline__ void find_bins(const int* hist, int k0, int k1, int* out, uint32_t* warp_sums) {
  const int tid = threadIdx.x;
  const int bin = 255 - tid;
  const uint32_t cnt = tid < 256 ? (uint32_t)hist[bin] : 0u;
  uint32_t total;
  const uint32_t above = block_exclusive_scan(cnt, warp_sums, total);
  if (tid < 256) {
    if ((int)above < k0 && (int)(above + cnt) >= k0) { out[0] = bin; out[1] = (int)above; }
    if ((int)above < k1 && (int)(above + cnt) >= k1) { out[2] = bin; out[3] = (int)above; }
  }
  __syncthreads();
}

struct SelectArgs {
  const float* scores;
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
  int C, gs, P, E, e_pad, page, buffer_pages, max_rows;
};

template <int DT>
__global__ void __launch_bounds__(kSelectThreads) wave_select_kernel(SelectArgs a) {
  extern __shared__ __align__(16) uint8_t dyn[];
  uint16_t* keys = reinterpret_cast<uint16_t*>(dyn);                       // [C]
  uint32_t* cand = reinterpret_cast<uint32_t*>(dyn + ri_align16(a.C * 2)); // [P]
  uint32_t* ranked = cand + a.P;                                           // [P]

  __shared__ float red[32][kMaxHeads];
  __shared__ float s_max[kMaxHeads], s_inv[kMaxHeads];
  __shared__ int hist_a[256], hist_b[256];
  __shared__ int bins[4], lows[4];
  __shared__ uint32_t warp_sums[32];
  __shared__ int s_keep, s_total_rows;

  const int g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = a.C, gs = a.gs;
  const float* sc = a.scores + (int64_t)g * gs * C;

  // ---- per-head maximum of the rounded scores ----
  float mx[kMaxHeads];
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) mx[h] = -INFINITY;
  for (int c = tid; c < C; c += kSelectThreads)
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) mx[h] = fmaxf(mx[h], Elem<DT>::round(sc[(int64_t)h * C + c]));
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
    if (lane == 0) red[warp][h] = mx[h];
  }
  if (tid < 256) { hist_a[tid] = 0; hist_b[tid] = 0; }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h) {
      float v = red[lane][h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) s_max[h] = v;
    }
  }
  __syncthreads();

  // ---- per-head sum of exp(s - max) ----
  float sm[kMaxHeads];
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) sm[h] = 0.f;
  for (int c = tid; c < C; c += kSelectThreads)
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) sm[h] += exp2f((Elem<DT>::round(sc[(int64_t)h * C + c]) - s_max[h]) * RI_LOG2E);
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sm[h] += __shfl_xor_sync(0xffffffffu, sm[h], o);
    if (lane == 0) red[warp][h] = sm[h];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h) {
      float v = red[lane][h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) s_inv[h] = 1.0f / v;
    }
  }
  __syncthreads();

  // ---- group distance -> 16-bit ordered keys, first-level histogram ----
  for (int c = tid; c < C; c += kSelectThreads) {
    float dist = 0.f;
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
      if (h < gs) {
        const float s = Elem<DT>::round(sc[(int64_t)h * C + c]);
        dist += Elem<DT>::round(exp2f((s - s_max[h]) * RI_LOG2E) * s_inv[h]);
      }
    uint16_t b = Elem<DT>::bits(dist);
    if (a.count[(int64_t)g * C + c] == 0) b = DT == RI_BF16 ? 0xFF7Fu : 0xFBFFu;   // most negative finite
    const uint16_t k = ri_ordered_key(b);
    keys[c] = k;
    a.dist_keys[(int64_t)g * C + c] = k;
    atomicAdd(&hist_a[k >> 8], 1);
  }
  __syncthreads();

  const int K = a.P + a.E;
  find_bins(hist_a, K, a.P, bins, warp_sums);
  const int binK = bins[0], aboveK1 = bins[1], binP = bins[2], aboveP1 = bins[3];
  if (tid < 256) hist_a[tid] = 0;
  __syncthreads();
  for (int c = tid; c < C; c += kSelectThreads) {
    const uint16_t k = keys[c];
    if ((k >> 8) == binK) atomicAdd(&hist_a[k & 255], 1);
    if ((k >> 8) == binP) atomicAdd(&hist_b[k & 255], 1);
  }
  __syncthreads();
  find_bins(hist_a, K - aboveK1, 1 << 30, lows, warp_sums);
  find_bins(hist_b, 1 << 30, a.P - aboveP1, lows, warp_sums);
  const uint16_t TK = (uint16_t)((binK << 8) | lows[0]);
  const uint16_t TP = (uint16_t)((binP << 8) | lows[2]);
  const int needK = K - aboveK1 - lows[1];       // how many keys equal to TK are taken
  const int needP = a.P - aboveP1 - lows[3];

  // ---- ordered compaction: estimation entries and retrieval candidates ----
  int tieK_base = 0, tieP_base = 0, est_base = 0, ret_base = 0;
  for (int c0 = 0; c0 < C; c0 += kSelectThreads) {
    const int c = c0 + tid;
    const bool in = c < C;
    const uint16_t k = in ? keys[c] : (uint16_t)0;
    const bool eqK = in && k == TK, eqP = in && k == TP;
    uint32_t total;
    const uint32_t pre = block_exclusive_scan((eqK ? 1u : 0u) | (eqP ? 0x10000u : 0u), warp_sums, total);
    const bool inK = in && (k > TK || (eqK && tieK_base + (int)(pre & 0xffffu) < needK));
    const bool inP = in && (k > TP || (eqP && tieP_base + (int)(pre >> 16) < needP));
    tieK_base += (int)(total & 0xffffu);
    tieP_base += (int)(total >> 16);
    const bool isEst = inK && !inP;
    uint32_t total2;
    const uint32_t pos = block_exclusive_scan((isEst ? 1u : 0u) | (inP ? 0x10000u : 0u), warp_sums, total2);
    if (isEst) {
      const int e = est_base + (int)(pos & 0xffffu);
      if (e < a.E) {
        a.est_ids[(int64_t)g * a.e_pad + e] = c;
        a.est_w[(int64_t)g * a.e_pad + e] = Elem<DT>::from_bits(a.size_dt[(int64_t)g * C + c]);
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h)
          if (h < gs) a.est_s2[((int64_t)g * kMaxHeads + h) * a.e_pad + e] = sc[(int64_t)h * C + c] * RI_LOG2E;
        if (a.estimated_ids) a.estimated_ids[(int64_t)g * a.E + e] = c;
      }
    }
    if (inP) {
      const int i = ret_base + (int)(pos >> 16);
      if (i < a.P) cand[i] = ((uint32_t)k << 16) | (uint32_t)(0xffff - c);
    }
    est_base += (int)(total2 & 0xffffu);
    ret_base += (int)(total2 >> 16);
  }
  __syncthreads();

  // ---- rank the P candidates: descending distance, ties towards the lower cluster id ----
  for (int i = tid; i < a.P; i += kSelectThreads) {
    const uint32_t mine = cand[i];
    int rank = 0;
    for (int j = 0; j < a.P; ++j) rank += cand[j] > mine;
    ranked[rank] = mine;
  }
  __syncthreads();

  // ---- page-budget rule, then the row list of the kept clusters ----
  {
    const bool in = tid < a.P;
    const int cid = in ? 0xffff - (int)(ranked[tid] & 0xffffu) : 0;
    const int cnt = in ? a.count[(int64_t)g * C + cid] : 0;
    const uint32_t pages = in ? (uint32_t)((cnt + a.page - 1) / a.page) : 0u;
    uint32_t total;
    const uint32_t pages_before = block_exclusive_scan(pages, warp_sums, total);
    const bool fits = in && (int)(pages_before + pages) <= a.buffer_pages;
    // the pages are non-negative, so the clusters that fit form a prefix of the ranking
    uint32_t kept_total;
    block_exclusive_scan(fits ? 1u : 0u, warp_sums, kept_total);
    uint32_t rows_total;
    const uint32_t row_start = block_exclusive_scan(fits ? (uint32_t)cnt : 0u, warp_sums, rows_total);
    if (tid == 0) { s_keep = (int)kept_total; s_total_rows = (int)rows_total; }
    if (in) {
      cand[tid] = row_start;   // reuse: start position of this ranked cluster in the row list
      if (a.retrieved_ids) a.retrieved_ids[(int64_t)g * a.P + tid] = cid;
    }
  }
  __syncthreads();
  const int keep = s_keep;
  if (tid == 0) {
    a.n_exact[g] = s_total_rows;
    if (a.retrieved_kept) a.retrieved_kept[g] = keep;
  }
  for (int i = warp; i < keep; i += kSelectThreads / 32) {
    const int cid = 0xffff - (int)(ranked[i] & 0xffffu);
    const int off = a.offset[(int64_t)g * (C + 1) + cid];
    const int cnt = a.count[(int64_t)g * C + cid];
    const int start = (int)cand[i];
    for (int j = lane; j < cnt; j += 32)
      if (start + j < a.max_rows) a.rows[(int64_t)g * a.max_rows + start + j] = off + j;
  }
}

// ---------------------------------------------------------------------------------------------
// attend
// ---------------------------------------------------------------------------------------------
struct AttendArgs {
  const uint4* q;
  const uint4* keys;
  const uint4* values;
  const uint4* steady_k;
  const uint4* steady_v;
  const uint4* value_sum;
  const int32_t* static_len;
  const int32_t* rows;
  const int32_t* n_exact;
  const int32_t* est_ids;
  const float* est_w;
  const float* est_s2;
  float* part_o;
  float* part_m;
  float* part_l;
  uint32_t* counters;
  void* out;
  int64_t N;
  int C, gs, E, e_pad, est_chunks, n_chunks, steady_stride, max_rows;
  float scale2;   // log2(e) / sqrt(d)
};

// One 16-row step of the PV product.  Lane (r, t) owns rows tt = {2t, 2t+1, 8+2t, 9+2t} of the
// step and, of each, the two 16-byte pieces r and r+8 (channels 8r..8r+7 and 64+8r..64+8r+7).
// O^T tile x (16 channels x 8 heads) takes channel word x of those pieces: its low halves are
// MMA rows r, its high halves rows r+8, so tile x / row r is channel ch(x) = (x<4 ? 8r+2x :
// 64+8r+2(x-4)) and row r+8 is ch(x)+1.
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

template <int DT>
__global__ void __launch_bounds__(128) wave_attend_kernel(AttendArgs a) {
  const int g = blockIdx.y, chunk = blockIdx.x;
  const int static_len = *a.static_len;
  const int n_ret = a.n_exact[g];
  const int total_exact = static_len + n_ret;
  const int n_active = a.est_chunks + (total_exact + kAttendChunk - 1) / kAttendChunk;
  if (chunk >= n_active) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int gs = a.gs;
  const bool is_est = chunk < a.est_chunks;
  const int rows_end = is_est ? a.E : total_exact;
  const int chunk_base = (is_est ? chunk : chunk - a.est_chunks) * kAttendChunk;

  __shared__ float sm_o[4][kMaxHeads][RI_HEAD_DIM];
  __shared__ float sm_m[4][kMaxHeads], sm_l[4][kMaxHeads];
  __shared__ int s_last;

  uint4 qa[4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    qa[kk] = (!is_est && r < gs) ? ri_ldg16(a.q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);

  float acc[8][4];
#pragma unroll
  for (int x = 0; x < 8; ++x)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[x][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;   // for head r (l: this lane's share, reduced over the quad later)

  constexpr int kSteps = kAttendChunk / 4 / 16;
#pragma unroll 1
  for (int step = 0; step < kSteps; ++step) {
    const int base = chunk_base + warp * (kAttendChunk / 4) + step * 16;
    if (base >= rows_end) break;
    const int last = rows_end - 1;

    // ---- V rows of this lane: tt = 2t, 2t+1, 8+2t, 9+2t ----
    uint4 v[4][2];
    {
      const int tt[4] = {2 * t, 2 * t + 1, 8 + 2 * t, 9 + 2 * t};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = min(base + tt[i], last);
        const uint4* p;
        if (is_est) {
          p = a.value_sum + ((int64_t)g * a.C + a.est_ids[(int64_t)g * a.e_pad + row]) * 16;
        } else if (row < static_len) {
          p = a.steady_v + ((int64_t)g * a.steady_stride + row) * 16;
        } else {
          p = a.values + ((int64_t)g * a.N + a.rows[(int64_t)g * a.max_rows + row - static_len]) * 16;
        }
        v[i][0] = ri_ldg16(p + r);
        v[i][1] = ri_ldg16(p + r + 8);
      }
    }

    // ---- scores (log2 domain) of head r for rows j*8 + 2t + {0,1} ----
    float s2[2][2];
    float w[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if (is_est) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i0 = base + j * 8 + 2 * t;   // even, e_pad is a multiple of 16: float2 aligned
        float2 s = make_float2(-INFINITY, -INFINITY);
        if (r < gs) s = *reinterpret_cast<const float2*>(a.est_s2 + ((int64_t)g * kMaxHeads + r) * a.e_pad + i0);
        const float2 ww = *reinterpret_cast<const float2*>(a.est_w + (int64_t)g * a.e_pad + i0);
        s2[j][0] = s.x; s2[j][1] = s.y;
        w[j][0] = i0 < rows_end ? ww.x : 0.f;        // the padding of the scratch rows is not initialised
        w[j][1] = i0 + 1 < rows_end ? ww.y : 0.f;
      }
    } else {
      uint4 kb[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = min(base + j * 8 + r, last);
        const uint4* p;
        if (row < static_len) {
          p = a.steady_k + ((int64_t)g * a.steady_stride + row) * 16;
        } else {
          p = a.keys + ((int64_t)g * a.N + a.rows[(int64_t)g * a.max_rows + row - static_len]) * 16;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) kb[j][kk] = ri_ldg16(p + t + kk * 4);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          Elem<DT>::mma16816(c, qa[kk].x, 0u, qa[kk].y, 0u, kb[j][kk].x, kb[j][kk].y);
          Elem<DT>::mma16816(c, qa[kk].z, 0u, qa[kk].w, 0u, kb[j][kk].z, kb[j][kk].w);
        }
        s2[j][0] = c[0] * a.scale2;
        s2[j][1] = c[1] * a.scale2;
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (base + j * 8 + 2 * t + e >= rows_end) s2[j][e] = -INFINITY;

    // ---- online softmax for head r ----
    float mx = fmaxf(fmaxf(s2[0][0], s2[0][1]), fmaxf(s2[1][0], s2[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_safe);   // m_run = -inf -> 0
    float p[2][2];
    float psum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[j][e] = exp2f(s2[j][e] - m_safe);
        psum += p[j][e] * w[j][e];
      }
    l_run = l_run * alpha + psum;
    m_run = m_new;
    // accumulators hold heads 2t and 2t+1: fetch their rescale factors from the quads that own them
    const float f0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4);
    const float f1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      acc[x][0] *= f0; acc[x][1] *= f1; acc[x][2] *= f0; acc[x][3] *= f1;
    }
    const uint32_t b0 = Elem<DT>::pack2(p[0][0], p[0][1]);
    const uint32_t b1 = Elem<DT>::pack2(p[1][0], p[1][1]);
    pv_step<DT>(acc, v, b0, b1);
  }

  // ---- merge the four warps of this chunk ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (t == 0) { sm_m[warp][r] = m_run; sm_l[warp][r] = l_run; }
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int ch = (x < 4) ? 8 * r + 2 * x : 64 + 8 * r + 2 * (x - 4);
    sm_o[warp][2 * t][ch] = acc[x][0];
    sm_o[warp][2 * t + 1][ch] = acc[x][1];
    sm_o[warp][2 * t][ch + 1] = acc[x][2];
    sm_o[warp][2 * t + 1][ch + 1] = acc[x][3];
  }
  __syncthreads();
  const int64_t pbase = (int64_t)g * a.n_chunks + chunk;
  for (int h = 0; h < gs; ++h) {
    float M = fmaxf(fmaxf(sm_m[0][h], sm_m[1][h]), fmaxf(sm_m[2][h], sm_m[3][h]));
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const float f = exp2f(sm_m[wi][h] - Ms);
      L += sm_l[wi][h] * f;
      O += sm_o[wi][h][tid] * f;
    }
    a.part_o[(pbase * gs + h) * RI_HEAD_DIM + tid] = O;
    if (tid == 0) { a.part_m[pbase * kMaxHeads + h] = M; a.part_l[pbase * kMaxHeads + h] = L; }
  }

  // ---- the last chunk of the group to arrive combines all partial results ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t ticket = atomicAdd(&a.counters[g], 1u);
    s_last = ticket == (uint32_t)(n_active - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int64_t gbase = (int64_t)g * a.n_chunks;
  // All loads below are independent of one another, so the whole merge costs a few L2 round
  // trips instead of one per chunk.  Tables (n_active <= 256 rows of 8 heads) reuse sm_o.
  float* tf = &sm_o[0][0][0];                 // running max, then the rescale factor 2^(m - M)
  float* tl = tf + 256 * kMaxHeads;           // denominators
  for (int i = tid; i < n_active * kMaxHeads; i += 128) {
    tf[i] = __ldcg(a.part_m + gbase * kMaxHeads + i);
    tl[i] = __ldcg(a.part_l + gbase * kMaxHeads + i);
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {            // warp w reduces heads 2w and 2w+1
    const int h = warp * 2 + hh;
    float M = -INFINITY;
    for (int c = lane; c < n_active; c += 32) M = fmaxf(M, tf[c * kMaxHeads + h]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f;
    for (int c = lane; c < n_active; c += 32) {
      const float f = exp2f(tf[c * kMaxHeads + h] - Ms);
      tf[c * kMaxHeads + h] = f;
      L += tl[c * kMaxHeads + h] * f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0) sm_l[0][h] = L;
  }
  __syncthreads();
  const int dq = tid >> 2, cl = tid & 3;      // 4 channels per thread, chunks split 4 ways
  for (int h = 0; h < gs; ++h) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int c = cl; c < n_active; c += 4) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(a.part_o + ((gbase + c) * gs + h) * RI_HEAD_DIM) + dq);
      const float f = tf[c * kMaxHeads + h];
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (cl == 0) {
      const float L = sm_l[0][h];
      const float inv = L > 0.f ? 1.0f / L : 0.f;
      uint2 o2;
      o2.x = Elem<DT>::pack2(acc.x * inv, acc.y * inv);
      o2.y = Elem<DT>::pack2(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.out) + ((int64_t)g * gs + h) * RI_HEAD_DIM + 4 * dq) = o2;
    }
  }
  if (tid == 0) a.counters[g] = 0u;   // leave the scratch reusable
}

__global__ void steady_append_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, uint4* sk, uint4* sv,
                                     const int32_t* __restrict__ pos, int groups, int stride) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece each
  if (i >= groups * 16) return;
  const int g = i >> 4, c = i & 15;
  const int p = *pos;
  if (p < 0 || p >= stride) return;
  sk[((int64_t)g * stride + p) * 16 + c] = k[i];
  sv[((int64_t)g * stride + p) * 16 + c] = v[i];
}

template <int DT>
int launch_scan(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  dim3 grid((p.n_centroids + kScanTile - 1) / kScanTile, p.groups);
  wave_scan_kernel<DT><<<grid, 128, 0, s>>>(static_cast<const uint4*>(p.d_q), static_cast<const uint4*>(p.d_centroids),
                                            reinterpret_cast<float*>(sc + L.scores), p.n_centroids, p.group_size,
                                            0.08838834764831845f);
  RI_LAUNCH_OK("wave_scan_kernel");
  return RI_OK;
}

template <int DT>
int launch_select(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  SelectArgs a;
  a.scores = reinterpret_cast<const float*>(sc + L.scores);
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
  a.page = p.page_size; a.buffer_pages = p.buffer_pages; a.max_rows = p.max_exact_rows;
  const size_t smem = ri_align16(p.n_centroids * 2) + (size_t)p.nprobe * 8;
  if (smem > 48 * 1024)
    RI_CUDA_OK(cudaFuncSetAttribute(wave_select_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  wave_select_kernel<DT><<<p.groups, kSelectThreads, smem, s>>>(a);
  RI_LAUNCH_OK("wave_select_kernel");
  return RI_OK;
}

template <int DT>
int launch_attend(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  uint8_t* sc = static_cast<uint8_t*>(p.d_scratch);
  AttendArgs a;
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
  a.part_o = reinterpret_cast<float*>(sc + L.part_o);
  a.part_m = reinterpret_cast<float*>(sc + L.part_m);
  a.part_l = reinterpret_cast<float*>(sc + L.part_l);
  a.counters = reinterpret_cast<uint32_t*>(sc + L.counters);
  a.out = p.d_out;
  a.N = p.tokens_per_group;
  a.C = p.n_centroids; a.gs = p.group_size; a.E = p.n_estimate; a.e_pad = L.e_pad;
  a.est_chunks = L.est_chunks; a.n_chunks = L.n_chunks; a.steady_stride = p.steady_stride;
  a.max_rows = p.max_exact_rows;
  a.scale2 = RI_LOG2E * 0.08838834764831845f;
  RI_REQUIRE(L.n_chunks <= 256, "geometry needs %d attention chunks per group, the merge handles 256", L.n_chunks);
  dim3 grid(L.n_chunks, p.groups);
  wave_attend_kernel<DT><<<grid, 128, 0, s>>>(a);
  RI_LAUNCH_OK("wave_attend_kernel");
  return RI_OK;
}

}  // namespace

extern "C" int64_t ri_wave_scratch_bytes(const ri_wave_layer* p) {
  if (validate_geometry_only(p) != RI_OK) return RI_ERR_INVALID;
  return make_layout(*p).total;
}

extern "C" int ri_wave_scratch_views(const ri_wave_layer* p, ri_wave_views* out) {
  int rc = validate_geometry_only(p);
  if (rc != RI_OK) return rc;
  RI_REQUIRE(out != nullptr && p->d_scratch != nullptr, "views or scratch pointer is null");
  const Layout L = make_layout(*p);
  uint8_t* sc = static_cast<uint8_t*>(p->d_scratch);
  out->d_scores = reinterpret_cast<const float*>(sc + L.scores);
  out->d_dist_keys = reinterpret_cast<const uint16_t*>(sc + L.dist_keys);
  out->d_exact_rows = reinterpret_cast<const int32_t*>(sc + L.rows);
  out->d_n_exact = reinterpret_cast<const int32_t*>(sc + L.n_exact);
  return RI_OK;
}

#define RI_DISPATCH(fn, p, L, s) ((p)->dtype == RI_BF16 ? fn<RI_BF16>(*(p), L, s) : fn<RI_F16>(*(p), L, s))

extern "C" int ri_wave_scan(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return RI_DISPATCH(launch_scan, p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_select(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return RI_DISPATCH(launch_select, p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_attend(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  return RI_DISPATCH(launch_attend, p, L, static_cast<cudaStream_t>(stream));
}

extern "C" int ri_wave_decode_layer(const ri_wave_layer* p, void* stream) {
  int rc = validate(p);
  if (rc != RI_OK) return rc;
  const Layout L = make_layout(*p);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((rc = RI_DISPATCH(launch_scan, p, L, s)) != RI_OK) return rc;
  if ((rc = RI_DISPATCH(launch_select, p, L, s)) != RI_OK) return rc;
  return RI_DISPATCH(launch_attend, p, L, s);
}

extern "C" int ri_steady_append(const void* d_k, const void* d_v, void* d_steady_keys, void* d_steady_values,
                                const int32_t* d_position, int32_t groups, int32_t steady_stride, void* stream) {
  RI_REQUIRE(d_k && d_v && d_steady_keys && d_steady_values && d_position, "ri_steady_append: null pointer");
  RI_REQUIRE(groups > 0 && steady_stride > 0, "ri_steady_append: bad sizes");
  const int n = groups * 16;
  steady_append_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(d_k), static_cast<const uint4*>(d_v), static_cast<uint4*>(d_steady_keys),
      static_cast<uint4*>(d_steady_values), d_position, groups, steady_stride);
  RI_LAUNCH_OK("steady_append_kernel");
  return RI_OK;
}
