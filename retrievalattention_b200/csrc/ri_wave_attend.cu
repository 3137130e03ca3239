// attend: split-K weighted flash decoding over (a) the estimation set — every estimated cluster is
// one row: score from the scan, value = the cluster's value sum, weight = cluster size in the
// softmax denominator — and (b) the exact set — steady zone followed by the retrieved clusters, read
// in place from the cluster-contiguous KV store through the row list.
// (reference: the two weighted_flash_decoding calls, cache_hub/retroinfer_cache.py:611-617 and
// :666-674, with gather_copy_vectors :601-605 and gather_copy_and_concat :642-648 in between).
//
// Work decomposition: the 16-row steps of all groups form one list (per group: ceil(E/16)
// estimation steps, then ceil((steady + retrieved rows)/16) exact steps).  A fixed grid of
// persistent warps (2 CTAs x 4 warps per SM) cuts the list into equal contiguous ranges, one per
// warp, whatever the per-group row counts turn out to be.  A warp streams its steps through a
// lane-private three-stage cp.async ring in shared memory (256 bytes per lane and step; row ids of
// the next step to issue are prefetched into registers), keeps running (max, sum, O) for the
// group it is in, and writes one partial result per group it touches into slot (warp + group).
// wave_combine_kernel then merges each group's slots by log-sum-exp.
//
// Tensor-core use: m16n8k16 MMA.  QK^T has the GQA group in M and 8 rows in N, with the same
// channel permutation on both operands as in the scan.  PV is computed transposed (16 channels in
// M, the 8 heads in N, 16 rows in K): lane (r, t) owns rows tt = {2t, 2t+1, 8+2t, 9+2t} of the step
// and, of each, the 16-byte pieces r and r+8 (channels 8r..8r+7 and 64+8r..64+8r+7).  O^T tile x
// takes channel word x of those pieces: low halves are MMA rows r, high halves rows r+8, so tile x,
// row r is channel ch(x) = (x<4 ? 8r+2x : 64+8r+2(x-4)) and row r+8 is ch(x)+1.  The probabilities
// come straight from the QK^T accumulators as the B fragment.
#include "ri_wave_internal.cuh"

namespace ri_wave {
namespace {

constexpr int kStages = 3;
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
  const int32_t* rows;
  const int32_t* n_exact;
  const int32_t* est_ids;
  const float* est_w;
  const float* est_s2;
  float* part_o;       // [slots, gs, 128]
  float* part_m;       // [slots, 8]
  float* part_l;       // [slots, 8]
  int32_t* prefix;     // [G + 1] exact steps of all earlier groups (written by CTA 0, read by the combine)
  void* out;
  int64_t N;
  int G, C, gs, E, e_pad, e_steps, steady_stride, max_rows;
  float scale2;        // log2(e) / sqrt(d)
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

template <int DT>
__global__ void __launch_bounds__(128, 2) wave_attend_kernel(AttendArgs a) {
  ri_pdl_enter();
  extern __shared__ __align__(16) uint8_t dyn[];
  uint8_t* ring = dyn;
  int* px = reinterpret_cast<int*>(dyn + kRingBytes);       // [G + 1] exact steps of all earlier groups
  int* texact = px + a.G + 1;                                // [G] steady + retrieved rows of each group
  __shared__ uint32_t scan_sums[4];
  __shared__ int s_carry;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int gs = a.gs;
  const int static_len = *a.static_len;

  // ---- the step list: exclusive prefix sum of the per-group step counts ----
  if (tid == 0) s_carry = 0;
  __syncthreads();
  for (int g0 = 0; g0 < a.G; g0 += 128) {
    const int g = g0 + tid;
    int steps = 0;
    if (g < a.G) {
      const int te = static_len + a.n_exact[g];
      texact[g] = te;
      steps = (te + 15) / 16;
    }
    uint32_t inc = (uint32_t)steps;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) scan_sums[warp] = inc;
    __syncthreads();
    uint32_t base = (uint32_t)s_carry, tot = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      if (w < warp) base += scan_sums[w];
      tot += scan_sums[w];
    }
    if (g < a.G) px[g] = (int)(base + inc) - steps;
    __syncthreads();
    if (tid == 0) s_carry += (int)tot;
    __syncthreads();
  }
  if (tid == 0) px[a.G] = s_carry;
  __syncthreads();
  if (blockIdx.x == 0)
    for (int g = tid; g <= a.G; g += 128) a.prefix[g] = px[g];
  // An estimation step moves half the bytes of an exact step (no keys), so ranges are cut in cost
  // units: 1 per estimation step, 2 per exact step.  A step belongs to the warp that holds its
  // first unit.
  const int es = a.e_steps;
  auto step_start = [&](int g) { return g * es + px[g]; };        // first step of group g
  auto unit_start = [&](int g) { return g * es + 2 * px[g]; };    // first cost unit of group g
  auto group_of_unit = [&](int u) {                               // last g with unit_start(g) <= u
    int a0 = 0, b0 = a.G - 1;
    while (a0 < b0) {
      const int mid = (a0 + b0 + 1) >> 1;
      if (unit_start(mid) <= u) a0 = mid; else b0 = mid - 1;
    }
    return a0;
  };
  auto steps_before_unit = [&](int u) {                           // steps whose first unit is < u
    const int g = group_of_unit(u);
    const int uu = u - unit_start(g);
    return step_start(g) + (uu < es ? uu : es + (uu - es + 1) / 2);
  };
  const int total_units = unit_start(a.G);

  // ---- this warp's contiguous range of steps (no CTA-wide barrier below this point) ----
  const int n_warps = gridDim.x * 4;
  const int per = max(2, (total_units + n_warps - 1) / n_warps);   // >= 2: every range inside a group holds a step
  const int wid = blockIdx.x * 4 + warp;
  const int lu = min(total_units, wid * per), hu = min(total_units, lu + per);
  const int lo = steps_before_unit(lu), hi = steps_before_unit(hu);
  if (lo >= hi) return;
  int g_issue = group_of_unit(lu);
  while (lo >= step_start(g_issue + 1)) ++g_issue;   // lu may sit in the middle of the previous group's last step
  int g_cur = g_issue;
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring) + warp * kStages * kStageBytes + lane * 16;
  const uint8_t* my_ring_ptr = ring + warp * kStages * kStageBytes + lane * 16;

  // ids of the rows this lane touches in step s of group g
  auto load_ids = [&](int s, int g) {
    RowIds id;
    const int j = s - step_start(g);
    const bool est = j < a.e_steps;
    const int base = (est ? j : j - a.e_steps) * 16;
    const int last = (est ? a.E : texact[g]) - 1;
    const int tt[4] = {2 * t, 2 * t + 1, 8 + 2 * t, 9 + 2 * t};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = min(base + tt[i], last);
      if (est) id.v[i] = a.est_ids[(int64_t)g * a.e_pad + row];
      else id.v[i] = row < static_len ? -1 - row : a.rows[(int64_t)g * a.max_rows + row - static_len];
    }
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int row = min(base + jj * 8 + r, last);
      id.k[jj] = est ? 0 : (row < static_len ? -1 - row : a.rows[(int64_t)g * a.max_rows + row - static_len]);
    }
    return id;
  };

  // start the copies of step s (group g) into ring stage `stage`
  auto issue = [&](int s, int g, int stage, const RowIds& id) {
    const uint32_t dst = my_ring + stage * kStageBytes;
    const int j = s - step_start(g);
    if (j < a.e_steps) {
      // pieces 0/1: this lane's scores and weights of the step; pieces 8..15: value-sum rows
      const int i0 = j * 16 + 2 * t;
      if (r < gs) {
        const float* sp = a.est_s2 + ((int64_t)g * kMaxHeads + r) * a.e_pad + i0;
        cp_async8(dst, sp);
        cp_async8(dst + 8, sp + 8);
      }
      const float* wp = a.est_w + (int64_t)g * a.e_pad + i0;
      cp_async8(dst + 512, wp);
      cp_async8(dst + 512 + 8, wp + 8);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4* p = a.value_sum + ((int64_t)g * a.C + id.v[i]) * 16;
        cp_async16(dst + (8 + 2 * i) * 512, p + r);
        cp_async16(dst + (9 + 2 * i) * 512, p + r + 8);
      }
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
  float acc[8][4];
  float m_run = -INFINITY, l_run = 0.f;   // head r (l: this lane's share, reduced over the quad when flushed)
  uint4 qa[4];
  auto reset = [&](int g) {
#pragma unroll
    for (int x = 0; x < 8; ++x)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[x][i] = 0.f;
    m_run = -INFINITY;
    l_run = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      qa[kk] = r < gs ? ri_ldg16(a.q + ((int64_t)g * gs + r) * 16 + t + kk * 4) : make_uint4(0, 0, 0, 0);
  };
  // one partial result per (warp, group): slot = warp + group is unique because both only grow
  auto flush = [&](int g) {
    const int64_t slot = (int64_t)wid + g;
    float l = l_run;
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0 && r < gs) { a.part_m[slot * kMaxHeads + r] = m_run; a.part_l[slot * kMaxHeads + r] = l; }
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const int ch = (x < 4) ? 8 * r + 2 * x : 64 + 8 * r + 2 * (x - 4);
      if (2 * t < gs)
        *reinterpret_cast<float2*>(a.part_o + (slot * gs + 2 * t) * RI_HEAD_DIM + ch) = make_float2(acc[x][0], acc[x][2]);
      if (2 * t + 1 < gs)
        *reinterpret_cast<float2*>(a.part_o + (slot * gs + 2 * t + 1) * RI_HEAD_DIM + ch) = make_float2(acc[x][1], acc[x][3]);
    }
  };

  // ---- prologue: fill the ring ----
  int s_issue = lo;
  RowIds nid = load_ids(lo, g_issue);
#pragma unroll
  for (int st = 0; st < kStages; ++st) {
    if (s_issue < hi) {
      issue(s_issue, g_issue, st, nid);
      ++s_issue;
      if (s_issue < hi) {
        while (s_issue >= step_start(g_issue + 1)) ++g_issue;
        nid = load_ids(s_issue, g_issue);
      }
    }
    cp_async_commit();
  }
  reset(g_cur);

  int stage = 0;
#pragma unroll 1
  for (int s = lo; s < hi; ++s) {
    if (s >= step_start(g_cur + 1)) {          // entering the next group: hand over what was accumulated
      flush(g_cur);
      while (s >= step_start(g_cur + 1)) ++g_cur;
      reset(g_cur);
    }
    cp_async_wait<kStages - 1>();           // the group of step s has landed (lane-private slots: no barrier)
    const uint8_t* src = my_ring_ptr + stage * kStageBytes;
    const int j = s - step_start(g_cur);
    const bool is_est = j < a.e_steps;
    const int base = (is_est ? j : j - a.e_steps) * 16;
    const int rows_end = is_est ? a.E : texact[g_cur];

    float s2[2][2];
    float w[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
    if (is_est) {
      const float4 sv = *reinterpret_cast<const float4*>(src);
      const float4 wv = *reinterpret_cast<const float4*>(src + 512);
      const bool head = r < gs;
      s2[0][0] = head ? sv.x : -INFINITY; s2[0][1] = head ? sv.y : -INFINITY;
      s2[1][0] = head ? sv.z : -INFINITY; s2[1][1] = head ? sv.w : -INFINITY;
      w[0][0] = wv.x; w[0][1] = wv.y; w[1][0] = wv.z; w[1][1] = wv.w;
    } else {
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint4 kb = *reinterpret_cast<const uint4*>(src + (4 * jj + kk) * 512);
          Elem<DT>::mma16816(c, qa[kk].x, 0u, qa[kk].y, 0u, kb.x, kb.y);
          Elem<DT>::mma16816(c, qa[kk].z, 0u, qa[kk].w, 0u, kb.z, kb.w);
        }
        s2[jj][0] = c[0] * a.scale2;
        s2[jj][1] = c[1] * a.scale2;
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
    if (s_issue < hi) {
      issue(s_issue, g_issue, stage, nid);
      ++s_issue;
      if (s_issue < hi) {
        while (s_issue >= step_start(g_issue + 1)) ++g_issue;
        nid = load_ids(s_issue, g_issue);
      }
    }
    cp_async_commit();
    stage = stage + 1 == kStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();
  flush(g_cur);
}

// Merge the partial results of one (group, head): slots wid + g for the warps whose ranges meet the
// group.  grid (gs, G), 128 threads: thread = (4 channels) x (slots split 4 ways).
template <int DT>
__global__ void __launch_bounds__(128) wave_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                                                           const float* __restrict__ part_l, const int32_t* __restrict__ prefix,
                                                           void* out, int G, int gs, int n_warps, int e_steps) {
  ri_pdl_enter();
  extern __shared__ float factor[];          // [slots of this group]
  __shared__ float red[4];
  __shared__ float s_M, s_L;
  const int h = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // same cost-unit arithmetic as the attend kernel (prefix[] = exact steps of all earlier groups)
  const int total_units = G * e_steps + 2 * prefix[G];
  const int per = max(2, (total_units + n_warps - 1) / n_warps);
  const int u0 = g * e_steps + 2 * prefix[g];                       // first unit of the group's first step
  const int x_steps = prefix[g + 1] - prefix[g];
  const int n_steps = e_steps + x_steps;
  uint16_t* o = reinterpret_cast<uint16_t*>(out) + ((int64_t)g * gs + h) * RI_HEAD_DIM;
  if (n_steps <= 0) {                          // a group without rows: zero output
    o[tid] = 0;
    return;
  }
  const int u_last = x_steps > 0 ? u0 + e_steps + 2 * (x_steps - 1) : u0 + e_steps - 1;   // first unit of its last step
  const int w0 = u0 / per, n = u_last / per - w0 + 1;
  const int64_t slot0 = (int64_t)w0 + g;
  float M = -INFINITY;
  for (int c = tid; c < n; c += 128) M = fmaxf(M, part_m[(slot0 + c) * kMaxHeads + h]);
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, x));
  if (lane == 0) red[warp] = M;
  __syncthreads();
  if (tid == 0) s_M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  const float Ms = s_M == -INFINITY ? 0.f : s_M;
  float L = 0.f;
  for (int c = tid; c < n; c += 128) {
    const float f = exp2f(part_m[(slot0 + c) * kMaxHeads + h] - Ms);
    factor[c] = f;
    L += part_l[(slot0 + c) * kMaxHeads + h] * f;
  }
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) L += __shfl_xor_sync(0xffffffffu, L, x);
  __syncthreads();                             // red[] reuse; factor[] visible
  if (lane == 0) red[warp] = L;
  __syncthreads();
  if (tid == 0) s_L = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  const int dq = tid >> 2, cl = tid & 3;
  float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int c = cl; c < n; c += 4) {
    const float4 v = *reinterpret_cast<const float4*>(part_o + ((slot0 + c) * gs + h) * RI_HEAD_DIM + 4 * dq);
    const float f = factor[c];
    o4.x += v.x * f; o4.y += v.y * f; o4.z += v.z * f; o4.w += v.w * f;
  }
#pragma unroll
  for (int x = 1; x <= 2; x <<= 1) {
    o4.x += __shfl_xor_sync(0xffffffffu, o4.x, x);
    o4.y += __shfl_xor_sync(0xffffffffu, o4.y, x);
    o4.z += __shfl_xor_sync(0xffffffffu, o4.z, x);
    o4.w += __shfl_xor_sync(0xffffffffu, o4.w, x);
  }
  if (cl == 0) {
    const float inv = s_L > 0.f ? 1.0f / s_L : 0.f;
    uint2 o2;
    o2.x = Elem<DT>::pack2(o4.x * inv, o4.y * inv);
    o2.y = Elem<DT>::pack2(o4.z * inv, o4.w * inv);
    *reinterpret_cast<uint2*>(o + 4 * dq) = o2;
  }
}

int attend_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kAttendMaxCtas;
  if (cached[dev] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cached[dev] = sms * 2 < kAttendMaxCtas ? sms * 2 : kAttendMaxCtas;
  }
  return cached[dev];
}

template <int DT>
int launch(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
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
  a.prefix = reinterpret_cast<int32_t*>(sc + L.prefix);
  a.out = p.d_out;
  a.N = p.tokens_per_group;
  a.G = p.groups; a.C = p.n_centroids; a.gs = p.group_size; a.E = p.n_estimate; a.e_pad = L.e_pad;
  a.e_steps = (p.n_estimate + 15) / 16;
  a.steady_stride = p.steady_stride; a.max_rows = p.max_exact_rows;
  a.scale2 = RI_LOG2E * 0.08838834764831845f;
  RI_REQUIRE(p.groups <= kAttendMaxGroups, "groups=%d exceeds the %d the attention stage indexes", p.groups, kAttendMaxGroups);
  const int ctas = attend_ctas();
  const int smem = kRingBytes + (2 * p.groups + 1) * 4;
  RI_CUDA_OK(cudaFuncSetAttribute(wave_attend_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  RI_CUDA_OK(ri_launch_pdl_id(2, wave_attend_kernel<DT>, dim3(ctas), dim3(128), (size_t)smem, s, a));
  RI_CUDA_OK(ri_launch_pdl_id(3, wave_combine_kernel<DT>, dim3(p.group_size, p.groups), dim3(128),
                           (size_t)ctas * 4 * sizeof(float), s, (const float*)a.part_o, (const float*)a.part_m,
                           (const float*)a.part_l, (const int32_t*)a.prefix, p.d_out, p.groups, p.group_size, ctas * 4, a.e_steps));
  return RI_OK;
}

}  // namespace

int launch_attend(const ri_wave_layer& p, const Layout& L, cudaStream_t s) {
  return p.dtype == RI_BF16 ? launch<RI_BF16>(p, L, s) : launch<RI_F16>(p, L, s);
}

}  // namespace ri_wave
