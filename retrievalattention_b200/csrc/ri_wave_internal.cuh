// Shared by the three stages of the fused decode path (scan, select, attend): tile constants,
// the carving of the caller's scratch buffer, and the stage launchers.
#pragma once

#include "ri_common.cuh"

namespace ri_wave {

constexpr int kScanTile = 256;      // centroids per scan CTA (4 warps x 2 rounds x 4 n-tiles of 8)
constexpr int kSelectCluster = 8;   // CTAs (one thread-block cluster) cooperating on one group's selection
constexpr int kSelectThreads = 256;
constexpr int kMaxHeads = 8;        // GQA group size limit (N dimension of the PV MMA)
constexpr int kAttendMaxCtas = 512; // persistent attend CTAs (2 per SM) the scratch is sized for; 4 warps each
constexpr int kAttendMaxGroups = 4096;

// Phase markers of the single-kernel path.  They compile to nothing; a timing build may define RI_FT(k)
// before this header to stamp a clock at each marker.
#ifndef RI_FT
#define RI_FT(k)
#endif

struct Layout {
  int64_t counters, scores, tile_max, tile_sum, dist_keys, est_ids, est_w, est_s2, rows, n_exact, total;
  int e_pad, n_tiles;
};

inline Layout make_layout(const ri_wave_layer& p) {
  Layout L;
  const int64_t G = p.groups;
  // Per-group strides of the estimation lists are whole 128-byte lines: in the single-kernel path a
  // list is written and read inside one launch, and an SM's L1 must never hold a line that another
  // group's cluster is still going to write.
  L.e_pad = (int)ri_align_up(p.n_estimate > 0 ? p.n_estimate : 1, 32);
  L.n_tiles = (p.n_centroids + kScanTile - 1) / kScanTile;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = ri_align_up(off + bytes, 256); return o; };
  L.counters = take(G * 4);   // reserved word per group at the front (unused by the kernels)
  L.scores = take(G * p.group_size * (int64_t)p.n_centroids * 4);
  L.tile_max = take(G * kMaxHeads * (int64_t)L.n_tiles * 4);
  L.tile_sum = take(G * kMaxHeads * (int64_t)L.n_tiles * 4);
  L.dist_keys = take(G * (int64_t)p.n_centroids * 2);
  L.est_ids = take(G * L.e_pad * 4);
  L.est_w = take(G * L.e_pad * 4);
  L.est_s2 = take(G * kMaxHeads * (int64_t)L.e_pad * 4);
  L.rows = take(G * (int64_t)p.max_exact_rows * 4);
  L.n_exact = take(G * 4);
  L.total = off;
  return L;
}

// Each launcher enqueues one stage on `s` and returns an ri_status.
int launch_scan(const ri_wave_layer& p, const Layout& L, cudaStream_t s);
int launch_select(const ri_wave_layer& p, const Layout& L, cudaStream_t s);
// `eb` (optional): attend over a dense execution buffer instead of the cluster-contiguous store.
struct ExecBuffer { const void* keys; const void* values; int64_t stride; const int32_t* lengths; float* lse_out; };
// `gather` (optional): also store the output into every rank's gather buffer (several GPUs).
int launch_attend(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ExecBuffer* eb = nullptr,
                  const ri_wave_gather* gather = nullptr);
int launch_weighted_decoding(const void* q, const void* k, const void* v, const void* weights, const int32_t* seqlens,
                             const void* prev_out, const float* prev_lse, void* out, float* lse_out, int groups,
                             int group_size, int64_t stride, int dtype, cudaStream_t s);
// scan + select + attend as one kernel (one 8-CTA cluster per group).
int launch_fused(const ri_wave_layer& p, const Layout& L, cudaStream_t s, const ri_wave_gather* gather = nullptr);
int launch_gather_wait(const ri_wave_gather& g, cudaStream_t s);
bool fused_supported(const ri_wave_layer& p);   // geometries the single kernel covers (others run the three stages)

}  // namespace ri_wave
