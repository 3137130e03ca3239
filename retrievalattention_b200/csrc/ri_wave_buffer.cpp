// Host-side wave buffer: per-(request, kv-head) LRU cache of GPU pages for clusters whose KV
// lives in pinned host memory, with the reference's access/update semantics
// (library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp: ClusterDescriptor :38-45,
// BufferManager::batch_access :190-257, BufferManager::batch_update :102-188, parse_clusters
// :513-542, the descriptor part of update_kv_func :646-684).
//
// Differences by design: plain C ABI (no torch, no pybind); free pages are handed out from a
// stack, so page ids are deterministic (the reference's come from an unordered_set); the KV
// re-layout itself (organize_kv) is done on the GPU by ri_kmeans_build, so this class only keeps
// descriptors.  Worker threads are plain std::threads, not pinned to cores.
#include <algorithm>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <functional>
#include <list>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include "ri_b200.h"

int ri_fail(int status, const char* fmt, ...);

namespace {

struct Cluster {
  bool cached = false;
  int start = 0;       // first row in the group's cluster-contiguous host list
  int pages = 0;
  int last_size = 0;   // rows in the last page
  std::vector<int> page_ids;
  std::list<int64_t>::iterator lru_pos;
};

// One group's page cache.
class GroupCache {
 public:
  GroupCache(int capacity, int page, int max_pages) : capacity_(capacity), page_(page), max_pages_(max_pages) {
    free_.reserve(capacity);
    for (int i = capacity - 1; i >= 0; --i) free_.push_back(i);   // pop_back hands out 0, 1, 2, ...
  }

  std::vector<Cluster> clusters;

  // Walk the retrieved clusters in rank order; stop at the first one that would exceed the page
  // budget (:207-216).  Miss -> host rows per page (:219-235); hit -> GPU page ids (:237-253).
  void access(const int64_t* keys, int n, int* hit_ids, int* hit_sizes, int* hit_cum, int* n_hit_pages, int* miss_ids,
              int* miss_sizes, int* miss_cum, int* n_miss_pages, bool* overflow) {
    hits_.clear();
    misses_.clear();
    int h = 0, m = 0, hp = 0, mp = 0, considered = 0;
    *overflow = false;
    for (int i = 0; i < n; ++i) {
      const int64_t key = keys[i];
      if (key < 0 || key >= (int64_t)clusters.size()) continue;   // never index outside the table
      Cluster& c = clusters[key];
      considered += c.pages;
      if (considered > max_pages_) { *overflow = true; break; }
      if (c.pages == 0) continue;   // an empty cluster carries no rows (the reference is undefined here, :167)
      if (!c.cached) {
        misses_.push_back(key);
        int row = c.start;
        for (int j = 0; j < c.pages; ++j) {
          const int sz = j == c.pages - 1 ? c.last_size : page_;
          miss_ids[mp] = row; miss_sizes[mp] = sz; miss_cum[mp] = m;
          m += sz; row += page_; ++mp;
        }
      } else {
        hits_.push_back(key);
        for (int j = 0; j < c.pages; ++j) {
          const int sz = j == c.pages - 1 ? c.last_size : page_;
          hit_ids[hp] = c.page_ids[j]; hit_sizes[hp] = sz; hit_cum[hp] = h;
          h += sz; ++hp;
        }
      }
    }
    *n_hit_pages = hp;
    *n_miss_pages = mp;
  }

  // Refresh the LRU order of the hits (in reverse, :106-114), admit misses in order while they fit
  // the capacity (:119-130), evict least-recently-used clusters until enough pages are free
  // (:140-142), hand out pages (:147-177).
  void update(int* cache_ids, int* sizes, int* buffer_offsets, int* n_pages) {
    for (int i = (int)hits_.size() - 1; i >= 0; --i) {
      Cluster& c = clusters[hits_[i]];
      lru_.erase(c.lru_pos);
      lru_.push_front(hits_[i]);
      c.lru_pos = lru_.begin();
    }
    int admit = 0, need = 0;
    for (int64_t key : misses_) {
      if (need + clusters[key].pages <= capacity_) { ++admit; need += clusters[key].pages; } else break;
    }
    int np = 0, cum = 0;
    if (admit > 0) {
      while ((int)free_.size() < need && !lru_.empty()) {
        Cluster& victim = clusters[lru_.back()];
        lru_.pop_back();
        for (int id : victim.page_ids) free_.push_back(id);
        victim.page_ids.clear();
        victim.cached = false;
      }
      for (int i = 0; i < admit; ++i) {
        Cluster& c = clusters[misses_[i]];
        c.cached = true;
        c.page_ids.resize(c.pages);
        for (int j = 0; j < c.pages; ++j) {
          const int id = free_.back();
          free_.pop_back();
          const int sz = j == c.pages - 1 ? c.last_size : page_;
          c.page_ids[j] = id;
          cache_ids[np] = id; sizes[np] = sz; buffer_offsets[np] = cum;
          cum += sz; ++np;
        }
        lru_.push_front(misses_[i]);
        c.lru_pos = lru_.begin();
      }
    }
    hits_.clear();
    misses_.clear();
    *n_pages = np;
  }

 private:
  int capacity_, page_, max_pages_;
  std::vector<int> free_;
  std::list<int64_t> lru_;
  std::vector<int64_t> hits_, misses_;
};

// Minimal worker pool: run f(i) for i in [0, n) on the workers; wait() blocks until idle.
class Pool {
 public:
  explicit Pool(int n) {
    for (int i = 0; i < std::max(1, n); ++i) workers_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    { std::lock_guard<std::mutex> l(m_); stop_ = true; }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  void submit(std::function<void()> f) {
    { std::lock_guard<std::mutex> l(m_); q_.push_back(std::move(f)); ++pending_; }
    cv_.notify_one();
  }
  void wait() {
    std::unique_lock<std::mutex> l(m_);
    idle_.wait(l, [this] { return pending_ == 0; });
  }

 private:
  void loop() {
    for (;;) {
      std::function<void()> f;
      {
        std::unique_lock<std::mutex> l(m_);
        cv_.wait(l, [this] { return stop_ || !q_.empty(); });
        if (stop_ && q_.empty()) return;
        f = std::move(q_.front());
        q_.erase(q_.begin());
      }
      f();
      { std::lock_guard<std::mutex> l(m_); if (--pending_ == 0) idle_.notify_all(); }
    }
  }
  std::vector<std::thread> workers_;
  std::vector<std::function<void()>> q_;
  std::mutex m_;
  std::condition_variable cv_, idle_;
  int pending_ = 0;
  bool stop_ = false;
};

}  // namespace

struct ri_wave_buffer {
  int batch, heads, groups, nprobe, page, n_centroids, final_n_centroids, buffer_pages, capacity;
  std::vector<GroupCache> caches;
  std::vector<int> rows_used;   // rows of the host list occupied per group
  Pool pool;
  int32_t *hit_ids = nullptr, *hit_sizes = nullptr, *hit_cum = nullptr, *hit_n = nullptr;
  int32_t *miss_ids = nullptr, *miss_sizes = nullptr, *miss_cum = nullptr, *miss_n = nullptr;
  int32_t *upd_buf = nullptr, *upd_sizes = nullptr, *upd_cache = nullptr, *upd_n = nullptr;
  const int64_t* searched = nullptr;
  int threads;
  bool update_pending = false;
  std::vector<uint8_t> overflowed;
  ri_wave_buffer(int b, int h, int np, int pg, int nc, int fnc, int bp, int cap, int th)
      : batch(b), heads(h), groups(b * h), nprobe(np), page(pg), n_centroids(nc), final_n_centroids(fnc),
        buffer_pages(bp), capacity(cap), rows_used(b * h, 0), pool(std::min(th, std::max(1, (b * h + 1) / 2))),
        threads(th), overflowed(b * h, 0) {
    caches.reserve(groups);
    for (int g = 0; g < groups; ++g) caches.emplace_back(cap, pg, bp);
  }
  template <class F>
  void for_groups(F f) {   // at least two groups per task, as the reference schedules (:334-336)
    const int tasks = std::min(threads, std::max(1, (groups + 1) / 2));
    const int per = (groups + tasks - 1) / tasks;
    for (int t = 0; t < tasks; ++t)
      pool.submit([=] { for (int g = t * per; g < std::min(groups, (t + 1) * per); ++g) f(g); });
  }
};

static void add_clusters(GroupCache& gc, int* rows_used, const int32_t* sizes, int n, int page) {
  for (int i = 0; i < n; ++i) {
    Cluster c;
    const int s = sizes[i];
    c.start = *rows_used;
    c.pages = (s + page - 1) / page;
    c.last_size = s % page == 0 ? page : s % page;
    gc.clusters.push_back(std::move(c));
    *rows_used += s;
  }
}

extern "C" ri_wave_buffer* ri_wb_create(int32_t batch_size, int32_t group_num, int32_t nprobe, int32_t block_size,
                                        int32_t n_centroids, int32_t final_n_centroids, int32_t buffer_size,
                                        int32_t capacity, int32_t threads) {
  if (batch_size <= 0 || group_num <= 0 || nprobe <= 0 || block_size <= 0 || n_centroids <= 0 ||
      final_n_centroids < n_centroids || buffer_size <= 0 || capacity <= 0 || threads <= 0) {
    ri_fail(RI_ERR_INVALID, "ri_wb_create: every size must be positive and final_n_centroids >= n_centroids");
    return nullptr;
  }
  return new (std::nothrow) ri_wave_buffer(batch_size, group_num, nprobe, block_size, n_centroids, final_n_centroids,
                                           buffer_size, capacity, threads);
}

extern "C" void ri_wb_destroy(ri_wave_buffer* wb) {
  if (wb) { wb->pool.wait(); delete wb; }
}

extern "C" int ri_wb_set_indices(ri_wave_buffer* wb, int32_t* hit_ids, int32_t* hit_sizes, int32_t* hit_cumsum,
                                 int32_t* hit_nums, int32_t* miss_ids, int32_t* miss_sizes, int32_t* miss_cumsum,
                                 int32_t* miss_nums, int32_t* update_buffer_indices, int32_t* update_sizes,
                                 int32_t* update_cache_indices, int32_t* update_nums, const int64_t* searched_clusters) {
  if (!wb || !hit_ids || !hit_sizes || !hit_cumsum || !hit_nums || !miss_ids || !miss_sizes || !miss_cumsum ||
      !miss_nums || !update_buffer_indices || !update_sizes || !update_cache_indices || !update_nums || !searched_clusters)
    return ri_fail(RI_ERR_INVALID, "ri_wb_set_indices: null pointer");
  wb->hit_ids = hit_ids; wb->hit_sizes = hit_sizes; wb->hit_cum = hit_cumsum; wb->hit_n = hit_nums;
  wb->miss_ids = miss_ids; wb->miss_sizes = miss_sizes; wb->miss_cum = miss_cumsum; wb->miss_n = miss_nums;
  wb->upd_buf = update_buffer_indices; wb->upd_sizes = update_sizes; wb->upd_cache = update_cache_indices;
  wb->upd_n = update_nums; wb->searched = searched_clusters;
  return RI_OK;
}

extern "C" int ri_wb_set_clusters(ri_wave_buffer* wb, int32_t batch_idx, const int32_t* cluster_sizes) {
  if (!wb || !cluster_sizes) return ri_fail(RI_ERR_INVALID, "ri_wb_set_clusters: null pointer");
  if (batch_idx < 0 || batch_idx >= wb->batch) return ri_fail(RI_ERR_INVALID, "ri_wb_set_clusters: batch_idx %d", batch_idx);
  wb->pool.wait();
  for (int h = 0; h < wb->heads; ++h) {
    const int g = batch_idx * wb->heads + h;
    wb->caches[g] = GroupCache(wb->capacity, wb->page, wb->buffer_pages);
    wb->caches[g].clusters.reserve(wb->final_n_centroids);
    wb->rows_used[g] = 0;
    add_clusters(wb->caches[g], &wb->rows_used[g], cluster_sizes + (int64_t)h * wb->n_centroids, wb->n_centroids, wb->page);
  }
  return RI_OK;
}

extern "C" int ri_wb_append_clusters(ri_wave_buffer* wb, const int32_t* cluster_sizes, int32_t n_new) {
  if (!wb || !cluster_sizes || n_new <= 0) return ri_fail(RI_ERR_INVALID, "ri_wb_append_clusters: bad argument");
  wb->pool.wait();
  for (int g = 0; g < wb->groups; ++g) {
    if ((int)wb->caches[g].clusters.size() + n_new > wb->final_n_centroids)
      return ri_fail(RI_ERR_INVALID, "ri_wb_append_clusters: more clusters than final_n_centroids=%d", wb->final_n_centroids);
    add_clusters(wb->caches[g], &wb->rows_used[g], cluster_sizes + (int64_t)g * n_new, n_new, wb->page);
  }
  return RI_OK;
}

extern "C" int ri_wb_batch_access(ri_wave_buffer* wb) {
  if (!wb || !wb->searched) return ri_fail(RI_ERR_STATE, "ri_wb_batch_access before ri_wb_set_indices");
  wb->pool.wait();
  const int64_t bs = wb->buffer_pages;
  wb->for_groups([wb, bs](int g) {
    bool of = false;
    wb->caches[g].access(wb->searched + (int64_t)g * wb->nprobe, wb->nprobe, wb->hit_ids + g * bs, wb->hit_sizes + g * bs,
                         wb->hit_cum + g * bs, wb->hit_n + g, wb->miss_ids + g * bs, wb->miss_sizes + g * bs,
                         wb->miss_cum + g * bs, wb->miss_n + g, &of);
    wb->overflowed[g] = of;
  });
  wb->pool.wait();
  // the LRU update runs in the background until ri_wb_sync (:801-806)
  wb->for_groups([wb, bs](int g) {
    wb->caches[g].update(wb->upd_cache + g * bs, wb->upd_sizes + g * bs, wb->upd_buf + g * bs, wb->upd_n + g);
  });
  wb->update_pending = true;
  int n = 0;
  for (uint8_t o : wb->overflowed) n += o;
  return n;   // number of groups whose retrieval was cut by the page budget (the reference prints a warning)
}

// After ri_wb_batch_access: the worker threads copy every missed page of every group from the cluster store in host
// memory into a staging area in host memory, group g's pages back to back from row 0 of its slot (page j at row
// miss_cumsum[g][j]) — the layout gather_copy_and_concat reads when it is given miss_cumsum as the source offsets.
// Blocks until the copies are done; *max_rows_out = the largest number of staged rows of any group.
extern "C" int ri_wb_stage_misses(ri_wave_buffer* wb, const void* h_src_keys, const void* h_src_values,
                                  int64_t src_rows_per_group, void* h_stage_keys, void* h_stage_values,
                                  int64_t stage_rows_per_group, int32_t row_bytes, int32_t* max_rows_out) {
  if (!wb || !wb->miss_ids || !h_src_keys || !h_src_values || !h_stage_keys || !h_stage_values || !max_rows_out)
    return ri_fail(RI_ERR_INVALID, "ri_wb_stage_misses: null pointer");
  if (row_bytes <= 0 || src_rows_per_group <= 0 || stage_rows_per_group <= 0)
    return ri_fail(RI_ERR_INVALID, "ri_wb_stage_misses: bad sizes");
  const int64_t bs = wb->buffer_pages;
  std::vector<int> rows(wb->groups, 0);
  int* rows_p = rows.data();
  const char *sk = static_cast<const char*>(h_src_keys), *sv = static_cast<const char*>(h_src_values);
  char *dk = static_cast<char*>(h_stage_keys), *dv = static_cast<char*>(h_stage_values);
  wb->for_groups([=](int g) {
    const int n = wb->miss_n[g];
    int total = 0;
    for (int j = 0; j < n; ++j) {
      const int64_t src = wb->miss_ids[g * bs + j], dst = wb->miss_cum[g * bs + j];
      const int sz = wb->miss_sizes[g * bs + j];
      if (src < 0 || src + sz > src_rows_per_group || dst < 0 || dst + sz > stage_rows_per_group) continue;   // never copy outside
      memcpy(dk + (g * stage_rows_per_group + dst) * row_bytes, sk + (g * src_rows_per_group + src) * row_bytes, (size_t)sz * row_bytes);
      memcpy(dv + (g * stage_rows_per_group + dst) * row_bytes, sv + (g * src_rows_per_group + src) * row_bytes, (size_t)sz * row_bytes);
      total = std::max(total, (int)(dst + sz));
    }
    rows_p[g] = total;
  });
  wb->pool.wait();
  *max_rows_out = *std::max_element(rows.begin(), rows.end());
  return RI_OK;
}

extern "C" int ri_wb_sync(ri_wave_buffer* wb) {
  if (!wb) return ri_fail(RI_ERR_INVALID, "ri_wb_sync: null");
  wb->pool.wait();
  wb->update_pending = false;
  return RI_OK;
}

extern "C" int64_t ri_wb_rows_used(const ri_wave_buffer* wb, int32_t group) {
  if (!wb || group < 0 || group >= wb->groups) return RI_ERR_INVALID;
  return wb->rows_used[group];
}
