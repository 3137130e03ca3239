"""CPU restatement of the reference's segmented inner-product k-means.
TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows cache_hub/kmeans.py:224-259 (``segment_k_means``) and the three Triton
kernels it drives (:6-49 assign, :52-80 update, :176-202 value sum, :128-152
inverted lists), plus the caller's centring and meta-index rounding
(cache_hub/retroinfer_cache.py:416-432).
"""
from __future__ import annotations

import torch


def initial_centroid_indices(num_tokens: int, num_centroids: int) -> torch.Tensor:
    """kmeans.py:234-236 — evaluated in float32, then truncated to int64."""
    idx = torch.arange(num_centroids, dtype=torch.float32) * (num_tokens / num_centroids)
    idx += num_tokens / num_centroids / 2
    return idx.to(torch.int64)


def assign(data: torch.Tensor, centroids: torch.Tensor, chunk: int = 16384) -> torch.Tensor:
    """kmeans.py:34-47 — argmax of the inner product, fp32 accumulation, the
    first maximum wins (strict ``>`` across centroid blocks, leftmost inside one)."""
    z, n, _ = data.shape
    out = torch.empty((z, n), dtype=torch.int32)
    cf = centroids.float().transpose(1, 2)
    for s in range(0, n, chunk):
        ip = torch.bmm(data[:, s:s + chunk].float(), cf)
        out[:, s:s + chunk] = torch.argmax(ip, dim=-1).to(torch.int32)
    return out


def train_step(data: torch.Tensor, centroids: torch.Tensor, normalize: bool):
    """One Lloyd iteration, kmeans.py:83-125.  Returns (centroids, max_idx, counts).

    Centroid = fp32 member sum / count (:73-76), optionally L2-normalised (:77-78),
    stored in the key dtype only where count > 0 (:75, :80)."""
    z, n, d = data.shape
    c = centroids.shape[1]
    max_idx = assign(data, centroids)
    data_sum = torch.zeros((z, c, d), dtype=torch.float32)
    counts = torch.zeros((z, c), dtype=torch.int32)
    for b in range(z):
        data_sum[b].index_add_(0, max_idx[b].long(), data[b].float())
        counts[b] = torch.bincount(max_idx[b].long(), minlength=c).to(torch.int32)
    x = data_sum / counts[..., None].float()
    if normalize:
        x = x / torch.sqrt(torch.sum(x * x, dim=-1, keepdim=True))
    new = torch.where(counts[..., None] > 0, x.to(centroids.dtype), centroids)
    return new, max_idx, counts


def value_sum(value: torch.Tensor, max_idx: torch.Tensor, num_centroids: int) -> torch.Tensor:
    """kmeans.py:205-221 — fp32 accumulation, cast to the value dtype at the end."""
    z, n, d = value.shape
    out = torch.zeros((z, num_centroids, d), dtype=torch.float32)
    for b in range(z):
        out[b].index_add_(0, max_idx[b].long(), value[b].float())
    return out.to(value.dtype)


def reverse_index(max_idx: torch.Tensor, num_centroids: int):
    """kmeans.py:155-173 — dense inverted lists.  The reference's intra-cluster
    order is the arrival order of atomics; here members are in ascending token order."""
    z, n = max_idx.shape
    sizes = torch.zeros((z, num_centroids), dtype=torch.int32)
    for b in range(z):
        sizes[b] = torch.bincount(max_idx[b].long(), minlength=num_centroids).to(torch.int32)
    width = int(sizes.max().item())
    clusters = torch.zeros((z, num_centroids, width), dtype=torch.int32)
    for b in range(z):
        order = torch.argsort(max_idx[b].long(), stable=True)
        starts = torch.cumsum(sizes[b].long(), 0) - sizes[b].long()
        sorted_cluster = max_idx[b].long()[order]
        slot = torch.arange(n) - starts[sorted_cluster]
        clusters[b, sorted_cluster, slot] = order.to(torch.int32)
    return clusters, sizes


def segment_k_means(key: torch.Tensor, value: torch.Tensor, num_centroids: int,
                    num_iters: int = 10, num_segments: int = 1, return_assignments: bool = False):
    """kmeans.py:224-259.  ``key`` is already mean-centred by the caller.

    Iterations 1..num_iters-1 run per segment (contiguous token ranges of
    ``N // num_segments`` tokens, ``C // num_segments`` centroids each, tail tokens
    ignored, :240-246) with normalised centroids; the last iteration assigns every
    token against all centroids and takes the plain mean (:248-250)."""
    groups, n, d = key.shape
    idx = initial_centroid_indices(n, num_centroids)
    centroids = torch.index_select(key, 1, idx)
    assert num_centroids % num_segments == 0
    n_seg = n // num_segments
    c_seg = num_centroids // num_segments
    data = key[:, :n_seg * num_segments].reshape(-1, n_seg, d)
    centroids = centroids.reshape(-1, c_seg, d)
    for _ in range(num_iters - 1):
        centroids, _, _ = train_step(data, centroids, normalize=True)
    centroids = centroids.reshape(groups, num_centroids, d)
    centroids, max_idx, _ = train_step(key, centroids, normalize=False)
    vsum = value_sum(value, max_idx, num_centroids)
    clusters, sizes = reverse_index(max_idx, num_centroids)
    if return_assignments:
        return centroids, vsum, clusters, sizes, max_idx
    return centroids, vsum, clusters, sizes


def build_meta_index(keys: torch.Tensor, values: torch.Tensor, num_centroids: int,
                     num_segments: int, num_iters: int = 10):
    """The caller's wrapping, cache_hub/retroinfer_cache.py:416-432: k-means on
    ``keys - mean(keys)`` (both in the key dtype), stored centroids = centroid + mean,
    ``mask = size == 0``, sizes additionally stored in the key dtype.

    ``keys``/``values``: ``[kv_heads, N, d]``.  Returns a dict."""
    mean_key = torch.mean(keys, dim=1, keepdim=True)
    cen, vsum, clusters, sizes, max_idx = segment_k_means(
        keys - mean_key, values, num_centroids, num_iters, num_segments, return_assignments=True)
    return {
        "centroids": cen + mean_key,
        "value_sum": vsum,
        "mask": sizes == 0,
        "cluster_size": sizes,
        "cluster_size_dtype": sizes.to(keys.dtype),
        "clusters": clusters,
        "assignments": max_idx,
        "mean_key": mean_key,
        "centroids_centred": cen,
    }


def organize_kv(keys: torch.Tensor, values: torch.Tensor, clusters: torch.Tensor, sizes: torch.Tensor):
    """library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp:513-567 —
    cluster-contiguous re-layout: cluster ``i`` starts at the exclusive prefix sum of
    the sizes (:534-539) and holds its members in inverted-list order (:561-565)."""
    z, n, d = keys.shape
    out_k = torch.zeros_like(keys)
    out_v = torch.zeros_like(values)
    starts = torch.zeros((z, sizes.shape[1] + 1), dtype=torch.int32)
    starts[:, 1:] = torch.cumsum(sizes, 1)
    for b in range(z):
        for c in range(sizes.shape[1]):
            m = int(sizes[b, c])
            if m:
                ids = clusters[b, c, :m].long()
                s = int(starts[b, c])
                out_k[b, s:s + m] = keys[b, ids]
                out_v[b, s:s + m] = values[b, ids]
    return out_k, out_v, starts
