"""Prefill clustering on the GPU, behind the reference's ``cache_hub/kmeans.py`` interface.

``segment_k_means`` keeps the reference signature and return values
(cache_hub/kmeans.py:224-259); ``build_index`` is the form the cache uses: it also centres the
keys, adds the mean back to the centroids and writes K/V in cluster-contiguous order, all on the
device (cache_hub/retroinfer_cache.py:416-436 and the CPU re-layout of wave_buffer_cpu.cpp:513-567).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


def _run(keys, values, num_centroids, num_iters, num_segments, center, want_layout, want_lists=True):
    assert keys.is_cuda and values.is_cuda, "k-means runs on the GPU only"
    assert keys.dim() == 3 and keys.shape == values.shape and keys.shape[-1] == 128, "expected [groups, tokens, 128]"
    keys, values = keys.contiguous(), values.contiguous()
    z, n, d = keys.shape
    dev, dt = keys.device, keys.dtype
    out = {
        "centroids": torch.empty((z, num_centroids, d), dtype=dt, device=dev),
        "value_sum": torch.empty((z, num_centroids, d), dtype=dt, device=dev),
        "cluster_size": torch.empty((z, num_centroids), dtype=dt, device=dev),
        "cluster_count": torch.empty((z, num_centroids), dtype=torch.int32, device=dev),
        "cluster_offset": torch.empty((z, num_centroids + 1), dtype=torch.int32, device=dev),
        "error": torch.zeros((1,), dtype=torch.int32, device=dev),
    }
    if want_lists:
        out["assign"] = torch.empty((z, n), dtype=torch.int32, device=dev)
        out["order"] = torch.empty((z, n), dtype=torch.int32, device=dev)
    if want_layout:
        out["keys"] = torch.empty_like(keys)
        out["values"] = torch.empty_like(values)
    if center:
        out["mean_key"] = torch.empty((z, 1, d), dtype=dt, device=dev)
    p = _lib.KMeans()
    p.groups, p.n_tokens, p.n_centroids, p.n_segments, p.n_iters = z, n, num_centroids, num_segments, num_iters
    p.dtype, p.center = _lib.dtype_code(dt), int(center)
    need = _lib.lib.ri_kmeans_scratch_bytes(C.byref(p))
    if need < 0:
        raise ValueError(f"ri_kmeans: {_lib.lib.ri_last_error().decode()}")
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    p.d_keys, p.d_values = keys.data_ptr(), values.data_ptr()
    p.d_centroids, p.d_value_sum = out["centroids"].data_ptr(), out["value_sum"].data_ptr()
    p.d_cluster_size = out["cluster_size"].data_ptr()
    p.d_cluster_count, p.d_cluster_offset = out["cluster_count"].data_ptr(), out["cluster_offset"].data_ptr()
    p.d_assign = _lib.ptr(out.get("assign"))
    p.d_order = _lib.ptr(out.get("order"))
    p.d_keys_out, p.d_values_out = _lib.ptr(out.get("keys")), _lib.ptr(out.get("values"))
    p.d_mean_key = _lib.ptr(out.get("mean_key"))
    p.d_scratch, p.d_error = scratch.data_ptr(), out["error"].data_ptr()
    _lib.check(_lib.lib.ri_kmeans_build(C.byref(p), _lib.current_stream()), "ri_kmeans_build")
    out["_scratch"] = scratch     # keep alive until the stream has consumed it
    return out


def build_index(keys: torch.Tensor, values: torch.Tensor, num_centroids: int, num_segments: int = 1,
                num_iters: int = 10, want_lists: bool = False) -> dict:
    """Index of one request's layer: ``keys``/``values`` ``[kv_heads, N, 128]`` (uncentred).

    Returns device tensors: ``centroids`` (mean added back), ``value_sum``, ``cluster_size`` (KV
    dtype), ``cluster_count``, ``cluster_offset``, cluster-contiguous ``keys``/``values``,
    ``mean_key``, ``error`` (1 if a device-side wait timed out) and, on request, ``assign``/``order``."""
    return _run(keys, values, num_centroids, num_iters, num_segments, True, True, want_lists)


def segment_k_means(key: torch.Tensor, value: torch.Tensor, num_centroids: int, num_iters: int = 10,
                    num_segments: int = 1):
    """Reference interface (cache_hub/kmeans.py:224-259): ``key`` is already centred.

    Returns ``(centroids, value_sum, clusters, cluster_size)`` with ``clusters`` the dense inverted
    lists ``[groups, num_centroids, max_cluster_size]`` (members in ascending token order; the
    reference's order inside a cluster is the arrival order of its atomics)."""
    r = _run(key, value, num_centroids, num_iters, num_segments, False, False, True)
    z, n = r["order"].shape
    count, offset = r["cluster_count"], r["cluster_offset"]
    width = int(count.max().item())               # the reference synchronises here too (kmeans.py:124)
    clusters = torch.zeros((z, num_centroids, max(width, 1)), dtype=torch.int32, device=key.device)
    cl_sorted = torch.gather(r["assign"], 1, r["order"].long()).long()
    slot = torch.arange(n, device=key.device)[None, :] - torch.gather(offset[:, :-1].long(), 1, cl_sorted)
    clusters[torch.arange(z, device=key.device)[:, None], cl_sorted, slot] = r["order"]
    return r["centroids"], r["value_sum"], clusters, count
