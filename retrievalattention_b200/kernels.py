"""The operator surface of the reference's ``retroinfer_kernels`` package
(library/retroinfer/retroinfer_kernels/__init__.py:1-3), bound to ``libri_b200.so``.

``ThreadPool`` / ``WaveBufferCPU`` keep the constructor and method names of the pybind classes
(wave_buffer_cpu.cpp:822-849).
"""
from __future__ import annotations

import torch

from . import _lib


class ThreadPool:
    """Placeholder with the reference's interface (``ThreadPool(n).get()``, wave_buffer_cpu.cpp:17-35).
    Each ``WaveBufferCPU`` here owns its workers, so the handle only carries the thread count."""

    def __init__(self, num_threads: int):
        self.num_threads = int(num_threads)

    def get(self):
        return self


class WaveBufferCPU:
    """Host-side LRU page cache of one layer (wave_buffer_cpu.cpp:261-816)."""

    def __init__(self, batch_size, group_num, dim, nprobe, block_size, n_centroids, final_n_centroids, buffer_size,
                 capacity, threads, pool=None):
        if dim != 128:
            raise ValueError("head_dim must be 128")
        self.batch_size, self.group_num, self.n_centroids = batch_size, group_num, n_centroids
        self._h = _lib.lib.ri_wb_create(batch_size, group_num, nprobe, block_size, n_centroids, final_n_centroids,
                                        buffer_size, capacity, threads)
        if not self._h:
            raise ValueError(_lib.lib.ri_last_error().decode())
        self._keep = []
        self._destroy = _lib.lib.ri_wb_destroy      # bound now: module globals may be gone at interpreter exit

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        destroy = getattr(self, "_destroy", None)
        if h and destroy is not None:
            destroy(h)

    def set_indices(self, hit_block_ids, hit_block_sizes, hit_block_sizes_cumsum, hit_block_nums, miss_block_ids,
                    miss_block_sizes, miss_block_sizes_cumsum, miss_block_nums, update_buffer_indices,
                    update_block_sizes, update_cache_indices, update_block_nums, searched_clusters):
        ts = [hit_block_ids, hit_block_sizes, hit_block_sizes_cumsum, hit_block_nums, miss_block_ids, miss_block_sizes,
              miss_block_sizes_cumsum, miss_block_nums, update_buffer_indices, update_block_sizes, update_cache_indices,
              update_block_nums]
        for t in ts:
            assert t.dtype == torch.int32 and t.device.type == "cpu" and t.is_contiguous()
        assert searched_clusters.dtype == torch.int64 and searched_clusters.device.type == "cpu"
        self._keep = ts + [searched_clusters]          # the library keeps raw pointers (as the reference does)
        _lib.check(_lib.lib.ri_wb_set_indices(self._h, *[t.data_ptr() for t in self._keep]), "ri_wb_set_indices")

    def set_kv(self, ivf_key, ivf_value, input_keys, input_values):
        """Accepted for compatibility: the cluster-contiguous copy is produced on the GPU by the
        clustering pass, not by host memcpy (wave_buffer_cpu.cpp:488-507, :545-567)."""
        return None

    def async_construction(self, clusters, cluster_size, batch_idx):
        """Register one request's cluster sizes ([group_num, n_centroids] int32); the inverted lists
        are not needed on the host (wave_buffer_cpu.cpp:592-616)."""
        cs = cluster_size.to(torch.int32).cpu().contiguous()
        _lib.check(_lib.lib.ri_wb_set_clusters(self._h, int(batch_idx), cs.data_ptr()), "ri_wb_set_clusters")

    def construction_sync(self):
        return None

    def update_kv(self, update_keys, update_values, clusters, cluster_size):
        cs = cluster_size.to(torch.int32).cpu().contiguous()
        _lib.check(_lib.lib.ri_wb_append_clusters(self._h, cs.data_ptr(), cs.shape[1]), "ri_wb_append_clusters")

    def batch_access(self) -> int:
        rc = _lib.lib.ri_wb_batch_access(self._h)
        if rc < 0:
            _lib.check(rc, "ri_wb_batch_access")
        return rc

    def sync(self):
        _lib.check(_lib.lib.ri_wb_sync(self._h), "ri_wb_sync")


def _p(t: torch.Tensor) -> int:
    """Address of a contiguous CUDA or pinned-host tensor."""
    assert t.is_contiguous(), "operator arguments must be contiguous"
    assert t.is_cuda or t.is_pinned(), "host tensors must be pinned (they are read through UVA)"
    return t.data_ptr()


def batch_gemm_softmax(A, B, D, Norm, Sum, Softmax, batch_count, m, n, k, alpha=1.0, beta=0.0):
    """``retroinfer_kernels.batch_gemm_softmax`` (src/batch_gemm_softmax.cu:201-208): ``D = alpha * A @ B^T`` and
    ``Softmax = softmax(D, -1)``, both in the dtype of ``A``; ``Norm``/``Sum`` are float32 scratch of
    ``batch_count * m * ceil(n / 256)`` elements.  On the current stream."""
    for t in (A, B, D, Norm, Sum, Softmax):
        if not (t.is_cuda and t.is_contiguous()):
            raise ValueError("batch_gemm_softmax: tensors must be contiguous CUDA tensors")
    if B.dtype != A.dtype or D.dtype != A.dtype or Softmax.dtype != A.dtype:
        raise TypeError("batch_gemm_softmax: A, B, D and Softmax must share one dtype")
    if Norm.dtype != torch.float32 or Sum.dtype != torch.float32:
        raise TypeError("batch_gemm_softmax: Norm and Sum must be float32")
    blocks = (n + 255) // 256
    if A.numel() != batch_count * m * k or B.numel() != batch_count * n * k or D.numel() != batch_count * m * n or \
            Softmax.numel() != D.numel() or Norm.numel() < batch_count * m * blocks or Sum.numel() < batch_count * m * blocks:
        raise ValueError("batch_gemm_softmax: tensor sizes do not match batch_count, m, n, k")
    _lib.check(_lib.lib.ri_batch_gemm_softmax(_p(A), _p(B), _p(D), _p(Norm), _p(Sum), _p(Softmax), batch_count, m, n, k,
                                              float(alpha), float(beta), _lib.dtype_code(A.dtype), _lib.current_stream()),
               "ri_batch_gemm_softmax")


def weighted_flash_decoding(q, k, v, weights=None, *, previous_out=None, previous_lse=None, cache_seqlens=None,
                            return_softmax_lse=False):
    """The operator the reference imports as ``weighted_flash_decoding`` (call sites
    cache_hub/retroinfer_cache.py:611-617, :666-674).  ``q`` [G, 1, gs, 128]; ``k``/``v`` [G, L, 1, 128];
    ``weights`` [G, 1, 1, L] (softmax-denominator weight of every row) or None; ``cache_seqlens`` [G] int32 or None
    (all L rows); ``previous_out`` [G, 1, gs, 128] with ``previous_lse`` [G, gs, 1] (float32, natural log): a partial
    result to merge with.  Returns ``out`` [G, 1, gs, 128], and ``lse`` [G, gs, 1] when asked."""
    g, one, gs, d = q.shape
    length = k.shape[1]
    if one != 1 or d != 128 or k.shape != (g, length, 1, d) or v.shape != k.shape:
        raise ValueError("weighted_flash_decoding: expected q [G,1,gs,128] and k, v [G,L,1,128]")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if cache_seqlens is None:
        cache_seqlens = torch.full((g,), length, dtype=torch.int32, device=q.device)
    cache_seqlens = cache_seqlens.to(torch.int32).contiguous()
    if weights is not None:
        weights = weights.to(q.dtype).reshape(g, length).contiguous()
    if (previous_out is None) != (previous_lse is None):
        raise ValueError("weighted_flash_decoding: previous_out and previous_lse go together")
    if previous_out is not None:
        previous_out = previous_out.to(q.dtype).reshape(g, gs, d).contiguous()
        previous_lse = previous_lse.to(torch.float32).reshape(g, gs).contiguous()
    out = torch.empty_like(q)
    lse = torch.empty((g, gs, 1), dtype=torch.float32, device=q.device) if return_softmax_lse else None
    _lib.check(_lib.lib.ri_weighted_flash_decoding(
        _p(q), _p(k), _p(v), None if weights is None else _p(weights), _p(cache_seqlens),
        None if previous_out is None else _p(previous_out), None if previous_lse is None else _p(previous_lse),
        _p(out), None if lse is None else _p(lse), g, gs, length, _lib.dtype_code(q.dtype), _lib.current_stream()),
        "ri_weighted_flash_decoding")
    return (out, lse) if return_softmax_lse else out


def gather_copy_vectors(key_data, key_buffer, value_data, value_buffer, src_metadata, dst_metadata, data_offsets,
                        groups, data_length, buffer_length, index_size, copy_start, copy_num):
    """gather_copy.cu:25-96 (same argument list)."""
    assert key_data.element_size() == 2 and key_data.shape[-1] == 128 and data_offsets.dtype == torch.int64
    _lib.check(_lib.lib.ri_gather_copy_vectors(
        _p(key_data), _p(key_buffer), _p(value_data), _p(value_buffer), _p(src_metadata), _p(dst_metadata),
        _p(data_offsets), groups, data_length, buffer_length, index_size, copy_start, copy_num, _lib.current_stream()),
        "ri_gather_copy_vectors")


def gather_copy_and_concat(key_data1, key_data2, key_data3, key_buffer, value_data1, value_data2, value_data3,
                           value_buffer, data_offsets2, data_copy_sizes2, buffer_offsets2, copy_chunks2, data_offsets3,
                           data_copy_sizes3, buffer_offsets3, copy_chunks3, valid_lengths, groups, data_length1,
                           data_length2, data_length3, buffer_length, offset_length, copy_vectors1):
    """gather_copy.cu:100-212 (same argument list)."""
    assert key_data1.element_size() == 2 and key_data1.shape[-1] == 128
    idx = (data_offsets2, data_copy_sizes2, buffer_offsets2, copy_chunks2, data_offsets3, data_copy_sizes3,
           buffer_offsets3, copy_chunks3, valid_lengths)
    assert all(t.dtype == torch.int32 for t in idx)
    _lib.check(_lib.lib.ri_gather_copy_and_concat(
        _p(key_data1), _p(key_data2), _p(key_data3), _p(key_buffer), _p(value_data1), _p(value_data2), _p(value_data3),
        _p(value_buffer), *[_p(t) for t in idx], groups, data_length1, data_length2, data_length3, buffer_length,
        offset_length, copy_vectors1, _lib.current_stream()), "ri_gather_copy_and_concat")


def gather_copy_and_scatter(key_data, key_buffer, value_data, value_buffer, s_offsets, copy_sizes, d_offsets,
                            copy_chunks, groups, data_length, buffer_length, offset_length, s_copy_start):
    """gather_copy.cu:216-283 (same argument list)."""
    assert all(t.dtype == torch.int32 for t in (s_offsets, copy_sizes, d_offsets, copy_chunks))
    _lib.check(_lib.lib.ri_gather_copy_and_scatter(
        _p(key_data), _p(key_buffer), _p(value_data), _p(value_buffer), _p(s_offsets), _p(copy_sizes), _p(d_offsets),
        _p(copy_chunks), groups, data_length, buffer_length, offset_length, s_copy_start, _lib.current_stream()),
        "ri_gather_copy_and_scatter")
