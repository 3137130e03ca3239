"""Host-side handle of one layer's wave index, bound to the fused decode kernels.

The tensors live in HBM in the layout the kernels read directly:

* meta index  — ``centroids``/``value_sum`` ``[G, C, 128]``, ``cluster_size`` ``[G, C]`` in the
  KV dtype (as the reference stores it, cache_hub/retroinfer_cache.py:212-227, :432), plus the
  exact integer ``cluster_count`` ``[G, C]`` and CSR ``cluster_offset`` ``[G, C+1]``;
* cluster-contiguous KV — ``keys``/``values`` ``[G, N, 128]`` (the reference's
  ``list_keys``/``list_values``, :264-274, which it keeps in pinned host memory);
* steady zone — ``[G, S, 128]`` sink + recent + generated tokens (:83-92).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib


@dataclass
class WaveShape:
    groups: int
    group_size: int
    n_centroids: int
    nprobe: int
    n_estimate: int
    page_size: int
    buffer_pages: int
    tokens_per_group: int
    steady_stride: int
    dtype: torch.dtype = torch.bfloat16

    @property
    def max_exact_rows(self) -> int:
        return self.buffer_pages * self.page_size

    def fill(self, p: _lib.WaveLayer) -> None:
        p.groups, p.group_size, p.n_centroids = self.groups, self.group_size, self.n_centroids
        p.nprobe, p.n_estimate = self.nprobe, self.n_estimate
        p.page_size, p.buffer_pages = self.page_size, self.buffer_pages
        p.dtype = _lib.dtype_code(self.dtype)
        p.tokens_per_group = self.tokens_per_group
        p.steady_stride = self.steady_stride
        p.max_exact_rows = self.max_exact_rows

    def scratch_bytes(self) -> int:
        p = _lib.WaveLayer()
        self.fill(p)
        n = _lib.lib.ri_wave_scratch_bytes(C.byref(p))
        if n < 0:
            raise RuntimeError(f"ri_wave_scratch_bytes: {_lib.lib.ri_last_error().decode()}")
        return int(n)


def new_scratch(shape: WaveShape, device) -> torch.Tensor:
    """Zero-filled scratch for ``ri_wave_decode_layer`` (shareable by all layers of a stream)."""
    return torch.zeros(shape.scratch_bytes(), dtype=torch.uint8, device=device)


class WaveIndexLayer:
    """One layer's index + KV store with a prepared parameter block for the C ABI."""

    def __init__(self, shape: WaveShape, *, centroids, value_sum, cluster_size, cluster_count, cluster_offset,
                 keys, values, steady_keys, steady_values, static_len, scratch, want_ids: bool = False,
                 host_tier: bool = False):
        self.shape = shape
        dev = centroids.device
        g, c = shape.groups, shape.n_centroids
        assert centroids.shape == (g, c, 128) and value_sum.shape == (g, c, 128)
        assert cluster_size.shape == (g, c) and cluster_size.dtype == shape.dtype
        assert cluster_count.shape == (g, c) and cluster_count.dtype == torch.int32
        assert cluster_offset.shape == (g, c + 1) and cluster_offset.dtype == torch.int32
        # host tier: `keys`/`values` are the execution buffers; the cluster store itself is in host memory
        self.host_tier = host_tier
        assert keys.shape == (g, shape.tokens_per_group, 128) and values.shape == keys.shape
        assert steady_keys.shape == (g, shape.steady_stride, 128) and steady_values.shape == steady_keys.shape
        assert static_len.dtype == torch.int32 and static_len.numel() == 1
        assert scratch.numel() >= shape.scratch_bytes()
        self.t = dict(centroids=centroids, value_sum=value_sum, cluster_size=cluster_size,
                      cluster_count=cluster_count, cluster_offset=cluster_offset, keys=keys, values=values,
                      steady_keys=steady_keys, steady_values=steady_values, static_len=static_len,
                      scratch=scratch)
        for k, v in self.t.items():
            assert v.is_cuda and v.is_contiguous(), k
        self.pending_kv = None
        self.retrieved_ids = self.retrieved_kept = self.estimated_ids = None
        if want_ids:
            self.retrieved_ids = torch.zeros((g, shape.nprobe), dtype=torch.int64, device=dev)
            self.retrieved_kept = torch.zeros((g,), dtype=torch.int32, device=dev)
            self.estimated_ids = torch.zeros((g, max(shape.n_estimate, 1)), dtype=torch.int64, device=dev)
        p = _lib.WaveLayer()
        shape.fill(p)
        p.d_centroids, p.d_value_sum = centroids.data_ptr(), value_sum.data_ptr()
        p.d_cluster_size, p.d_cluster_count = cluster_size.data_ptr(), cluster_count.data_ptr()
        p.d_cluster_offset = cluster_offset.data_ptr()
        p.d_keys, p.d_values = keys.data_ptr(), values.data_ptr()
        p.d_steady_keys, p.d_steady_values = steady_keys.data_ptr(), steady_values.data_ptr()
        p.d_static_len = static_len.data_ptr()
        p.d_scratch = scratch.data_ptr()
        p.d_retrieved_ids = _lib.ptr(self.retrieved_ids)
        p.d_retrieved_kept = _lib.ptr(self.retrieved_kept)
        p.d_estimated_ids = _lib.ptr(self.estimated_ids)
        self.params = p

    def _bind(self, q: torch.Tensor, out: torch.Tensor) -> None:
        s = self.shape
        assert q.is_cuda and q.is_contiguous() and q.dtype == s.dtype and q.numel() == s.groups * s.group_size * 128
        assert out.is_cuda and out.is_contiguous() and out.dtype == s.dtype and out.numel() == q.numel()
        self.params.d_q, self.params.d_out = q.data_ptr(), out.data_ptr()
        kv, self.pending_kv = self.pending_kv, None
        if kv is None:
            self.params.d_new_keys = self.params.d_new_values = None
        else:                      # this step's rows: the decode call appends them itself (one launch less)
            self.params.d_new_keys, self.params.d_new_values = kv[0].data_ptr(), kv[1].data_ptr()
            self._kv_alive = kv    # until the next call

    def append_with_next_compute(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Hand this step's key/value rows ``[G, 128]`` (any shape with that many elements) to the next
        ``compute`` call, which stores them at row ``static_len - 1`` of the steady zone before attending."""
        s = self.shape
        assert k.is_cuda and k.is_contiguous() and k.dtype == s.dtype and k.numel() == s.groups * 128
        assert v.is_cuda and v.is_contiguous() and v.dtype == s.dtype and v.numel() == k.numel()
        self.pending_kv = (k, v)

    def compute(self, q: torch.Tensor, out: torch.Tensor | None = None, gather=None) -> torch.Tensor:
        """scan + select + attend (one kernel) on the current stream.  ``q``: [B, 1, Hq, 128] (or [G, gs, 128]).
        ``gather`` (a ``_lib.WaveGather``): the kernel also stores the output into every rank's gather
        buffer and raises this rank's flags there (several GPUs, see ``head_shard.PeerGather``)."""
        if out is None:
            out = torch.empty_like(q)
        self._bind(q, out)
        if gather is None:
            _lib.check(_lib.lib.ri_wave_decode_layer(C.byref(self.params), _lib.current_stream()), "ri_wave_decode_layer")
        else:
            _lib.check(_lib.lib.ri_wave_decode_layer_gather(C.byref(self.params), C.byref(gather), _lib.current_stream()),
                       "ri_wave_decode_layer_gather")
        return out

    def compute_staged(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """The same step as three stage kernels (scan, select, attend) instead of the single kernel
        ``compute`` launches — profiling one stage at a time, and a cross-check of the two forms."""
        if out is None:
            out = torch.empty_like(q)
        for name in ("scan", "select", "attend"):
            self.stage(name, q, out)
        return out

    def compute_static(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``compute`` without caller scratch, for hosts that must not allocate device memory (a
        server whose pool already owns all of HBM, or a loop that bans cudaMalloc because it stalls
        the device).  Uses the library's built-in 16 MiB scratch; larger geometries raise.  All
        calls share that array: do not let two of them overlap on the GPU.  Call it once at
        start-up, outside stream capture, so the array's address is resolved."""
        if out is None:
            out = torch.empty_like(q)
        self._bind(q, out)
        _lib.check(_lib.lib.ri_wave_decode_layer_static(C.byref(self.params), _lib.current_stream()),
                   "ri_wave_decode_layer_static")
        return out

    def attend_buffer(self, q: torch.Tensor, out: torch.Tensor, exec_keys: torch.Tensor, exec_values: torch.Tensor,
                      valid_lengths: torch.Tensor) -> torch.Tensor:
        """Host tier: attend over execution buffers ``[G, stride, 128]`` (steady zone ++ retrieved pages),
        using the estimation set the select stage left in the scratch."""
        self._bind(q, out)
        assert exec_keys.is_cuda and exec_keys.is_contiguous() and exec_values.shape == exec_keys.shape
        assert valid_lengths.dtype == torch.int32 and valid_lengths.is_cuda
        _lib.check(_lib.lib.ri_wave_attend_buffer(C.byref(self.params), exec_keys.data_ptr(), exec_values.data_ptr(),
                                                  exec_keys.shape[1], valid_lengths.data_ptr(), _lib.current_stream()),
                   "ri_wave_attend_buffer")
        return out

    def stage(self, name: str, q: torch.Tensor, out: torch.Tensor) -> None:
        """Run one stage alone (``scan``/``select``/``attend``) — tests and profiling."""
        self._bind(q, out)
        fn = getattr(_lib.lib, "ri_wave_" + name)
        _lib.check(fn(C.byref(self.params), _lib.current_stream()), "ri_wave_" + name)

    def views(self) -> dict:
        """Typed views into the scratch after ``select`` (tests)."""
        v = _lib.WaveViews()
        _lib.check(_lib.lib.ri_wave_scratch_views(C.byref(self.params), C.byref(v)), "ri_wave_scratch_views")
        s, sc = self.shape, self.t["scratch"]
        base = sc.data_ptr()

        def view(addr, nbytes, dtype, shape):
            return sc[addr - base: addr - base + nbytes].view(dtype).view(shape)

        return {
            "scores": view(v.d_scores, s.groups * s.group_size * s.n_centroids * 4, torch.float32,
                           (s.groups, s.group_size, s.n_centroids)),
            "dist_keys": view(v.d_dist_keys, s.groups * s.n_centroids * 2, torch.int16, (s.groups, s.n_centroids)),
            "exact_rows": view(v.d_exact_rows, s.groups * s.max_exact_rows * 4, torch.int32,
                               (s.groups, s.max_exact_rows)),
            "n_exact": view(v.d_n_exact, s.groups * 4, torch.int32, (s.groups,)),
        }


def steady_append(k: torch.Tensor, v: torch.Tensor, steady_keys: torch.Tensor, steady_values: torch.Tensor,
                  position: torch.Tensor) -> None:
    """Write this step's K/V ([B, 1, Hk, 128]) at row ``position[0]`` of every group's steady zone."""
    groups, stride = steady_keys.shape[0], steady_keys.shape[1]
    assert k.is_contiguous() and v.is_contiguous() and k.numel() == groups * 128
    _lib.check(_lib.lib.ri_steady_append(k.data_ptr(), v.data_ptr(), steady_keys.data_ptr(),
                                         steady_values.data_ptr(), position.data_ptr(), groups, stride,
                                         _lib.current_stream()), "ri_steady_append")
