"""ctypes binding of ``libri_b200.so`` (the C ABI declared in ``include/ri_b200.h``).

There is no CPU fallback: importing this module without the built library raises, and every
wrapper raises ``RuntimeError`` with the library's message when a call fails.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# RI_B200_LIB names another build of the same library (e.g. one installed outside the package)
LIB_PATH = os.environ.get("RI_B200_LIB") or os.path.join(_PKG, "lib", "libri_b200.so")

RI_BF16, RI_F16 = 0, 1


class WaveLayer(C.Structure):
    """Mirror of ``struct ri_wave_layer``."""

    _fields_ = [
        ("groups", C.c_int32), ("group_size", C.c_int32), ("n_centroids", C.c_int32), ("nprobe", C.c_int32),
        ("n_estimate", C.c_int32), ("page_size", C.c_int32), ("buffer_pages", C.c_int32), ("dtype", C.c_int32),
        ("tokens_per_group", C.c_int64), ("steady_stride", C.c_int32), ("max_exact_rows", C.c_int32),
        ("d_centroids", C.c_void_p), ("d_value_sum", C.c_void_p), ("d_cluster_size", C.c_void_p),
        ("d_cluster_count", C.c_void_p), ("d_cluster_offset", C.c_void_p),
        ("d_keys", C.c_void_p), ("d_values", C.c_void_p),
        ("d_steady_keys", C.c_void_p), ("d_steady_values", C.c_void_p), ("d_static_len", C.c_void_p),
        ("d_q", C.c_void_p), ("d_out", C.c_void_p), ("d_scratch", C.c_void_p),
        ("d_retrieved_ids", C.c_void_p), ("d_retrieved_kept", C.c_void_p), ("d_estimated_ids", C.c_void_p),
        ("d_new_keys", C.c_void_p), ("d_new_values", C.c_void_p),
    ]


class WaveGather(C.Structure):
    """Mirror of ``struct ri_wave_gather``."""

    _fields_ = [
        ("n_ranks", C.c_int32), ("rank", C.c_int32), ("wait_limit_us", C.c_int32), ("reserved", C.c_int32),
        ("d_out_slots", C.c_void_p), ("d_flag_slots", C.c_void_p), ("d_flags", C.c_void_p),
        ("d_epoch", C.c_void_p), ("d_error", C.c_void_p), ("d_stamps", C.c_void_p),
    ]


class KMeans(C.Structure):
    """Mirror of ``struct ri_kmeans``."""

    _fields_ = [
        ("groups", C.c_int32), ("n_tokens", C.c_int32), ("n_centroids", C.c_int32), ("n_segments", C.c_int32),
        ("n_iters", C.c_int32), ("dtype", C.c_int32), ("center", C.c_int32), ("reserved", C.c_int32),
        ("d_keys", C.c_void_p), ("d_values", C.c_void_p), ("d_centroids", C.c_void_p), ("d_value_sum", C.c_void_p),
        ("d_cluster_size", C.c_void_p), ("d_cluster_count", C.c_void_p), ("d_cluster_offset", C.c_void_p),
        ("d_assign", C.c_void_p), ("d_order", C.c_void_p), ("d_keys_out", C.c_void_p), ("d_values_out", C.c_void_p),
        ("d_mean_key", C.c_void_p), ("d_scratch", C.c_void_p), ("d_error", C.c_void_p),
    ]


class WaveViews(C.Structure):
    _fields_ = [("d_scores", C.c_void_p), ("d_dist_keys", C.c_void_p), ("d_exact_rows", C.c_void_p),
                ("d_n_exact", C.c_void_p)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m retrievalattention_b200.build` "
            "(there is no CPU fallback for the wave-index kernels)")
    lib = C.CDLL(LIB_PATH)
    lib.ri_last_error.restype = C.c_char_p
    lib.ri_version.restype = C.c_int
    lib.ri_wave_scratch_bytes.restype = C.c_int64
    lib.ri_wave_scratch_bytes.argtypes = [C.POINTER(WaveLayer)]
    for name in ("ri_wave_decode_layer", "ri_wave_decode_layer_static", "ri_wave_scan", "ri_wave_select",
                 "ri_wave_attend", "ri_wave_rescore"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(WaveLayer), C.c_void_p]
    lib.ri_wave_test_local_cap.restype = C.c_int
    lib.ri_wave_test_local_cap.argtypes = [C.c_int]
    lib.ri_wave_attend_buffer.restype = C.c_int
    lib.ri_wave_attend_buffer.argtypes = [C.POINTER(WaveLayer), C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
    lib.ri_wave_decode_layer_gather.restype = C.c_int
    lib.ri_wave_decode_layer_gather.argtypes = [C.POINTER(WaveLayer), C.POINTER(WaveGather), C.c_void_p]
    lib.ri_wave_gather_wait.restype = C.c_int
    lib.ri_wave_gather_wait.argtypes = [C.POINTER(WaveGather), C.c_void_p]
    lib.ri_wave_scratch_views.restype = C.c_int
    lib.ri_wave_scratch_views.argtypes = [C.POINTER(WaveLayer), C.POINTER(WaveViews)]
    lib.ri_kmeans_scratch_bytes.restype = C.c_int64
    lib.ri_kmeans_scratch_bytes.argtypes = [C.POINTER(KMeans)]
    lib.ri_kmeans_build.restype = C.c_int
    lib.ri_kmeans_build.argtypes = [C.POINTER(KMeans), C.c_void_p]
    lib.ri_wb_create.restype = C.c_void_p
    lib.ri_wb_create.argtypes = [C.c_int32] * 9
    lib.ri_wb_destroy.restype = None
    lib.ri_wb_destroy.argtypes = [C.c_void_p]
    lib.ri_wb_set_indices.restype = C.c_int
    lib.ri_wb_set_indices.argtypes = [C.c_void_p] * 14
    lib.ri_wb_set_clusters.restype = C.c_int
    lib.ri_wb_set_clusters.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    lib.ri_wb_append_clusters.restype = C.c_int
    lib.ri_wb_append_clusters.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
    lib.ri_wb_batch_access.restype = C.c_int
    lib.ri_wb_batch_access.argtypes = [C.c_void_p]
    lib.ri_wb_sync.restype = C.c_int
    lib.ri_wb_sync.argtypes = [C.c_void_p]
    lib.ri_wb_stage_misses.restype = C.c_int
    lib.ri_wb_stage_misses.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                       C.c_int32, C.POINTER(C.c_int32)]
    lib.ri_stage_upload.restype = C.c_int
    lib.ri_stage_upload.argtypes = [C.c_void_p] * 4 + [C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
    lib.ri_wave_attend_buffer_lse.restype = C.c_int
    lib.ri_wave_attend_buffer_lse.argtypes = [C.POINTER(WaveLayer), C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
                                              C.c_void_p]
    lib.ri_wb_rows_used.restype = C.c_int64
    lib.ri_wb_rows_used.argtypes = [C.c_void_p, C.c_int32]
    lib.ri_batch_gemm_softmax.restype = C.c_int
    lib.ri_batch_gemm_softmax.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_float, C.c_float, C.c_int32, C.c_void_p]
    lib.ri_weighted_flash_decoding.restype = C.c_int
    lib.ri_weighted_flash_decoding.argtypes = [C.c_void_p] * 9 + [C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_void_p]
    lib.ri_gather_copy_vectors.restype = C.c_int
    lib.ri_gather_copy_vectors.argtypes = [C.c_void_p] * 7 + [C.c_int32] * 6 + [C.c_void_p]
    lib.ri_gather_copy_and_concat.restype = C.c_int
    lib.ri_gather_copy_and_concat.argtypes = ([C.c_void_p] * 17 + [C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                                                  C.c_int32, C.c_int32, C.c_void_p])
    lib.ri_gather_copy_and_scatter.restype = C.c_int
    lib.ri_gather_copy_and_scatter.argtypes = [C.c_void_p] * 8 + [C.c_int32] * 5 + [C.c_void_p]
    lib.ri_rmsnorm.restype = C.c_int
    lib.ri_rmsnorm.argtypes = [C.c_void_p] * 4 + [C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_void_p]
    lib.ri_rope_split.restype = C.c_int
    lib.ri_rope_split.argtypes = [C.c_void_p] * 6 + [C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_void_p]
    lib.ri_silu_and_mul.restype = C.c_int
    lib.ri_silu_and_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.ri_prefill_attn_scratch_bytes.restype = C.c_int64
    lib.ri_prefill_attn_scratch_bytes.argtypes = [C.c_int32] * 3
    lib.ri_prefill_attn.restype = C.c_int
    lib.ri_prefill_attn.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 6 + [C.c_void_p]
    lib.ri_steady_append.restype = C.c_int
    lib.ri_steady_append.argtypes = [C.c_void_p] * 5 + [C.c_int32, C.c_int32, C.c_void_p]
    return lib


lib = _load()


def check(rc: int, what: str = "libri_b200") -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {lib.ri_last_error().decode()}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return RI_BF16
    if dtype == torch.float16:
        return RI_F16
    raise TypeError(f"only bfloat16 and float16 are supported, got {dtype}")


def ptr(t: torch.Tensor | None) -> int | None:
    """Device (or pinned host) address of a contiguous tensor; None passes NULL."""
    if t is None:
        return None
    if not t.is_contiguous():
        raise ValueError("tensor passed to libri_b200 must be contiguous")
    return t.data_ptr()


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream
