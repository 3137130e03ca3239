"""CPU restatement of centroid scoring and cluster selection.
TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows the reference's own kernel-test oracle
(library/retroinfer/test/test_batch_gemm_softmax.py:9-18: bmm -> /sqrt(d) -> softmax)
with the rounding points of the CUTLASS kernels it checks
(library/retroinfer/retroinfer_kernels/src/batch_gemm_softmax.cu:94-101 — the GEMM
epilogue stores ``bf16(alpha*acc)``; batch_gemm_softmax.h:226-243 — the softmax
kernel re-reads those bf16 scores and stores ``bf16(exp(s-max)*inv_sum)``), then the
selection in cache_hub/retroinfer_cache.py:572-575.
"""
from __future__ import annotations

import math

import torch


def batch_gemm_softmax(q: torch.Tensor, centroids: torch.Tensor, alpha: float | None = None):
    """``q`` [G, gs, d], ``centroids`` [G, C, d] (bf16/fp16).  Returns (scores, probs)
    in the input dtype, both [G, gs, C]."""
    if alpha is None:
        alpha = 1.0 / math.sqrt(q.shape[-1])
    acc = torch.bmm(q.float(), centroids.float().transpose(1, 2))
    scores = (acc * alpha).to(q.dtype)
    s = scores.float()
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    inv = 1.0 / e.sum(dim=-1, keepdim=True)
    probs = (e * inv).to(q.dtype)
    return scores, probs


def cluster_distance(q: torch.Tensor, centroids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """retroinfer_cache.py:569-573 — sum of the per-head probabilities over the GQA
    group (a bf16 tensor reduction: fp32 accumulate, one rounding), empty clusters
    forced to the most negative finite value of the dtype."""
    _, probs = batch_gemm_softmax(q, centroids)
    dist = torch.sum(probs, dim=1)
    dist = dist.masked_fill(mask, torch.finfo(q.dtype).min)
    return dist


def select_clusters(dist: torch.Tensor, nprobe: int, max_compute: int):
    """retroinfer_cache.py:574-575, :601-605 — one sorted top-``max_compute``;
    ranks [0, nprobe) are retrieved exactly, ranks [nprobe, max_compute) are
    estimated from their centroid.  Ties are broken towards the lower cluster id
    (the reference leaves the order among equal keys unspecified)."""
    order = torch.argsort(dist.float(), dim=-1, descending=True, stable=True)
    top = order[:, :max_compute]
    return top[:, :nprobe].contiguous(), top[:, nprobe:].contiguous()


def selection_matches(dist: torch.Tensor, got: torch.Tensor, k: int, band: float = 1e-3) -> bool:
    """Set parity with the tie rule: ``got`` (ids, any order) must contain every
    cluster whose distance is more than ``band`` above the k-th largest and nothing
    more than ``band`` below it; size must be k with no duplicates."""
    ok = True
    for g in range(dist.shape[0]):
        d = dist[g].float()
        ids = got[g].long()
        if ids.numel() != k or torch.unique(ids).numel() != k:
            return False
        kth = torch.topk(d, k).values[-1]
        must = torch.nonzero(d > kth + band).flatten()
        chosen = torch.zeros_like(d, dtype=torch.bool)
        chosen[ids] = True
        ok &= bool(chosen[must].all())
        ok &= bool((d[ids] >= kth - band).all())
    return ok
