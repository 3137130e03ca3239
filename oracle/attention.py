"""CPU restatement of the weighted flash decoding calls and of the whole decode
``compute`` step.  TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Parity unpinned for ``weighted_flash_decoding``: its source
(git+https://github.com/Starmys/flash-attention@weighted, README.md:27, no commit
pin) is not available.  The arithmetic below is flash decoding with a per-key
weight on the softmax denominator, which is what the operands at the two call
sites imply (cache_hub/retroinfer_cache.py:611-617: key = centroid, value =
per-cluster value SUM, weight = cluster size; :666-674: exact keys/values, merge
with a previous (out, lse) pair), evaluated in fp32.  What can be checked is checked against the
flash-attn library the operator was forked from (tests/test_oracle_attention_gpu.py): the
unweighted case, the merge, and the weighted case as attention over tokens that carry their
centroid as key.
"""
from __future__ import annotations

import math

import torch

from . import score_select


def weighted_flash_decoding(q, k, v, weights=None, *, previous_out=None, previous_lse=None,
                            cache_seqlens=None, return_softmax_lse=False, out_dtype=None):
    """``q`` [G, 1, gs, d]; ``k``/``v`` [G, L, 1, d]; ``weights`` [G, 1, 1, L] or None;
    ``cache_seqlens`` [G] int or None; ``previous_out`` [G, 1, gs, d],
    ``previous_lse`` [G, gs, 1] (natural log).

    ``out = sum_j e^{s_j} v_j / sum_j w_j e^{s_j}``, ``lse = log sum_j w_j e^{s_j}``,
    then the log-sum-exp merge with the previous partial result."""
    g, _, gs, d = q.shape
    length = k.shape[1]
    qf = q.float().reshape(g, gs, d)
    kf = k.float().reshape(g, length, d)
    vf = v.float().reshape(g, length, d)
    s = torch.bmm(qf, kf.transpose(1, 2)) / math.sqrt(d)          # [G, gs, L]
    if cache_seqlens is not None:
        valid = torch.arange(length)[None, :] < cache_seqlens.reshape(g, 1).long()
        s = s.masked_fill(~valid[:, None, :], float("-inf"))
    w = torch.ones((g, 1, length)) if weights is None else weights.float().reshape(g, 1, length)
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(s - m)
    denom = (w * e).sum(-1, keepdim=True)
    num = torch.bmm(e, vf)                                         # [G, gs, d]
    lse = m + torch.log(denom)                                      # [G, gs, 1]
    out = num / denom
    out = torch.where(denom > 0, out, torch.zeros_like(out))
    if previous_out is not None:
        p_lse = previous_lse.float().reshape(g, gs, 1)
        p_out = previous_out.float().reshape(g, gs, d)
        new_lse = torch.logaddexp(lse, p_lse)
        out = out * torch.exp(lse - new_lse) + p_out * torch.exp(p_lse - new_lse)
        lse = new_lse
    out = out.reshape(g, 1, gs, d).to(out_dtype or q.dtype)
    if return_softmax_lse:
        return out, lse
    return out


def surviving_clusters(ranked_ids: torch.Tensor, sizes: torch.Tensor, page_size: int, buffer_pages: int):
    """The overflow rule of ``BufferManager::batch_access``
    (library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp:207-216): walk the
    retrieved clusters in rank order and stop at the first one that would push the
    cumulative page count past ``buffer_pages``.  Returns the kept prefix length."""
    pages = 0
    keep = 0
    for cid in ranked_ids.tolist():
        pages += (int(sizes[cid]) + page_size - 1) // page_size
        if pages > buffer_pages:
            break
        keep += 1
    return keep


def compute(q, centroids, value_sum, cluster_size_dtype, mask, sizes, offsets, csr_keys, csr_values,
            steady_keys, steady_values, static_len, nprobe, max_compute, page_size, buffer_pages,
            return_parts=False, select_q=None):
    """One decode attention step for one layer, cache_hub/retroinfer_cache.py:549-697,
    with every cluster read from the cluster-contiguous store (which is what the
    execution buffer holds after ``gather_copy_and_concat``, :642-648, whether the
    pages came from the host list or the GPU page cache).

    q [B, 1, Hq, d]; centroids/value_sum [G, C, d]; cluster_size_dtype [G, C] (bf16);
    mask [G, C] bool; sizes [G, C] int32; offsets [G, C+1] int32;
    csr_keys/values [G, N, d]; steady_keys/values [G, S_max, d].
    ``select_q`` (same shape as q): the query the clusters are searched with when it is not the attending query —
    ``use_cluster_estimation`` searches a layer's clusters one layer early with an estimate of its query (:582-595)
    and attends them with the real one (:611-617, :666-674).
    Returns out [B, 1, Hq, d] in q.dtype."""
    g, c, d = centroids.shape
    b, _, hq, _ = q.shape
    gs = hq * b // g
    qg = q.reshape(g, gs, d)
    dist = score_select.cluster_distance(qg if select_q is None else select_q.reshape(g, gs, d), centroids, mask)
    ret_ids, est_ids = score_select.select_clusters(dist, nprobe, max_compute)
    e = est_ids.shape[1]
    out = torch.empty((g, 1, gs, d), dtype=q.dtype)
    kept = []
    for gi in range(g):
        qi = qg[gi].reshape(1, 1, gs, d)
        if e > 0:
            ids = est_ids[gi].long()
            es_out, es_lse = weighted_flash_decoding(
                qi, centroids[gi, ids].reshape(1, e, 1, d), value_sum[gi, ids].reshape(1, e, 1, d),
                cluster_size_dtype[gi, ids].reshape(1, 1, 1, e), return_softmax_lse=True)
        else:
            es_out, es_lse = None, None
        keep = surviving_clusters(ret_ids[gi], sizes[gi], page_size, buffer_pages)
        kept.append(keep)
        rows_k = [steady_keys[gi, :static_len]]
        rows_v = [steady_values[gi, :static_len]]
        for cid in ret_ids[gi, :keep].tolist():
            s0, s1 = int(offsets[gi, cid]), int(offsets[gi, cid + 1])
            rows_k.append(csr_keys[gi, s0:s1])
            rows_v.append(csr_values[gi, s0:s1])
        ek = torch.cat(rows_k, 0)
        ev = torch.cat(rows_v, 0)
        out[gi] = weighted_flash_decoding(
            qi, ek.reshape(1, -1, 1, d), ev.reshape(1, -1, 1, d),
            previous_out=es_out, previous_lse=es_lse)[0]
    out = out.reshape(b, 1, hq, d)
    if return_parts:
        return out, {"dist": dist, "retrieval": ret_ids, "estimation": est_ids, "kept": kept}
    return out


def full_attention_fp32(q, keys, values):
    """Dense softmax attention in fp32 over every token (accuracy yard-stick only)."""
    g, gs, d = q.shape
    s = torch.bmm(q.float(), keys.float().transpose(1, 2)) / math.sqrt(d)
    p = torch.softmax(s, dim=-1)
    return torch.bmm(p, values.float())
