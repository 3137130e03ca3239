"""The oracle's ``weighted_flash_decoding`` (source of the real operator not available: parity unpinned) tied to what IS
available: the flash-attn library the operator was forked from.

* without weights it must be plain flash decoding: output and log-sum-exp of ``flash_attn_with_kvcache``;
* the merge with a previous (out, lse) pair must reproduce attention over both halves at once;
* with weights: fed (centroid, value SUM, cluster size) — the operands of the estimation call,
  cache_hub/retroinfer_cache.py:611-617 — it must equal plain attention over a sequence in which every token of a
  cluster carries the centroid as its key and its own value, which is the reading of the operator that the call site
  implies (``out = sum_c e^{s_c} V_c / sum_c n_c e^{s_c}``).
"""
import pytest
import torch

from oracle import attention as oat

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


def library(q, k, v, lens=None):
    from flash_attn import flash_attn_with_kvcache

    out, lse = flash_attn_with_kvcache(q=q.cuda(), k_cache=k.cuda(), v_cache=v.cuda(),
                                       cache_seqlens=None if lens is None else lens.cuda().to(torch.int32),
                                       return_softmax_lse=True)
    return out.float().cpu(), lse.float().cpu()          # out [G, 1, gs, d]; lse [G, gs, 1]


def rand(*shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(DT)


def test_unweighted_oracle_is_flash_decoding():
    g, gs, length, d = 6, 4, 777, 128
    q, k, v = rand(g, 1, gs, d, seed=1), rand(g, length, 1, d, seed=2), rand(g, length, 1, d, seed=3)
    lens = torch.tensor([777, 1, 300, 512, 64, 700])
    ref, ref_lse = library(q, k, v, lens)
    out, lse = oat.weighted_flash_decoding(q, k, v, None, cache_seqlens=lens, return_softmax_lse=True)
    assert (out.float() - ref).abs().max() <= 2e-2
    assert (lse.float().reshape(g, gs) - ref_lse.reshape(g, gs)).abs().max() <= 2e-2


def test_merge_with_previous_result_is_attention_over_both_parts():
    g, gs, length, d = 4, 7, 600, 128
    q, k, v = rand(g, 1, gs, d, seed=4), rand(g, length, 1, d, seed=5), rand(g, length, 1, d, seed=6)
    ref, _ = library(q, k, v)
    first, lse = oat.weighted_flash_decoding(q, k[:, :250], v[:, :250], None, return_softmax_lse=True, out_dtype=torch.float32)
    both = oat.weighted_flash_decoding(q, k[:, 250:], v[:, 250:], None, previous_out=first, previous_lse=lse)
    assert (both.float() - ref).abs().max() <= 2e-2


def test_weighted_oracle_is_attention_over_tokens_that_carry_their_centroid():
    g, gs, d, clusters = 3, 4, 128, 40
    gen = torch.Generator().manual_seed(7)
    sizes = torch.randint(1, 9, (g, clusters), generator=gen)
    cent = rand(g, clusters, 1, d, seed=8)
    q = rand(g, 1, gs, d, seed=9)
    total = int(sizes.sum(1).max())
    keys = torch.zeros((g, total, 1, d), dtype=DT)
    vals = torch.zeros((g, total, 1, d), dtype=DT)
    vsum = torch.zeros((g, clusters, 1, d), dtype=torch.float32)
    lens = sizes.sum(1)
    for i in range(g):
        pos = 0
        for c in range(clusters):
            n = int(sizes[i, c])
            keys[i, pos:pos + n] = cent[i, c]
            tok = torch.randn((n, 1, d), generator=gen).to(DT)
            vals[i, pos:pos + n] = tok
            vsum[i, c] = tok.float().sum(0)
            pos += n
    ref, ref_lse = library(q, keys, vals, lens)
    out, lse = oat.weighted_flash_decoding(q, cent, vsum, sizes.reshape(g, 1, 1, clusters).float(), return_softmax_lse=True)
    assert (out.float() - ref).abs().max() <= 2e-2
    assert (lse.float().reshape(g, gs) - ref_lse.reshape(g, gs)).abs().max() <= 2e-2
