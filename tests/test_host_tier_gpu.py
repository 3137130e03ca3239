"""Host tier (``kv_on_host=True``): cluster-contiguous KV in pinned host memory, LRU page cache on the
GPU, execution buffer assembled per step — the reference's own arrangement
(cache_hub/retroinfer_cache.py:558-697) on this library's kernels.  Outputs must match the oracle
within max-abs 2e-2 / mean-abs 2e-3 and agree with the HBM-resident tier; repeated queries must be
served from the GPU page cache."""
import pytest
import torch

from oracle import attention as oat
from retrievalattention_b200.config import generate_config
from retrievalattention_b200.synthetic import make_kv, make_queries

pytestmark = pytest.mark.gpu


def build(kv_on_host, batch, layers, kv_heads, q_heads, seq_len, max_new, miss_path="pull", ahead=False):
    from retrievalattention_b200.cache_hub import retroinfer_cache

    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=2)
    mapping = {str(l): "cuda:0" for l in range(layers)}
    cache = retroinfer_cache([0] * batch, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,
                             mapping, max_new, num_gpus=1, model_size=8, kv_on_host=kv_on_host, miss_path=miss_path,
                             use_cluster_estimation=ahead, **cfg.as_kwargs())
    for b in range(batch):
        for l in range(layers):
            k, v = make_kv(kv_heads, seq_len, 128, seed=100 * l + b, device="cuda")
            cache.prefill_update_kv_cache(None, k, v, l, b)
            cache.sync(l, b)
    cache.prepare_cache()
    return cache, cfg


# pull: a copy kernel on a side stream reads the missed pages from the pinned store while the first attention pass runs;
# staged: the host's worker threads copy them into a pinned staging area and one strided copy sends them up on the side
# stream; uva: the reference's pattern (blocking id copy, the copy kernel on the main stream, one attention pass)
@pytest.mark.parametrize("miss_path", ["pull", "staged", "uva"])
def test_host_tier_matches_oracle_and_hbm_tier(miss_path):
    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 2, 2, 8, 2048 + 68, 8
    host, cfg = build(True, batch, layers, kv_heads, q_heads, seq_len, max_new, miss_path)
    hbm, _ = build(False, batch, layers, kv_heads, q_heads, seq_len, max_new)
    g = batch * kv_heads
    for l in range(layers):   # same index, same cluster-contiguous rows, different memory
        assert host.list_keys[l].is_pinned() and not host.list_keys[l].is_cuda
        assert torch.equal(host.list_keys[l].view(torch.int16), hbm.list_keys[l].cpu().view(torch.int16))
        assert torch.equal(host.cluster_count[l], hbm.cluster_count[l])
    hits_seen = 0
    for step in range(5):
        for l in range(layers):
            k_new = make_queries(batch, kv_heads, 128, seed=7000 + 10 * step + l, device="cuda")
            v_new = make_queries(batch, kv_heads, 128, seed=8000 + 10 * step + l, device="cuda")
            # steps 0-1 and 3-4 reuse a query, so their retrieved clusters repeat
            q = make_queries(batch, q_heads, 128, seed=9000 + 10 * (step // 2 if step != 2 else 77) + l, device="cuda")
            host.decode_update_kv_cache(k_new, v_new, l)
            hbm.decode_update_kv_cache(k_new, v_new, l)
            out_host = host.compute(q, l).clone()
            out_hbm = hbm.compute(q, l).clone()
            torch.cuda.synchronize()
            ref = oat.compute(q.cpu(), hbm.centroids[l].cpu(), hbm.value_sum[l].cpu(), hbm.cluster_size[l].cpu(),
                              hbm.centroids_mask[l].cpu(), hbm.cluster_count[l].cpu(), hbm.cluster_offset[l].cpu(),
                              hbm.list_keys[l].cpu().view(g, -1, 128), hbm.list_values[l].cpu().view(g, -1, 128),
                              hbm.steady_zone_keys[l].cpu().view(g, -1, 128),
                              hbm.steady_zone_values[l].cpu().view(g, -1, 128), 68 + step + 1, cfg.nprobe,
                              cfg.max_compute_cluster_num, cfg.cache_unit_size, hbm.buffer_size)
            for name, out in (("host", out_host), ("hbm", out_hbm)):
                err = (out.cpu().float() - ref.float()).abs()
                assert err.max() <= 2e-2 and err.mean() <= 2e-3, (name, step, l, float(err.max()), float(err.mean()))
            assert (out_host.float() - out_hbm.float()).abs().max() <= 2e-2
            hit_n, miss_n = host.page_lists[l][3], host.page_lists[l][7]
            assert int((hit_n + miss_n).min()) > 0
            if step in (1, 4):
                hits_seen += int(hit_n.sum())
            # the execution buffer holds steady rows + every retrieved row
            lens = host._per_device["cuda:0"]["valid_lengths"].cpu()
            assert int(lens.min()) >= 68 + step + 1
    assert hits_seen > 0, "repeated queries should be served from the GPU page cache"


def test_host_tier_searches_and_pulls_one_layer_ahead():
    """Host tier with ``use_cluster_estimation``: the call for layer l searches layer l + 1 with ``queries_next``, walks
    its page lists and starts the pull of its missed pages; layer l + 1 then attends those clusters with its real query.
    Against the oracle with the search query and the attending query kept apart, three layers (both execution buffers
    in use at once), repeated queries so that later steps are served from the GPU page cache."""
    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 3, 2, 8, 2048 + 68, 8
    host, cfg = build(True, batch, layers, kv_heads, q_heads, seq_len, max_new, "pull", ahead=True)
    hbm, _ = build(False, batch, layers, kv_heads, q_heads, seq_len, max_new)
    g = batch * kv_heads
    hits_seen = 0
    for step in range(4):
        qs = [make_queries(batch, q_heads, 128, seed=9000 + 10 * (step // 2) + l, device="cuda") for l in range(layers)]
        # layer 1 is searched ahead with a noisy estimate of its query, layer 2 with the exact one
        noise = torch.randn(qs[1].shape, generator=torch.Generator().manual_seed(step // 2)).cuda()
        guess = [None, (qs[1].float() + 0.3 * noise).to(torch.bfloat16), qs[2]]
        for l in range(layers):
            k_new = make_queries(batch, kv_heads, 128, seed=7000 + 10 * step + l, device="cuda")
            v_new = make_queries(batch, kv_heads, 128, seed=8000 + 10 * step + l, device="cuda")
            host.decode_update_kv_cache(k_new, v_new, l)
            hbm.decode_update_kv_cache(k_new, v_new, l)
            out = host.compute(qs[l], l, guess[l + 1] if l + 1 < layers else None).clone()
            hbm.compute(qs[l], l)
            torch.cuda.synchronize()
            ref = oat.compute(qs[l].cpu(), hbm.centroids[l].cpu(), hbm.value_sum[l].cpu(), hbm.cluster_size[l].cpu(),
                              hbm.centroids_mask[l].cpu(), hbm.cluster_count[l].cpu(), hbm.cluster_offset[l].cpu(),
                              hbm.list_keys[l].cpu().view(g, -1, 128), hbm.list_values[l].cpu().view(g, -1, 128),
                              hbm.steady_zone_keys[l].cpu().view(g, -1, 128),
                              hbm.steady_zone_values[l].cpu().view(g, -1, 128), 68 + step + 1, cfg.nprobe,
                              cfg.max_compute_cluster_num, cfg.cache_unit_size, hbm.buffer_size,
                              select_q=None if guess[l] is None else guess[l].cpu())
            err = (out.cpu().float() - ref.float()).abs()
            assert err.max() <= 2e-2 and err.mean() <= 2e-3, (step, l, float(err.max()), float(err.mean()))
            if step % 2 == 1:
                hits_seen += int(host.page_lists[l][3].sum())
    assert hits_seen > 0 and not any(host._ahead)
