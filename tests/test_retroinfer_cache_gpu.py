"""The drop-in ``retroinfer_cache`` driven the way the reference's model runtime drives it
(model_hub/LLM.py:57-62 prefill, :116-117 decode, :185 prepare), checked against the oracle.

The index itself is checked in test_kmeans_gpu.py; here the oracle consumes the index the cache
built (copied to the host) and must reproduce every decode step's attention output within
max-abs 2e-2 / mean-abs 2e-3."""
import pytest
import torch

from oracle import attention as oat
from retrievalattention_b200.config import generate_config
from retrievalattention_b200.synthetic import make_kv, make_queries

pytestmark = pytest.mark.gpu


def make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new, valid_start, dtype=torch.bfloat16, n_segment=2):
    from retrievalattention_b200.cache_hub import retroinfer_cache

    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=n_segment)
    mapping = {str(l): "cuda:0" for l in range(layers)}
    cache = retroinfer_cache(valid_start, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, dtype, mapping,
                             max_new, num_gpus=1, model_size=8, **cfg.as_kwargs())
    return cache, cfg


def test_prefill_then_decode_matches_oracle():
    from retrievalattention_b200.attn_hub import retroinfer_decode_attn

    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 2, 2, 8, 2048 + 68, 6
    valid_start = [0, 37]                      # second request is left-padded
    cache, cfg = make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new, valid_start)
    assert cache.buffer_size == max(cfg.nprobe * 4, 16) * 1 or cache.buffer_size > 0

    for b in range(batch):
        for l in range(layers):
            k, v = make_kv(kv_heads, seq_len, 128, seed=100 * l + b, device="cuda")
            q = torch.empty((1, seq_len, q_heads, 128), dtype=torch.bfloat16, device="cuda")
            rk, rv = cache.prefill_update_kv_cache(q, k, v, l, b)
            assert rk.shape[1] == seq_len - valid_start[b]
            cache.sync(l, b)
    cache.prepare_cache()
    assert cache.context == seq_len

    g = batch * kv_heads
    host = []
    for l in range(layers):
        host.append({
            "centroids": cache.centroids[l].cpu(), "value_sum": cache.value_sum[l].cpu(),
            "cluster_size": cache.cluster_size[l].cpu(), "mask": cache.centroids_mask[l].cpu(),
            "count": cache.cluster_count[l].cpu(), "offset": cache.cluster_offset[l].cpu(),
            "keys": cache.list_keys[l].cpu().view(g, -1, 128), "values": cache.list_values[l].cpu().view(g, -1, 128),
        })
        # masks agree with counts; the padded request clusters fewer tokens
        assert torch.equal(host[l]["mask"], host[l]["count"] == 0)
        sums = host[l]["count"].sum(1)
        assert sums[:kv_heads].eq(seq_len - 68).all() and sums[kv_heads:].eq(seq_len - 68 - 37).all()

    for step in range(3):
        for l in range(layers):
            k_new = make_queries(batch, kv_heads, 128, seed=7000 + 10 * step + l, device="cuda")
            v_new = make_queries(batch, kv_heads, 128, seed=8000 + 10 * step + l, device="cuda")
            q = make_queries(batch, q_heads, 128, seed=9000 + 10 * step + l, device="cuda")
            assert cache.decode_update_kv_cache(k_new, v_new, l) == (None, None)
            out = retroinfer_decode_attn(q, k_new, v_new, l, cache)
            assert out.shape == (batch, 1, q_heads, 128)
            static_len = 68 + step + 1
            h = host[l]
            ref = oat.compute(q.cpu(), h["centroids"], h["value_sum"], h["cluster_size"], h["mask"], h["count"],
                              h["offset"], h["keys"], h["values"],
                              cache.steady_zone_keys[l].cpu().view(g, -1, 128),
                              cache.steady_zone_values[l].cpu().view(g, -1, 128), static_len, cfg.nprobe,
                              cfg.max_compute_cluster_num, cfg.cache_unit_size, cache.buffer_size)
            err = (out.cpu().float() - ref.float()).abs()
            assert err.max() <= 2e-2 and err.mean() <= 2e-3, (step, l, float(err.max()), float(err.mean()))
        assert cache.static_pattern_total == 68 + step + 1
        assert cache.context == seq_len + step + 1
    # the appended tokens sit where the reference puts them (:539-540)
    assert torch.equal(cache.steady_zone_keys[0][:, :, 68 + 2].cpu(),
                       make_queries(batch, kv_heads, 128, seed=7000 + 20, device="cuda").cpu()[:, 0])


def test_decode_step_can_be_captured_in_a_graph():
    """No host synchronisation inside a decode step: the whole step replays as one CUDA graph
    while the steady zone grows (lengths are read on the device)."""
    batch, layers, kv_heads, q_heads, seq_len, max_new = 1, 2, 2, 8, 1024 + 68, 8
    cache, cfg = make_cache(batch, layers, kv_heads, q_heads, seq_len, max_new, [0], n_segment=1)
    for l in range(layers):
        k, v = make_kv(kv_heads, seq_len, 128, seed=l, device="cuda")
        cache.prefill_update_kv_cache(None, k, v, l, 0)
    cache.prepare_cache()
    q = [make_queries(batch, q_heads, 128, seed=50 + l, device="cuda") for l in range(layers)]
    kn = [make_queries(batch, kv_heads, 128, seed=60 + l, device="cuda") for l in range(layers)]
    outs = [torch.empty_like(q[0]) for _ in range(layers)]

    def step():
        for l in range(layers):
            cache.decode_update_kv_cache(kn[l], kn[l], l)
            outs[l].copy_(cache.compute(q[l], l))

    step()                                   # eager step 1
    eager2 = None
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):            # captured step (device state not advanced by capture)
        step()
    graph.replay()                           # step 2
    torch.cuda.synchronize()
    eager2 = [o.clone() for o in outs]
    assert int(cache._per_device["cuda:0"]["append_pos"].item()) == 68 + 2
    graph.replay()                           # step 3 attends one more row
    torch.cuda.synchronize()
    assert int(cache._per_device["cuda:0"]["static_len"].item()) == 68 + 4
    assert all(torch.isfinite(o.float()).all() for o in outs)
    assert any(not torch.equal(a, b) for a, b in zip(eager2, outs))


def test_use_cluster_estimation_attends_clusters_searched_one_layer_ahead():
    """``use_cluster_estimation``: layer l + 1 attends, with its real query, the clusters that the call for layer l
    searched with ``queries_next`` (model_hub/LLM.py:102-107, cache_hub/retroinfer_cache.py:582-595).  Against the
    oracle with the search query and the attending query kept apart; with a perfect estimate the result is the
    ordinary path's."""
    from retrievalattention_b200.cache_hub import retroinfer_cache

    batch, layers, kv_heads, q_heads, seq_len, max_new = 2, 3, 2, 8, 2048 + 68, 6
    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=2)
    mapping = {str(l): "cuda:0" for l in range(layers)}
    mk = lambda est: retroinfer_cache([0, 0], layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,  # noqa: E731
                                      mapping, max_new, num_gpus=1, model_size=8, use_cluster_estimation=est,
                                      **cfg.as_kwargs())
    ahead, plain = mk(True), mk(False)
    for cache in (ahead, plain):
        for b in range(batch):
            for l in range(layers):
                k, v = make_kv(kv_heads, seq_len, 128, seed=100 * l + b, device="cuda")
                cache.prefill_update_kv_cache(None, k, v, l, b)
        cache.prepare_cache()
    g = batch * kv_heads
    for step in range(2):
        qs = [make_queries(batch, q_heads, 128, seed=500 + 10 * step + l, device="cuda") for l in range(layers)]
        # layer 1 is searched ahead with a noisy estimate of its query, layer 2 with the exact one
        guess = [None, (qs[1].float() + 0.3 * torch.randn_like(qs[1].float())).to(torch.bfloat16), qs[2]]
        for l in range(layers):
            k_new = make_queries(batch, kv_heads, 128, seed=600 + 10 * step + l, device="cuda")
            for cache in (ahead, plain):
                cache.decode_update_kv_cache(k_new, k_new, l)
            q_next = guess[l + 1] if l + 1 < layers else None
            out = ahead.compute(qs[l], l, q_next)
            base = plain.compute(qs[l], l)
            static_len = 68 + step + 1
            ref = oat.compute(qs[l].cpu(), ahead.centroids[l].cpu(), ahead.value_sum[l].cpu(), ahead.cluster_size[l].cpu(),
                              ahead.centroids_mask[l].cpu(), ahead.cluster_count[l].cpu(), ahead.cluster_offset[l].cpu(),
                              ahead.list_keys[l].cpu().view(g, -1, 128), ahead.list_values[l].cpu().view(g, -1, 128),
                              ahead.steady_zone_keys[l].cpu().view(g, -1, 128),
                              ahead.steady_zone_values[l].cpu().view(g, -1, 128), static_len, cfg.nprobe,
                              cfg.max_compute_cluster_num, cfg.cache_unit_size, ahead.buffer_size,
                              select_q=None if guess[l] is None else guess[l].cpu())
            err = (out.cpu().float() - ref.float()).abs()
            assert err.max() <= 2e-2 and err.mean() <= 2e-3, (step, l, float(err.max()), float(err.mean()))
            if l != 1:          # no estimate, or a perfect one: the same clusters as the ordinary path
                assert (out.float() - base.float()).abs().max() <= 1e-2
    assert not any(ahead._ahead)
