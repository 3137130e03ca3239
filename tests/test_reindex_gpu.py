"""Re-indexing of generated tokens (cache_hub/retroinfer_cache.py:462-524 ``_update_kv_cache``): after
1024 decode steps the tokens behind the sink tokens are clustered into 64 more clusters per group and
appended to the index; decoding goes on over the longer index.

Checked: the bookkeeping the reference does (sizes, the moved local window, the reset steady length), that the
appended clusters partition exactly the 1024 rows that left the steady zone (bit-exact rows, sizes and
offsets consistent, value sums equal to the members' sums), and the attention output of the steps after
the re-index against the oracle over the longer index (max-abs 2e-2 / mean-abs 2e-3)."""
import pytest
import torch

from oracle import attention as oat
from retrievalattention_b200.config import generate_config
from retrievalattention_b200.synthetic import make_kv

pytestmark = pytest.mark.gpu

THRESHOLD = 1024


# (kv_on_host, batch, kv_heads): the single-group case is the one where the steady-zone slice handed to the
# clustering is contiguous in memory (it must still be a copy: the local window is moved over its first rows)
@pytest.mark.parametrize("kv_on_host,batch,kv_heads", [(False, 2, 2), (True, 2, 2), (False, 1, 1)],
                         ids=["hbm_tier", "host_tier", "hbm_tier_single_group"])
def test_reindex_after_1024_generated_tokens(kv_on_host, batch, kv_heads):
    from retrievalattention_b200.cache_hub import retroinfer_cache

    layers, q_heads, seq_len = 2, 4 * kv_heads, 1024 + 68
    max_new = THRESHOLD + 16
    valid_start = [0, 21][:batch]
    cfg = generate_config(seq_len, 0.05, 0.2, n_segments=1)
    mapping = {str(l): "cuda:0" for l in range(layers)}
    cache = retroinfer_cache(valid_start, layers, batch, seq_len + max_new, kv_heads, q_heads, 128, torch.bfloat16,
                             mapping, max_new, num_gpus=1, model_size=8, kv_on_host=kv_on_host, **cfg.as_kwargs())
    assert cache.input_length_new == THRESHOLD and cache.n_centroids_per_update_segment == 64
    for b in range(batch):
        for l in range(layers):
            k, v = make_kv(kv_heads, seq_len, 128, seed=17 * l + b, device="cuda")
            cache.prefill_update_kv_cache(None, k, v, l, b)
    cache.prepare_cache()
    g, c0 = batch * kv_heads, cache.n_centroids
    n_before = [cache.cluster_offset[l][:, -1].clone() for l in range(layers)]

    gen = torch.Generator(device="cuda").manual_seed(99)
    rnd = lambda heads: torch.randn((batch, 1, heads, 128), generator=gen, device="cuda").to(torch.bfloat16)  # noqa: E731

    def step():
        outs = []
        for l in range(layers):
            k_new, v_new, q = rnd(kv_heads), rnd(kv_heads), rnd(q_heads)
            cache.decode_update_kv_cache(k_new, v_new, l)
            outs.append((q, cache.compute(q, l)))
        return outs

    for _ in range(THRESHOLD):
        step()
    torch.cuda.synchronize()
    assert cache.static_pattern_total == 68 + THRESHOLD and cache.n_centroids == c0
    old_keys = [cache.steady_zone_keys[l].clone() for l in range(layers)]
    old_values = [cache.steady_zone_values[l].clone() for l in range(layers)]

    outs = step()          # its first decode_update_kv_cache re-indexes
    torch.cuda.synchronize()
    assert cache.n_centroids == c0 + 64 and cache.reindex_count == 1
    assert cache.static_pattern_total == 68 + 1
    assert cache.context == seq_len + THRESHOLD + 1

    for l in range(layers):
        assert cache.centroids[l].shape == (g, c0 + 64, 128) and cache.cluster_offset[l].shape == (g, c0 + 65)
        count, off = cache.cluster_count[l], cache.cluster_offset[l]
        assert torch.equal(count[:, c0:].sum(1), torch.full((g,), THRESHOLD, device="cuda", dtype=count.dtype))
        assert torch.equal(off[:, 1:] - off[:, :-1], count)                      # CSR stays consistent
        assert torch.equal(off[:, c0], n_before[l])
        assert torch.equal(cache.centroids_mask[l], count == 0)
        assert torch.equal(cache.cluster_size[l][:, c0:].float(), count[:, c0:].float().to(torch.bfloat16).float())
        # local window moved behind the sink tokens; the new token follows it
        assert torch.equal(cache.steady_zone_keys[l][:, :, 4:68], old_keys[l][:, :, 68 + THRESHOLD - 64:68 + THRESHOLD])
        assert torch.equal(cache.steady_zone_values[l][:, :, 4:68], old_values[l][:, :, 68 + THRESHOLD - 64:68 + THRESHOLD])
        lk = cache.list_keys[l].view(g, -1, 128).cuda()        # pinned host memory on the host tier
        lv = cache.list_values[l].view(g, -1, 128).cuda()
        moved_k = old_keys[l].view(g, -1, 128)[:, 4:4 + THRESHOLD]
        moved_v = old_values[l].view(g, -1, 128)[:, 4:4 + THRESHOLD]
        for grp in range(g):
            n0 = int(n_before[l][grp])
            new_k, new_v = lk[grp, n0:n0 + THRESHOLD], lv[grp, n0:n0 + THRESHOLD]
            # the appended rows are a permutation of the rows that left the steady zone (keys and values together)
            def rows_sorted(a, b):
                both = torch.cat((a, b), dim=1).view(torch.int16).to(torch.int64)
                order = sorted(range(both.shape[0]), key=lambda i: tuple(both[i, :6].tolist()))
                return both[order]
            assert torch.equal(rows_sorted(new_k.cpu(), new_v.cpu()), rows_sorted(moved_k[grp].cpu(), moved_v[grp].cpu()))
            # value sums of the new clusters = sums of their members
            o = off[grp, c0:].tolist()
            for j in (0, 17, 63):
                if o[j + 1] > o[j]:
                    want = lv[grp, o[j]:o[j + 1]].float().sum(0)
                    got = cache.value_sum[l][grp, c0 + j].float()
                    torch.testing.assert_close(got, want, rtol=2.0 ** -7, atol=2e-2)

    def check(outs, static_len):
        for l, (q, out) in enumerate(outs):
            ref = oat.compute(q.cpu(), cache.centroids[l].cpu(), cache.value_sum[l].cpu(), cache.cluster_size[l].cpu(),
                              cache.centroids_mask[l].cpu(), cache.cluster_count[l].cpu(), cache.cluster_offset[l].cpu(),
                              cache.list_keys[l].cpu().view(g, -1, 128), cache.list_values[l].cpu().view(g, -1, 128),
                              cache.steady_zone_keys[l].cpu().view(g, -1, 128),
                              cache.steady_zone_values[l].cpu().view(g, -1, 128), static_len, cfg.nprobe,
                              cfg.max_compute_cluster_num, cfg.cache_unit_size, cache.buffer_size)
            err = (out.cpu().float() - ref.float()).abs()
            assert err.max() <= 2e-2 and err.mean() <= 2e-3, (l, float(err.max()), float(err.mean()))

    check(outs, 68 + 1)
    check(step(), 68 + 2)


def test_reindex_needs_room_announced_at_construction():
    from retrievalattention_b200.cache_hub import retroinfer_cache

    cfg = generate_config(1024 + 68, 0.05, 0.2, n_segments=1)
    cache = retroinfer_cache([0], 1, 1, 1024 + 68 + 8, 2, 8, 128, torch.bfloat16, {"0": "cuda:0"}, 8, num_gpus=1,
                             model_size=8, **cfg.as_kwargs())
    assert cache.input_length_new == 0
    with pytest.raises(RuntimeError, match="no room"):
        cache._update_kv_cache()
