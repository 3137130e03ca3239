"""The decode kernel and the clustering at the benchmark's full size (configuration 1: 32 groups, 131072 tokens,
8192 centroids, nprobe 147, 1900 estimated clusters; one layer), where the CPU oracle is too slow: checks of
properties that do not depend on the size.

* selection: retrieved / estimated ids are distinct and disjoint, and every retrieved key >= every estimated
  key >= every unselected key (the 16-bit distance keys the kernel ranks by); empty clusters are never taken;
* page budget and row list: the kept clusters are a prefix, their rows are exactly the CSR ranges, in order;
* attention: for a few groups, an fp32 evaluation over exactly the rows and clusters the kernel selected
  (max-abs 2e-2, mean-abs 2e-3), the single kernel against the three stage kernels, the output-only form
  against the id-producing form, and bit-exact repeatability;
* clustering: counts and offsets form a CSR partition of the tokens, the cluster-contiguous copy is a
  permutation of the input rows (bit-exact gather), every centroid is the mean of its members and the value
  sums are the sums of the members' values (the assignment itself is pinned at small sizes by the golden
  fixtures)."""
import pytest
import torch

from retrievalattention_b200 import wave
from retrievalattention_b200.cache_hub.kmeans import build_index
from retrievalattention_b200.config import GEOMETRIES
from retrievalattention_b200.synthetic import make_kv, make_queries

pytestmark = pytest.mark.gpu

SINK, RECENT = 4, 64


@pytest.fixture(scope="module")
def full_layer():
    geo = GEOMETRIES["cfg1"]
    cfg = geo.index()
    dev = torch.device("cuda", 0)
    n = geo.context - SINK - RECENT
    parts = []
    for b in range(geo.batch):
        k, v = make_kv(geo.kv_heads, geo.context, 128, seed=500 + b, theta=geo.rope_theta, device=dev)
        k, v = k[0].transpose(0, 1).contiguous(), v[0].transpose(0, 1).contiguous()       # [kv_heads, ctx, 128]
        r = build_index(k[:, SINK:SINK + n].contiguous(), v[:, SINK:SINK + n].contiguous(), cfg.n_centroids,
                        cfg.n_segment, 10, want_lists=True)
        assert int(r["error"]) == 0
        r["raw_k"], r["raw_v"] = k, v
        parts.append(r)
    cat = lambda name: torch.cat([p[name] for p in parts], 0).contiguous()          # noqa: E731
    g = geo.batch * geo.kv_heads
    stride = SINK + RECENT + 8
    steady_k = torch.zeros((g, stride, 128), dtype=torch.bfloat16, device=dev)
    steady_v = torch.zeros_like(steady_k)
    raw_k, raw_v = cat("raw_k"), cat("raw_v")
    steady_k[:, :SINK], steady_v[:, :SINK] = raw_k[:, :SINK], raw_v[:, :SINK]
    steady_k[:, SINK:SINK + RECENT], steady_v[:, SINK:SINK + RECENT] = raw_k[:, SINK + n:], raw_v[:, SINK + n:]
    buffer_pages = max(cfg.nprobe * 4, 16) * 2          # cache_hub/retroinfer_cache.py:111 with 16-token clusters
    shape = wave.WaveShape(g, geo.q_heads // geo.kv_heads, cfg.n_centroids, cfg.nprobe,
                           cfg.max_compute_cluster_num - cfg.nprobe, cfg.cache_unit_size, buffer_pages, n, stride,
                           torch.bfloat16)
    t = dict(centroids=cat("centroids"), value_sum=cat("value_sum"), cluster_size=cat("cluster_size"),
             cluster_count=cat("cluster_count"), cluster_offset=cat("cluster_offset"), keys=cat("keys"),
             values=cat("values"), steady_keys=steady_k, steady_values=steady_v)
    static_len = torch.full((1,), SINK + RECENT, dtype=torch.int32, device=dev)
    mk = lambda ids: wave.WaveIndexLayer(shape, want_ids=ids, static_len=static_len,       # noqa: E731
                                         scratch=wave.new_scratch(shape, dev), **t)
    q = make_queries(geo.batch, geo.q_heads, 128, seed=77, device=dev)
    return dict(geo=geo, cfg=cfg, shape=shape, t=t, with_ids=mk(True), plain=mk(False), q=q, parts=parts, n=n,
                raw_k=raw_k, raw_v=raw_v, buffer_pages=buffer_pages)


def test_selection_budget_rows_and_attention(full_layer):
    f = full_layer
    s, t, layer = f["shape"], f["t"], f["with_ids"]
    out = layer.compute(f["q"]).clone()
    torch.cuda.synchronize()
    v = layer.views()
    ret, est, kept = layer.retrieved_ids, layer.estimated_ids, layer.retrieved_kept
    keys = (v["dist_keys"].to(torch.int32) & 0xFFFF)
    g, c = s.groups, s.n_centroids
    both = torch.cat((ret, est), 1)
    assert both.min() >= 0 and both.max() < c
    assert (torch.sort(both, 1).values.diff(dim=1) > 0).all()                   # distinct and disjoint
    k_ret, k_est = torch.gather(keys, 1, ret), torch.gather(keys, 1, est)
    rest = torch.ones((g, c), dtype=torch.bool, device=keys.device).scatter_(1, both, False)
    k_rest_max = torch.where(rest, keys, torch.zeros_like(keys)).max(1).values
    assert (k_ret.min(1).values >= k_est.max(1).values).all()
    assert (k_est.min(1).values >= k_rest_max).all()
    assert (k_ret[:, :-1] >= k_ret[:, 1:]).all()                                # ranked
    assert (torch.gather(t["cluster_count"], 1, both) > 0).all()                # no empty cluster is ever taken
    # page budget: the kept clusters are the longest prefix of the ranking whose pages fit
    cnt = torch.gather(t["cluster_count"], 1, ret).long()
    pages = ((cnt + s.page_size - 1) // s.page_size).cumsum(1)
    expect_kept = (pages <= f["buffer_pages"]).long().cumprod(1).sum(1)
    assert torch.equal(kept.long(), expect_kept)
    # row list = the kept clusters' CSR ranges, in rank order
    n_exact = v["n_exact"].long()
    for gi in range(0, g, 5):
        rows = []
        for cid in ret[gi, :int(kept[gi])].tolist():
            rows.append(torch.arange(int(t["cluster_offset"][gi, cid]), int(t["cluster_offset"][gi, cid + 1])))
        rows = torch.cat(rows)
        assert int(n_exact[gi]) == rows.numel()
        assert torch.equal(v["exact_rows"][gi, :rows.numel()].cpu().long(), rows)
        # attention in fp32 over exactly that selection
        qg = f["q"].reshape(g, s.group_size, 128)[gi].float()
        kk = torch.cat((t["steady_keys"][gi, :SINK + RECENT], t["keys"][gi, rows.cuda()])).float()
        vv = torch.cat((t["steady_values"][gi, :SINK + RECENT], t["values"][gi, rows.cuda()])).float()
        ce = t["centroids"][gi, est[gi]].float()
        se = qg @ ce.T / 128 ** 0.5
        sx = qg @ kk.T / 128 ** 0.5
        m = torch.maximum(se.max(1).values, sx.max(1).values)[:, None]
        we = t["cluster_size"][gi, est[gi]].float()[None, :]
        num = torch.exp(se - m) @ t["value_sum"][gi, est[gi]].float() + torch.exp(sx - m) @ vv
        den = (we * torch.exp(se - m)).sum(1, keepdim=True) + torch.exp(sx - m).sum(1, keepdim=True)
        ref = num / den
        err = (out.reshape(g, s.group_size, 128)[gi].float() - ref).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (gi, float(err.max()), float(err.mean()))


def test_forms_agree_and_repeat(full_layer):
    f = full_layer
    a = f["with_ids"].compute(f["q"]).clone()
    ids_a = f["with_ids"].retrieved_ids.clone()
    b = f["with_ids"].compute_staged(f["q"]).clone()
    ids_b = f["with_ids"].retrieved_ids.clone()
    c = f["plain"].compute(f["q"]).clone()
    d = f["plain"].compute(f["q"]).clone()
    torch.cuda.synchronize()
    assert torch.equal(ids_a, ids_b)                                            # same ranking in both forms
    assert (a.float() - b.float()).abs().max() <= 1e-2
    assert (a.float() - c.float()).abs().max() <= 1e-2
    assert torch.equal(c.view(torch.int16), d.view(torch.int16))                # bit-exact repeatability


def test_clustering_invariants(full_layer):
    f = full_layer
    n, c = f["n"], f["cfg"].n_centroids
    for r in f["parts"][:2]:
        count, offset = r["cluster_count"].long(), r["cluster_offset"].long()
        assert (count.sum(1) == n).all() and (offset[:, 0] == 0).all()
        assert torch.equal(offset[:, 1:], count.cumsum(1))
        assign, order = r["assign"].long(), r["order"].long()
        assert torch.equal(torch.sort(order, 1).values, torch.arange(n, device=order.device).expand_as(order))
        sorted_cl = torch.gather(assign, 1, order)
        assert (sorted_cl.diff(dim=1) >= 0).all()                               # cluster-major
        same = sorted_cl.diff(dim=1) == 0
        assert (order.diff(dim=1)[same] > 0).all()                              # ascending inside a cluster
        raw_k, raw_v = r["raw_k"][:, SINK:SINK + n], r["raw_v"][:, SINK:SINK + n]
        idx = order[:, :, None].expand(-1, -1, 128)
        assert torch.equal(r["keys"].view(torch.int16), torch.gather(raw_k, 1, idx).view(torch.int16))
        assert torch.equal(r["values"].view(torch.int16), torch.gather(raw_v, 1, idx).view(torch.int16))
        # value sums and centroids from the members (fp32 sums; one rounding of slack)
        h = 1
        vs = torch.zeros((c, 128), device=raw_v.device).index_add_(0, assign[h], raw_v[h].float())
        assert (r["value_sum"][h].float() - vs).abs().max() <= 0.02 * vs.abs().max()
        ks = torch.zeros((c, 128), device=raw_k.device).index_add_(0, assign[h], raw_k[h].float())
        mean = ks / count[h].clamp(min=1)[:, None].float()
        nonempty = count[h] > 0
        assert (r["centroids"][h].float() - mean)[nonempty].abs().max() <= 0.05 * mean[nonempty].abs().max()
