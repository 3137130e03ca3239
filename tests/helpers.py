"""Test helpers: build a small wave index with the CPU oracle and mirror it on the GPU."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from oracle import kmeans as okm
from retrievalattention_b200.synthetic import make_kv, make_queries

SINK, RECENT = 4, 64


@dataclass
class Case:
    batch: int
    kv_heads: int
    group_size: int
    context: int
    n_centroids: int
    n_segment: int
    nprobe: int
    n_estimate: int
    max_new: int = 8
    page_size: int = 8
    buffer_pages: int | None = None
    iters: int = 4
    seed: int = 0
    dtype: torch.dtype = torch.bfloat16
    planted: int = 0
    duplicate_rows: int = 0   # >0: only that many distinct key rows (forces empty clusters)

    @property
    def groups(self):
        return self.batch * self.kv_heads

    @property
    def q_heads(self):
        return self.kv_heads * self.group_size

    @property
    def n_clustered(self):
        return self.context - SINK - RECENT

    @property
    def steady_stride(self):
        return SINK + RECENT + self.max_new

    def pages(self):
        if self.buffer_pages is not None:
            return self.buffer_pages
        avg = self.n_clustered // self.n_centroids
        return max(self.nprobe * 4, 16) * math.ceil(avg / self.page_size)


def build_cpu_index(case: Case) -> dict:
    """Per-request prefill as the reference does it (cache_hub/retroinfer_cache.py:368-441),
    evaluated by the oracle; returns CPU tensors in the [G, ...] layout."""
    g, c, n = case.groups, case.n_centroids, case.n_clustered
    out = {
        "centroids": torch.zeros((g, c, 128), dtype=case.dtype),
        "value_sum": torch.zeros((g, c, 128), dtype=case.dtype),
        "cluster_size": torch.zeros((g, c), dtype=case.dtype),
        "cluster_count": torch.zeros((g, c), dtype=torch.int32),
        "cluster_offset": torch.zeros((g, c + 1), dtype=torch.int32),
        "mask": torch.zeros((g, c), dtype=torch.bool),
        "keys": torch.zeros((g, n, 128), dtype=case.dtype),
        "values": torch.zeros((g, n, 128), dtype=case.dtype),
        "steady_keys": torch.zeros((g, case.steady_stride, 128), dtype=case.dtype),
        "steady_values": torch.zeros((g, case.steady_stride, 128), dtype=case.dtype),
        "raw_keys": [], "raw_values": [],
    }
    for b in range(case.batch):
        k, v = make_kv(case.kv_heads, case.context, 128, seed=case.seed * 1000 + b, dtype=case.dtype,
                       planted_centres=case.planted)
        k = k[0].transpose(0, 1).contiguous()   # [Hk, ctx, d]
        v = v[0].transpose(0, 1).contiguous()
        if case.duplicate_rows:
            k = k[:, torch.arange(case.context) % case.duplicate_rows].contiguous()
        out["raw_keys"].append(k)
        out["raw_values"].append(v)
        sl = slice(b * case.kv_heads, (b + 1) * case.kv_heads)
        mid_k = k[:, SINK:case.context - RECENT].contiguous()
        mid_v = v[:, SINK:case.context - RECENT].contiguous()
        meta = okm.build_meta_index(mid_k, mid_v, c, case.n_segment, case.iters)
        lk, lv, starts = okm.organize_kv(mid_k, mid_v, meta["clusters"], meta["cluster_size"])
        out["centroids"][sl] = meta["centroids"]
        out["value_sum"][sl] = meta["value_sum"]
        out["cluster_size"][sl] = meta["cluster_size_dtype"]
        out["cluster_count"][sl] = meta["cluster_size"]
        out["cluster_offset"][sl] = starts
        out["mask"][sl] = meta["mask"]
        out["keys"][sl] = lk
        out["values"][sl] = lv
        out["steady_keys"][sl, :SINK] = k[:, :SINK]
        out["steady_keys"][sl, SINK:SINK + RECENT] = k[:, case.context - RECENT:]
        out["steady_values"][sl, :SINK] = v[:, :SINK]
        out["steady_values"][sl, SINK:SINK + RECENT] = v[:, case.context - RECENT:]
    return out


def to_gpu_layer(case: Case, cpu: dict, static_len: int, want_ids: bool = True):
    from retrievalattention_b200 import wave

    dev = torch.device("cuda:0")
    shape = wave.WaveShape(case.groups, case.group_size, case.n_centroids, case.nprobe, case.n_estimate,
                           case.page_size, case.pages(), case.n_clustered, case.steady_stride, case.dtype)
    names = ("centroids", "value_sum", "cluster_size", "cluster_count", "cluster_offset", "keys", "values",
             "steady_keys", "steady_values")
    t = {k: cpu[k].to(dev).contiguous() for k in names}
    t["static_len"] = torch.tensor([static_len], dtype=torch.int32, device=dev)
    t["scratch"] = wave.new_scratch(shape, dev)
    return wave.WaveIndexLayer(shape, want_ids=want_ids, **t)


def queries(case: Case, seed: int = 100) -> torch.Tensor:
    return make_queries(case.batch, case.q_heads, 128, seed=seed, dtype=case.dtype)


def gpu_built_layer(batch: int, kv_heads: int, group_size: int, n_clustered: int, n_centroids: int, n_segment: int,
                    nprobe: int, n_estimate: int, seed: int = 0, iters: int = 3, want_ids: bool = True,
                    n_layers: int = 1):
    """Layers whose index is built on the GPU by ``ri_kmeans_build`` (sizes the CPU oracle would take too long to
    cluster).  Returns (list of WaveIndexLayer over the same tensors, dict of the tensors, queries [B, 1, Hq, 128])."""
    from retrievalattention_b200 import wave
    from retrievalattention_b200.cache_hub.kmeans import build_index

    dev = torch.device("cuda", 0)
    context = n_clustered + SINK + RECENT
    parts = []
    raw = []
    for b in range(batch):
        k, v = make_kv(kv_heads, context, 128, seed=seed * 1000 + b, device=dev)
        k, v = k[0].transpose(0, 1).contiguous(), v[0].transpose(0, 1).contiguous()
        r = build_index(k[:, SINK:SINK + n_clustered].contiguous(), v[:, SINK:SINK + n_clustered].contiguous(),
                        n_centroids, n_segment, iters)
        assert int(r["error"]) == 0
        parts.append(r)
        raw.append((k, v))
    cat = lambda name: torch.cat([p[name] for p in parts], 0).contiguous()          # noqa: E731
    g = batch * kv_heads
    stride = SINK + RECENT + 8
    steady_k = torch.zeros((g, stride, 128), dtype=torch.bfloat16, device=dev)
    steady_v = torch.zeros_like(steady_k)
    raw_k, raw_v = torch.cat([r[0] for r in raw], 0), torch.cat([r[1] for r in raw], 0)
    steady_k[:, :SINK], steady_v[:, :SINK] = raw_k[:, :SINK], raw_v[:, :SINK]
    steady_k[:, SINK:SINK + RECENT] = raw_k[:, SINK + n_clustered:]
    steady_v[:, SINK:SINK + RECENT] = raw_v[:, SINK + n_clustered:]
    pages = max(nprobe * 4, 16) * math.ceil((n_clustered // n_centroids) / 8)
    shape = wave.WaveShape(g, group_size, n_centroids, nprobe, n_estimate, 8, pages, n_clustered, stride, torch.bfloat16)
    t = dict(centroids=cat("centroids"), value_sum=cat("value_sum"), cluster_size=cat("cluster_size"),
             cluster_count=cat("cluster_count"), cluster_offset=cat("cluster_offset"), keys=cat("keys"),
             values=cat("values"), steady_keys=steady_k, steady_values=steady_v)
    static_len = torch.full((1,), SINK + RECENT, dtype=torch.int32, device=dev)
    layers = [wave.WaveIndexLayer(shape, want_ids=want_ids, static_len=static_len, scratch=wave.new_scratch(shape, dev), **t)
              for _ in range(n_layers)]
    q = make_queries(batch, kv_heads * group_size, 128, seed=seed + 100, device=dev)
    return layers, t, q
