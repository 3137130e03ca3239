"""Wave-index parameters derived from a context length and two ratios.

Restates the integer arithmetic of the reference's ``generate_config``
(benchmark/config.py:17-56) and the per-model defaults it starts from
(config/Llama-3-8B-Instruct-Gradient-1048k.json:1-12), without reading any
JSON file: the defaults are identical for every model the reference ships.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict

# config/*.json "RetroInfer" block: identical across the shipped model files.
STATIC_PATTERN_START = 4
STATIC_PATTERN_END = 64
CORE = 22
CACHE_UNIT_SIZE = 8
APPROX_CLUSTER_SIZE = 16  # benchmark/config.py:25


@dataclass(frozen=True)
class WaveIndexConfig:
    """Constructor kwargs of ``retroinfer_cache`` that come from the config file."""

    static_pattern_start: int
    static_pattern_end: int
    core: int
    n_centroids: int
    n_segment: int
    nprobe: int
    max_compute_cluster_num: int
    cache_unit_size: int
    cache_cluster_num: int

    def as_kwargs(self) -> dict:
        return asdict(self)


def generate_config(context_len: int, budget_ratio: float = 0.018,
                    estimate_ratio: float = 0.25, n_segments: int | None = None) -> WaveIndexConfig:
    """benchmark/config.py:34-53 — cluster count snapped to a multiple of
    ``32*n_segments``, ``nprobe = max(1, int(C*budget))``, ``cache = 3*nprobe``,
    ``max_compute = int(C*estimate) + nprobe``."""
    if n_segments is None:
        n_segments = max(1, context_len // 8192)
    n_clusters = math.ceil(context_len / APPROX_CLUSTER_SIZE)
    step = n_segments * 32
    lower = (n_clusters // step) * step
    upper = lower + step
    n_clusters = lower if abs(n_clusters - lower) <= abs(n_clusters - upper) else upper
    nprobe = max(1, int(n_clusters * budget_ratio))
    return WaveIndexConfig(
        static_pattern_start=STATIC_PATTERN_START,
        static_pattern_end=STATIC_PATTERN_END,
        core=CORE,
        n_centroids=n_clusters,
        n_segment=n_segments,
        nprobe=nprobe,
        max_compute_cluster_num=int(n_clusters * estimate_ratio) + nprobe,
        cache_unit_size=CACHE_UNIT_SIZE,
        cache_cluster_num=int(nprobe * 3),
    )


@dataclass(frozen=True)
class Geometry:
    """Attention geometry of one benchmark configuration."""

    name: str
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    batch: int
    context: int
    rope_theta: float
    budget_ratio: float = 0.018
    estimate_ratio: float = 0.232
    hidden: int = 0
    intermediate: int = 0
    vocab: int = 0

    @property
    def group_size(self) -> int:
        return self.q_heads // self.kv_heads

    @property
    def groups(self) -> int:
        return self.batch * self.kv_heads

    def index(self) -> WaveIndexConfig:
        return generate_config(self.context, self.budget_ratio, self.estimate_ratio)


# The five benchmark configurations (shapes only; all data is synthetic).
GEOMETRIES = {
    "cfg0": Geometry("cfg0-cpu-8k", 1, 32, 8, 128, 1, 8192, 5e5),
    "cfg1": Geometry("llama3-8b-128k", 32, 32, 8, 128, 4, 131072, 5e5,
                     hidden=4096, intermediate=14336, vocab=128256),
    "cfg2": Geometry("kmeans-128k", 1, 32, 8, 128, 4, 131072, 5e5),
    "cfg3": Geometry("qwen2.5-7b-256k", 28, 28, 4, 128, 8, 262144, 1e6,
                     hidden=3584, intermediate=18944, vocab=152064),
    "cfg4": Geometry("qwen2.5-72b-128k", 80, 64, 8, 128, 16, 131072, 1e6,
                     hidden=8192, intermediate=29568, vocab=152064),
}
