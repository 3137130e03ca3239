#!/usr/bin/env python
"""Decode-throughput benchmark of the wave-index attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config cfg1|cfg2|cfg3|cfg4] [--no-model]
                    [--kv-on-host [--miss-path pull|staged|uva] [--layers L]] [--prefill-seq S] [--no-cfg4]

Workload (default, N=1): Llama-3-8B decode-attention geometry — 32 layers, 32 q / 8 kv heads,
head_dim 128, batch 4, context 131072, 8192 centroids per kv head, budget 0.018, estimate 0.232 —
on seeded synthetic bf16 K/V/q, driven through the ``retroinfer_cache`` interface: prefill
clustering per request and layer (untimed set-up, ``ri_kmeans_build``), then per decode step and
layer ``decode_update_kv_cache`` + ``compute``.

Prints ONE JSON line (rank 0).  ``value`` is tokens/s with every input resident in HBM and the
whole step replayed as one CUDA graph; ``e2e`` is the same step with q/k/v starting in pinned host
memory and the attention output copied back to the host inside the timed region.  On one GPU the line
also carries ``parity`` (layer 0 of the workload on the GPU against the CPU oracle: selected sets with the
1e-3 tie rule, kept clusters, attention error), ``decode_model`` (the whole model step — projections, MLP,
vocabulary head with random weights — around the same caches; ``--no-model`` skips it) and ``kmeans``
(the prefill clustering of configuration 2 against the tensor-core roofline).

``--config cfg2`` times the prefill clustering alone (32 groups x 131072 keys, 8192 centroids,
10 iterations) in more detail.  ``--kv-on-host`` times the host tier (cluster store in pinned host memory, page
cache on the GPU) for every way of bringing missed pages up; under torchrun the batch is split over the ranks.
``--prefill-seq S`` times the dense prefill attention of one prompt of S tokens alone.  The default line carries a
short host-tier run as ``host_tier`` (``--no-host-tier`` skips it; a ``--layers`` override does too).  On several GPUs the
line also carries ``cfg4``: configuration 4 (64q/8kv heads, batch 16) with its KV heads sharded over the ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from dataclasses import replace

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from retrievalattention_b200.config import GEOMETRIES  # noqa: E402
from retrievalattention_b200.synthetic import make_kv  # noqa: E402

SINK, RECENT = 4, 64
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from ncu captures of one layer of configuration 1 (32 groups)
NCU_TRAFFIC = {"decode": 118.4e6, "scan": 70.18e6, "select": 6.33e6, "attend": 46.67e6}
METRIC = "decode tok/s at 128K ctx (Llama-3-8B geometry); attn kernel HBM GB/s vs peak"


# ----------------------------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------------------------
class Workload:
    """One rank's resident state: the cache of every layer and the per-step inputs."""

    def __init__(self, geo, device, total_steps, kmeans_iters=10, rank=0, log=None, world=1, weak=True):
        from retrievalattention_b200.cache_hub import retroinfer_cache
        from retrievalattention_b200.head_shard import HeadGather, HeadShard

        # N ranks, weak scaling: global batch = batch * N requests, KV heads sharded over the ranks (then batch), so
        # every rank holds the same number of (request, kv-head) groups as the 1-GPU workload.  Not weak: the
        # geometry's own batch, so a rank's share shrinks with N.
        self.global_geo = geo
        self.shard = HeadShard(rank, world, geo.kv_heads, geo.q_heads, geo.batch * (world if weak else 1))
        geo = replace(geo, kv_heads=self.shard.local_kv_heads, q_heads=self.shard.local_q_heads,
                      batch=self.shard.local_batch)
        self.gather = HeadGather(self.shard, HeadGather.make_groups(self.shard)) if world > 1 else None
        self.geo, self.device = geo, device
        self.cfg = cfg = geo.index()
        max_new = total_steps + 2
        dev = str(device)
        mapping = {str(l): dev for l in range(geo.layers)}
        self.cache = retroinfer_cache([0] * geo.batch, geo.layers, geo.batch, geo.context + max_new, geo.kv_heads,
                                      geo.q_heads, geo.head_dim, torch.bfloat16, mapping, max_new, num_gpus=1,
                                      model_size=8, **cfg.as_kwargs())
        t0 = time.time()
        ev = []
        for l in range(geo.layers):
            for b in range(geo.batch):
                k, v = make_kv(geo.kv_heads, geo.context, geo.head_dim, seed=(rank * 131 + l) * 1000 + b,
                               theta=geo.rope_theta, device=device)
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                self.cache.prefill_update_kv_cache(None, k, v, l, b)
                z.record()
                ev.append((a, z))
                self.cache.sync(l, b)
                del k, v
            if log and (l % 8 == 7 or l == geo.layers - 1):
                torch.cuda.synchronize()
                log(f"set-up: {l + 1}/{geo.layers} layers indexed, {time.time() - t0:.1f}s, "
                    f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB")
        self.cache.prepare_cache()
        self.prefill_index_ms = statistics.median(a.elapsed_time(z) for a, z in ev)
        self.shape = self.cache.shape
        g = torch.Generator(device=device)
        g.manual_seed(12345 + rank)
        shp_q = (total_steps, geo.layers, geo.batch, 1, geo.q_heads, geo.head_dim)
        shp_kv = (total_steps, geo.layers, geo.batch, 1, geo.kv_heads, geo.head_dim)
        rnd = lambda s: torch.randn(s, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)  # noqa: E731
        self.q_all, self.k_all, self.v_all = rnd(shp_q), rnd(shp_kv), rnd(shp_kv)
        self.q_in = torch.zeros(shp_q[1:], dtype=torch.bfloat16, device=device)
        self.k_in = torch.zeros(shp_kv[1:], dtype=torch.bfloat16, device=device)
        self.v_in = torch.zeros(shp_kv[1:], dtype=torch.bfloat16, device=device)
        self.out = torch.zeros(shp_q[1:], dtype=torch.bfloat16, device=device)
        self.gathered = None
        self.peer = None
        if self.gather is not None:
            # the gather of the head slices: done by the decode kernel itself through peer-mapped buffers
            # (PeerGather); a failed set-up of those buffers is an error.  The NCCL all-gather is opt-in only
            # (RI_GATHER=nccl): there is no silent change of the exchange under a measurement.
            if os.environ.get("RI_GATHER", "peer") != "nccl":
                from retrievalattention_b200.head_shard import PeerGather
                self.peer = PeerGather(self.shard, geo.layers, geo.batch, geo.q_heads, geo.head_dim, torch.bfloat16,
                                       device, group=self.gather.group)
            if self.peer is None:
                self.gathered = torch.zeros((geo.layers, self.shard.head_shards) + tuple(shp_q[2:]),
                                            dtype=torch.bfloat16, device=device)
        self.graph = None

    def step_body(self):
        """One decode step of the hot path over all layers on the current stream: per layer the
        reference's two calls (model_hub/LLM.py:116-117), which end up as one launch: the decode kernel
        stores the step's key/value rows into the steady zone before it attends.
        Several GPUs: the head slices of all ranks -> [B, 1, Hq, d] for the output projection, either
        written by the decode kernel into every rank's buffer (then one bounded flag wait per layer) or
        by an NCCL all-gather."""
        if self.peer is not None:
            self.peer.next_step()
        for l in range(self.geo.layers):
            self.cache.decode_update_kv_cache(self.k_in[l], self.v_in[l], l)
            self.cache.compute(self.q_in[l], l, out=self.out[l], gather=self.peer)
            if self.peer is not None:
                self.peer.wait(l)
            elif self.gather is not None:
                self.gather(self.out[l], self.gathered[l])

    def capture(self):
        self.step_body()                     # one eager step first (also advances the steady zone)
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.step_body()
            self.graph = graph
        except Exception as exc:             # an NCCL collective that cannot be captured (RI_GATHER=nccl): step eagerly
            if self.gather is None or self.peer is not None:
                raise
            self.graph = None
            self.capture_error = repr(exc)[:200]
            torch.cuda.synchronize()

    def replay(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_body()

    def launches_per_step(self):
        # per layer: the single decode kernel, which also appends the step's key/value rows (RI_WAVE_STAGED=1:
        # steady append, scan, select, attend), plus the flag wait of the peer-store gather
        # geometries beyond 8192 centroids are outside the single kernel's range: the library runs the stages
        staged = os.environ.get("RI_WAVE_STAGED", "0") not in ("", "0") or self.cfg.n_centroids > 8192
        return ((4 if staged else 1) + (1 if self.peer is not None else 0)) * self.geo.layers

    def static_len(self):
        return int(self.cache._per_device[str(self.device)]["static_len"].item())


# ----------------------------------------------------------------------------------------------
# measurement helpers
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    PERIOD_MS = 20
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", str(self.PERIOD_MS)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        num = lambda s: s.replace(".", "").isdigit()  # noqa: E731
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and num(r[1])]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and num(r[2])]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


def algorithmic_bytes(wl, n_ret_rows, static_len):
    """Per layer-step, all groups (bf16): centroids once, value sums of the estimation set, K and V
    of retrieved + steady rows, cluster sizes, q and out."""
    s, d = wl.shape, 128
    g = s.groups
    scan = g * (2 * d * s.n_centroids + 2 * s.group_size * d)
    select = g * 2 * s.n_centroids
    attend = 2 * d * (g * s.n_estimate + 2 * (n_ret_rows + g * static_len)) + g * 2 * 2 * s.group_size * d
    return {"scan": scan, "select": select, "attend": attend}


def time_stages(wl, first_step, steps):
    """Device time per layer of the single decode kernel, and of each stage of the three-kernel
    form, averaged over layers and steps.  CUDA graphs replay, over ALL layers (so every launch
    works on cold data, as in the real step, and no host launch gap is timed), the single kernel
    and the stage prefixes scan / scan+select / scan+select+attend; a stage's time is the
    difference between consecutive prefixes."""
    names = ("scan", "select", "attend")
    layers = wl.cache._layers
    graphs = []
    wl.q_in.copy_(wl.q_all[first_step]); wl.k_in.copy_(wl.k_all[first_step]); wl.v_in.copy_(wl.v_all[first_step])
    for upto in range(0, 4):
        def body():
            for l, layer in enumerate(layers):
                if upto == 0:
                    layer.compute(wl.q_in[l], wl.out[l])      # what the step launches (ri_wave_decode_layer)
                for n in names[:upto]:
                    layer.stage(n, wl.q_in[l], wl.out[l])
        body()                                       # warm (and validate) outside capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        graphs.append(g)
    prefix_ms = []
    for g in graphs:
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for st in range(steps):
            wl.q_in.copy_(wl.q_all[first_step + st])
            g.replay()
        b.record()
        torch.cuda.synchronize()
        prefix_ms.append(a.elapsed_time(b) / (steps * len(layers)))
    ms = {"decode": prefix_ms[0], "scan": prefix_ms[1], "select": prefix_ms[2] - prefix_ms[1],
          "attend": prefix_ms[3] - prefix_ms[2]}
    n_ret = 0
    for l, layer in enumerate(layers):
        for n in names[:2]:
            layer.stage(n, wl.q_in[l], wl.out[l])
        n_ret += int(layer.views()["n_exact"].sum().item())
    return ms, n_ret / len(layers), wl.static_len()


def cpu_layer_seconds(wl, layer_idx, step, repeats, static_len=SINK + RECENT + 1, with_parts=False):
    """The oracle port of the reference arithmetic for one layer (all groups) on the host cores.
    Returns the median seconds per evaluation (and, on request, the output and the selection it made)."""
    from oracle import attention as oat

    torch.set_num_threads(os.cpu_count())
    c, g = wl.cache, wl.shape.groups
    cpu = dict(centroids=c.centroids[layer_idx].cpu(), value_sum=c.value_sum[layer_idx].cpu(),
               size=c.cluster_size[layer_idx].cpu(), count=c.cluster_count[layer_idx].cpu(),
               offset=c.cluster_offset[layer_idx].cpu(), keys=c.list_keys[layer_idx].cpu().view(g, -1, 128),
               values=c.list_values[layer_idx].cpu().view(g, -1, 128),
               sk=c.steady_zone_keys[layer_idx].cpu().view(g, -1, 128),
               sv=c.steady_zone_values[layer_idx].cpu().view(g, -1, 128))
    q = wl.q_all[step, layer_idx].cpu()
    s = wl.shape
    times = []
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        ref, parts = oat.compute(q, cpu["centroids"], cpu["value_sum"], cpu["size"], cpu["count"] == 0, cpu["count"],
                                 cpu["offset"], cpu["keys"], cpu["values"], cpu["sk"], cpu["sv"], static_len, s.nprobe,
                                 s.nprobe + s.n_estimate, s.page_size, s.buffer_pages, return_parts=True)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times[1:])
    return (sec, ref, parts) if with_parts else sec


def layer_parity(wl, layer_idx, step):
    """Layer ``layer_idx`` of the workload, all groups, one decode step: the GPU path (through the C ABI, with the
    id outputs switched on) against the CPU oracle fed the same index, query and steady zone.  Also returns the
    oracle's seconds per evaluation, which is the CPU baseline's sample."""
    from oracle import score_select as oss
    from retrievalattention_b200 import wave

    bound = wl.cache._layers[layer_idx]
    s = wl.shape
    static_len = wl.static_len()
    t = dict(bound.t)
    t["scratch"] = wave.new_scratch(s, wl.device)
    probe = wave.WaveIndexLayer(s, want_ids=True, **t)
    q = wl.q_all[step, layer_idx].contiguous()
    out = probe.compute(q)
    torch.cuda.synchronize()
    sec, ref, parts = cpu_layer_seconds(wl, layer_idx, step, 2, static_len=static_len, with_parts=True)
    ret, est = probe.retrieved_ids.cpu(), probe.estimated_ids.cpu()
    err = (out.cpu().float() - ref.float()).abs()
    parity = {
        "config": f"layer {layer_idx} of the workload, all {s.groups} groups, GPU (C ABI, id outputs on) vs CPU oracle",
        "max_abs": round(float(err.max()), 5), "mean_abs": round(float(err.mean()), 6),
        "tolerance": "max_abs <= 2e-2, mean_abs <= 2e-3; sets bit-exact outside a 1e-3 tie band at the cut",
        "retrieval_sets_ok": bool(oss.selection_matches(parts["dist"], ret, s.nprobe)),
        "estimation_sets_ok": bool(oss.selection_matches(parts["dist"], torch.cat((ret, est), 1), s.nprobe + s.n_estimate)),
        "kept_ok": probe.retrieved_kept.cpu().tolist() == list(parts["kept"]),
    }
    parity["ok"] = bool(parity["retrieval_sets_ok"] and parity["estimation_sets_ok"] and parity["kept_ok"]
                        and parity["max_abs"] <= 2e-2 and parity["mean_abs"] <= 2e-3)
    return parity, sec


def reference_gpu_sequence(wl, steps):
    """The reference's OWN CUDA kernels on the same GPU and the same layers: the part of its ``compute`` that its
    shipped extension modules cover — ``batch_gemm_softmax`` (CUTLASS GEMM + softmax), the group sum, the mask,
    ``torch.topk`` of max_compute clusters and ``gather_copy_vectors`` of the estimation rows
    (cache_hub/retroinfer_cache.py:569-575, :601-605) — compiled for sm_100a into ``oracle/_ref``.  Its two
    ``weighted_flash_decoding`` calls come from a package that is not available, and its host wave buffer is left
    out, so this is a LOWER bound of the reference's per-layer GPU time.  Times all layers from one CUDA graph;
    returns None when the modules were never built."""
    from oracle import build_ref

    gs_mod, cp_mod = build_ref.load("gemm_softmax"), build_ref.load("Copy")
    if gs_mod is None or cp_mod is None:
        return None
    c, s, dev = wl.cache, wl.shape, wl.device
    g, gsz, n_c, d = s.groups, s.group_size, s.n_centroids, 128
    k_all = s.nprobe + s.n_estimate
    gemm_o = torch.zeros((g, gsz, n_c), dtype=torch.bfloat16, device=dev)
    softmax_o = torch.zeros_like(gemm_o)
    blocks = (n_c + 255) // 256
    norm = torch.zeros((g, gsz, blocks), dtype=torch.float32, device=dev)
    ssum = torch.zeros_like(norm)
    es_c = torch.zeros((g, s.n_estimate, d), dtype=torch.bfloat16, device=dev)
    es_v = torch.zeros_like(es_c)
    es_s = torch.zeros((g, s.n_estimate), dtype=torch.bfloat16, device=dev)
    dtype_min = torch.finfo(torch.bfloat16).min

    def body():
        for l in range(len(c.centroids)):
            q = wl.q_in[l].view(g, gsz, d)
            gs_mod.batch_gemm_softmax(q, c.centroids[l], gemm_o, norm, ssum, softmax_o, g, gsz, n_c, d, 1 / 128 ** 0.5, 0)
            dist = torch.sum(softmax_o, dim=1)
            dist.masked_fill_(c.centroids_mask[l], dtype_min)
            ci = torch.topk(dist, k_all, dim=-1, largest=True, sorted=True)[1]
            cp_mod.gather_copy_vectors(c.centroids[l], es_c, c.value_sum[l], es_v, c.cluster_size[l], es_s, ci, g, n_c,
                                       s.n_estimate, k_all, s.nprobe, s.n_estimate)

    # the reference's GEMM is issued on the legacy default stream (batch_gemm_softmax.h:520), which cannot be captured
    # in a graph: time eager launches on the default stream, launch gaps included (as the reference itself runs)
    body()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        body()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (steps * len(c.centroids))
    return {"sequence": "reference kernels built for sm_100a: batch_gemm_softmax + sum + masked_fill + topk + gather_copy_vectors "
                        "(scores, selection, estimation gather; its attention calls are not available)",
            "ms_per_layer": round(ms, 4), "launch": "eager on the default stream, as the reference issues it"}


def model_decode(wl, geo, args, warm, log):
    """Decode tokens/s of the whole model step around the same caches: embedding,
    per layer RMS norm -> fused QKV projection -> rotary embedding -> cache update + wave-index
    attention -> output projection -> RMS norm -> MLP, final norm, vocabulary projection and greedy
    arg-max, with seeded random weights at the model's published shapes; one CUDA graph per step.
    The second figure feeds the token ids from pinned host memory and reads the next ids back every step."""
    from retrievalattention_b200 import decode_layer as dl

    shapes = {"llama3-8b": dl.LLAMA3_8B, "qwen2.5-7b": dl.QWEN25_7B, "qwen2.5-72b": dl.QWEN25_72B}
    shape = next((v for k, v in shapes.items() if geo.name.startswith(k)), None)
    if shape is None:
        return {"unavailable": f"no model shape for {geo.name}"}
    need = shape.layers * (shape.qkv_dim + shape.q_heads * 128 + 3 * shape.intermediate) * shape.hidden * 2 \
        + 2 * shape.vocab * shape.hidden * 2
    free = torch.cuda.mem_get_info(wl.device)[0]
    if need > free - (4 << 30):
        return {"unavailable": f"weights need {need / 2**30:.0f} GiB, {free / 2**30:.0f} GiB free on this GPU"}
    dec = dl.SyntheticDecoder(replace(shape, layers=geo.layers), wl.cache, geo.batch, geo.context + 4096, wl.device)
    dec.positions.fill_(geo.context + wl.static_len() - (SINK + RECENT + 1))
    dec.decode_forward()                                   # eager once, then captured
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dec.decode_forward()
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    ids_host = torch.randint(0, shape.vocab, (warm + args.steps, geo.batch), dtype=torch.int64).pin_memory()
    next_host = torch.zeros((geo.batch,), dtype=torch.int64).pin_memory()

    def run(first, count):
        for st in range(first, first + count):
            dec.input_ids.copy_(ids_host[st], non_blocking=True)
            graph.replay()
            next_host.copy_(dec.next_ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    run(0, warm)
    e0.record()
    run(warm, args.steps)
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    log(f"model step: {ms:.3f} ms resident, {ms_e2e:.3f} ms with host ids")
    return {"model": f"{geo.name.split('-128k')[0]} shapes, random-init bf16 weights (std 0.02)",
            "tok_s": round(geo.batch / ms * 1e3, 1), "ms_per_step": round(ms, 4),
            "e2e_tok_s": round(geo.batch / ms_e2e * 1e3, 1), "weight_bytes_per_step": dec.weight_bytes_per_step(),
            "launches_per_step": 9 * geo.layers + 7,
            "note": "per layer: 3 of this library's element-wise kernels + the decode kernel + 4 library GEMMs"}


def measure_steps(wl, args, warm, rank, world, local_rank, dist, cpu_group):
    """Times ``args.steps`` decode steps twice — inputs resident in HBM (one graph replay per step), then end to
    end with q/k/v starting in pinned host memory and the outputs ending there — each after ``warm`` untimed
    steps, between barriers, with CUDA events; several ranks: the maximum over the ranks.  Returns
    (ms resident, ms end to end, clock record of rank 0, result of the gather check)."""
    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=cpu_group)

    def run_resident(first, count):
        for st in range(first, first + count):
            wl.q_in.copy_(wl.q_all[st]); wl.k_in.copy_(wl.k_all[st]); wl.v_in.copy_(wl.v_all[st])
            wl.replay()

    run_resident(0, warm)
    barrier()
    sampler = ClockSampler(local_rank)     # samples over both timed regions
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_resident(warm, args.steps)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)

    base = warm + args.steps
    q_host, k_host, v_host = (t.cpu().pin_memory() for t in (wl.q_all, wl.k_all, wl.v_all))
    out_host = torch.empty(wl.out.shape, dtype=wl.out.dtype).pin_memory()

    def run_e2e(first, count):
        for st in range(first, first + count):
            wl.q_in.copy_(q_host[st], non_blocking=True)
            wl.k_in.copy_(k_host[st], non_blocking=True)
            wl.v_in.copy_(v_host[st], non_blocking=True)
            wl.replay()
            out_host.copy_(wl.out, non_blocking=True)
            torch.cuda.current_stream().synchronize()    # the caller consumes this step's output

    run_e2e(base, warm)
    barrier()
    e0.record()
    run_e2e(base + warm, args.steps)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    gather_check = None
    if world > 1:
        t = torch.tensor([ms, ms_e2e])
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=cpu_group)
        ms, ms_e2e = t.tolist()
        if wl.peer is not None:
            # every rank's slice of the last step must have arrived in this rank's gather buffer: compare
            # per-layer sums of the ranks' own outputs with the sums of the slices received
            torch.cuda.synchronize()
            mine = wl.out.float().sum(dim=tuple(range(1, wl.out.dim()))).cpu()
            sums = [None] * world
            dist.all_gather_object(sums, mine, group=cpu_group)
            got = wl.peer.gathered.float().sum(dim=(2, 3, 4, 5)).cpu()
            ok = not wl.peer.timed_out()
            for slot, r in enumerate(wl.shard.head_group_ranks()):
                ok = ok and bool(torch.allclose(got[:, slot], sums[r], rtol=1e-3, atol=1e-2))
            flags = torch.tensor([1.0 if ok else 0.0])
            dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=cpu_group)
            gather_check = "ok" if flags.item() == 1.0 else "MISMATCH"
            if rank == 0:
                gather_check += " " + json.dumps(wl.peer.wait_times_us())
    return ms, ms_e2e, clocks, gather_check


# ----------------------------------------------------------------------------------------------
# decode benchmark
# ----------------------------------------------------------------------------------------------
def run_decode(geo, args, rank, world, local_rank, log):
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist, cpu_group = None, None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION", "WARN"):
            os.environ["NCCL_DEBUG"] = "ERROR"     # keep NCCL's banner off stdout: one JSON line only
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
        # Host-side barriers and the max-over-ranks reduction go over gloo, so that no eager NCCL collective
        # is ever issued on a communicator that also carries graph-captured work.
        cpu_group = dist.new_group(backend="gloo")

    warm = max(args.warmup, 3)
    stage_steps = min(args.steps, 4)
    total = 2 * (warm + args.steps) + stage_steps + 2
    with_model = world == 1 and not args.no_model
    if with_model:
        total += 2 * (warm + args.steps) + 2      # the model run appends to the same steady zones
    wl = Workload(geo, device, total, args.kmeans_iters, rank, log, world)
    wl.capture()      # consumes 2 steps of the steady zone
    ms, ms_e2e, clocks, gather_check = measure_steps(wl, args, warm, rank, world, local_rank, dist, cpu_group)

    # ---- per-kernel time and roofline (separate eager pass, events around each launch) ----
    stage_ms, n_ret_rows, static_len = time_stages(wl, 2 * (warm + args.steps), stage_steps)
    peak, _, peak_kind = measured_peaks()
    alg = algorithmic_bytes(wl, n_ret_rows, static_len)
    # the library's switch to the three-kernel form, which it also takes beyond 8192 centroids
    staged = os.environ.get("RI_WAVE_STAGED", "0") not in ("", "0") or wl.cfg.n_centroids > 8192
    alg["decode"] = sum(alg.values())                # the single kernel does all three stages' work
    kernels = {n: {"ms": round(stage_ms[n], 5), "alg_bytes": int(alg[n]), "gbs": round(alg[n] / stage_ms[n] / 1e6, 1),
                   "frac": round(alg[n] / stage_ms[n] / 1e6 / peak, 4)} for n in stage_ms}
    top = max(("scan", "select", "attend"), key=stage_ms.get) if staged else "decode"
    kernel_name = {"decode": "wave_fused_kernel"}.get(top, "wave_" + top + "_kernel")
    # measured DRAM traffic of one launch (ncu capture of this geometry with 32 groups), scaled by this rank's groups
    traffic = None
    if geo.name.startswith("llama3-8b-128k") and NCU_TRAFFIC[top]:
        traffic = int(NCU_TRAFFIC[top] * wl.shape.groups / 32)
    step_alg = alg["decode"] * geo.layers
    tokens = geo.batch * world * args.steps
    cfg = wl.cfg
    lg = wl.geo
    result = {
        "metric": METRIC, "value": round(tokens / (ms / 1e3), 2), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{geo.name}: wave-index decode attention hot path through retroinfer_cache "
                               f"(decode_update_kv_cache + compute), {geo.layers} layers, {geo.q_heads}q/{geo.kv_heads}kv "
                               f"heads, d128, global batch {geo.batch * world}, ctx {geo.context}, {cfg.n_centroids} "
                               f"centroids, {cfg.n_segment} segments, nprobe {cfg.nprobe}, estimate {wl.shape.n_estimate}",
                   "parallelism": (f"{world} ranks: {wl.shard.head_shards} KV-head shards x {wl.shard.batch_shards} batch "
                                   f"shards; per rank {lg.kv_heads} kv heads x batch {lg.batch} = {wl.shape.groups} groups; "
                                   + ("head slices stored into every rank's gather buffer by the decode kernel "
                                      "(peer stores over NVLink), one flag exchange with a bounded wait per layer"
                                      if wl.peer is not None else "one NCCL all-gather of the head slices per layer"))
                                  if world > 1 else "single GPU",
                   "l2": "inputs larger than L2 (each layer-step touches its own ~110 MB; ~3.5 GB per step)",
                   "index": f"built by ri_kmeans_build during untimed set-up ({args.kmeans_iters} iterations, "
                            f"median {wl.prefill_index_ms:.1f} ms per request-layer incl. layout)",
                   "gather_check": gather_check,    # "ok" + the flag wait's microseconds per layer on rank 0 (last step)
                   "graph": "one CUDA graph per decode step" if wl.graph is not None else
                            "eager stepping (capture failed: " + getattr(wl, "capture_error", "?") + ")"},
        "e2e": {"value": round(tokens / (ms_e2e / 1e3), 2), "unit": "tok/s",
                "h2d_bytes_per_step": int(2 * (wl.q_in.numel() + wl.k_in.numel() + wl.v_in.numel())),
                "d2h_bytes_per_step": int(2 * wl.out.numel())},
        "gpu_launches": wl.launches_per_step() * args.steps,
        "nccl_collectives": (geo.layers * args.steps) if (world > 1 and wl.peer is None) else 0,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": kernels[top]["gbs"], "peak": peak,
                     "unit": "GB/s", "frac": kernels[top]["frac"], "peak_kind": "of " + peak_kind, "traffic": traffic,
                     "kernels": kernels,
                     "kernels_note": "decode = the one kernel per layer the step launches (wave_fused_kernel); scan/select/"
                                     "attend = the same work as three stage kernels (RI_WAVE_STAGED=1); all are marginal "
                                     "times per layer from CUDA graphs over all layers",
                     "path": {"alg_bytes_per_step": int(step_alg), "gbs": round(step_alg / (ms / args.steps) / 1e6, 1),
                              "frac": round(step_alg / (ms / args.steps) / 1e6 / peak, 4)}},
    }
    cfgd = result["config"]
    cfgd["kernels"] = "; ".join(f"{n} {k['ms'] * 1e3:.1f}us {k['gbs']:.0f}GB/s {k['frac']:.3f}" for n, k in kernels.items())
    if with_model:
        dm = result["decode_model"] = model_decode(wl, geo, args, warm, log)
        mb = dm.get("weight_bytes_per_step")
        if mb:
            gbs = (mb + step_alg) / dm["ms_per_step"] / 1e6
            dm.update({"gbs": round(gbs, 1), "frac": round(gbs / peak, 4)})
            cfgd["decode_model"] = (f"whole model step: {dm['tok_s']} tok/s ({dm['ms_per_step']} ms/step), {dm['e2e_tok_s']} tok/s "
                                    f"with host token ids, {gbs:.0f} GB/s = {gbs / peak:.3f} of peak")
        else:
            cfgd["decode_model"] = dm.get("unavailable", "unavailable")
    if world == 1 and not args.no_cpu_baseline:
        parity, sec = layer_parity(wl, 0, warm)
        result["parity"] = parity
        cfgd["parity"] = (f"layer 0, {geo.groups} groups vs CPU oracle: " + ("ok" if parity["ok"] else "FAILED")
                          + f", max_abs {parity['max_abs']}, mean_abs {parity['mean_abs']}, sets "
                          + f"{parity['retrieval_sets_ok']}/{parity['estimation_sets_ok']}, kept {parity['kept_ok']}")
        result["cpu_baseline"] = {"value": round(geo.batch / (sec * geo.layers), 3), "unit": "tok/s",
                                  "cores": os.cpu_count(), "kind": "port",
                                  "sample": f"layer 0 of the same workload, all {geo.groups} groups, median of 2 runs "
                                            f"({sec * 1e3:.1f} ms), scaled by {geo.layers} layers"}
    if world == 1 and not args.no_cpu_baseline:
        rg = reference_gpu_sequence(wl, min(args.steps, 8))
        if rg is not None:
            ours = stage_ms["scan"] + stage_ms["select"]
            rg["this_library_scan_plus_select_ms_per_layer"] = round(ours, 4)
            result["reference_gpu"] = rg
            cfgd["reference_gpu"] = (f"reference's own kernels (scores+softmax, topk, estimation gather): {rg['ms_per_layer'] * 1e3:.1f} us "
                                     f"per layer; same work here (scan + select stage kernels): {ours * 1e3:.1f} us; whole layer "
                                     f"here (single kernel, attention included): {stage_ms['decode'] * 1e3:.1f} us")
    if world == 1 and not args.no_kmeans and args.config == "cfg1":
        pf = prefill_summary(geo, log)
        result["prefill_attn"] = pf
        cfgd["prefill_attn"] = (f"S=16384 causal: {pf['ms']} ms, {pf['tflops']} TFLOP/s = {pf['frac']} of bf16 peak; flash-attn "
                                f"library on the same tensors: {pf.get('flash_attn_library_tflops', 'n/a')} TFLOP/s")
        km = kmeans_summary(GEOMETRIES["cfg2"], args, log)
        result["kmeans"] = km
        cfgd["kmeans"] = (f"cfg2 build {km['ms']} ms, {km['tflops']} TFLOP/s = {km['frac']} of sustained bf16 peak "
                          f"({km['frac_of_burst_peak']} of burst)")
    if world > 1 and not args.no_cfg4 and args.config == "cfg1":
        # configuration 4 (Qwen2.5-72B geometry, KV heads sharded over the ranks, batch 16) on the same ranks
        wl.graph = wl.cache = wl.peer = wl.gather = None
        del wl
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        c4 = run_cfg4(args, rank, world, local_rank, device, dist, cpu_group, log)
        result["cfg4"] = c4
        cfgd["cfg4"] = (f"{c4['layers']} of 80 layers: {c4['ms_per_step']} ms/step, {c4['tok_s']} tok/s "
                        f"({c4['tok_s_at_80_layers']} at 80 layers), e2e {c4['e2e_tok_s']}, gather {c4['gather_check']}")
    if world == 1 and not args.no_host_tier and not args.layers and args.config == "cfg1":
        # the host tier in short (configuration 3's geometry): the caches of the workload above are released first
        wl.graph = wl.cache = None
        del wl
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        ht = result["host_tier"] = host_tier_summary(args, log)
        best, ref = ht["results"]["pull, one layer ahead"], ht["results"]["uva (the reference's pattern)"]
        full = GEOMETRIES["cfg3"]
        at_model = lambda r: round(full.batch / (r["ms_per_layer"] * 1e-3 * full.layers), 1)   # noqa: E731
        cfgd["host_tier"] = ("cfg3 geometry, 2 layers timed, KV in pinned host memory: "
                             + "; ".join(f"{k}: {best[k]['ms_per_layer']} ms/layer = {at_model(best[k])} tok/s at the model's "
                                         f"{full.layers} layers, {best[k]['missed_page_gbs']} GB/s of missed pages (the "
                                         f"reference's pattern: {ref[k]['ms_per_layer']} ms/layer)"
                                         for k in ("fresh queries", "drifting queries")))
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier(group=cpu_group)


def run_cfg4(args, rank, world, local_rank, device, dist, cpu_group, log):
    """Configuration 4 on the ranks of this run: 64 q / 8 kv heads (gs 8), batch 16, context 131072, the KV heads
    sharded over the ranks (8 ranks: one head each), the head slices gathered by the decode kernel's peer stores.
    As many of the 80 layers as fit beside the allocator's leftovers (all 80 at 8 ranks)."""
    from retrievalattention_b200.head_shard import HeadShard

    geo = GEOMETRIES["cfg4"]
    shard = HeadShard(rank, world, geo.kv_heads, geo.q_heads, geo.batch)
    cfg = geo.index()
    groups = shard.local_kv_heads * shard.local_batch
    per_layer = groups * ((geo.context - SINK - RECENT) * 512 + cfg.n_centroids * (512 + 16) + 4096 * 512)
    free = torch.cuda.mem_get_info(device)[0]
    layers = torch.tensor([min(geo.layers, int((free - (20 << 30)) // per_layer))])
    dist.all_reduce(layers, op=dist.ReduceOp.MIN, group=cpu_group)
    layers = max(int(layers.item()), 1)
    steps, warm = min(args.steps, 16), 3
    sub = argparse.Namespace(**{**vars(args), "steps": steps})
    wl = Workload(replace(geo, layers=layers), device, 2 * (warm + steps) + 4, args.kmeans_iters, rank, log, world, weak=False)
    wl.capture()
    ms, ms_e2e, _, gather_check = measure_steps(wl, sub, warm, rank, world, local_rank, dist, cpu_group)
    ms_step = ms / steps
    out = {"workload": f"{geo.name}: {geo.q_heads}q/{geo.kv_heads}kv heads, batch {geo.batch}, ctx {geo.context}, "
                       f"{cfg.n_centroids} centroids, nprobe {cfg.nprobe}; per rank {shard.local_kv_heads} kv heads x batch "
                       f"{shard.local_batch} = {groups} groups, gs {geo.q_heads // geo.kv_heads}",
           "layers": layers, "steps": steps, "ms_per_step": round(ms_step, 4), "ms_per_layer": round(ms_step / layers, 5),
           "tok_s": round(geo.batch / ms_step * 1e3, 1),
           "tok_s_at_80_layers": round(geo.batch / (ms_step / layers * geo.layers) * 1e3, 1),
           "e2e_tok_s": round(geo.batch * steps / ms_e2e * 1e3, 1), "gather_check": gather_check,
           "scaling": "strong (batch 16 fixed, a rank's share of the heads shrinks with the ranks)"}
    wl.graph = wl.cache = wl.peer = None
    return out


HOST_TIER_MODES = {"pull, one layer ahead": ("pull", True), "pull": ("pull", False), "staged": ("staged", False),
                   "uva (the reference's pattern)": ("uva", False)}


def host_tier_measure(geo, modes, steps, warm, device, log, rank=0, world=1, dist=None):
    """Eager decode steps of ``geo`` (one rank's share) on the host tier for each of ``modes`` (name -> (miss path,
    look ahead)), with fresh Gaussian queries every step (no temporal locality: the worst case for the page cache) and
    with slowly drifting ones (q_t = 0.95 q_{t-1} + 0.31 noise).  Wall clock (the host takes part in every layer)."""
    from retrievalattention_b200.cache_hub import retroinfer_cache

    cfg = geo.index()
    max_new = 2 * len(modes) * (steps + warm) + 4
    mapping = {str(l): str(device) for l in range(geo.layers)}
    results, cache, built = {}, None, None
    for mode, (path, ahead) in modes.items():
        if built != path:
            cache = None
            torch.cuda.empty_cache()
            cache = retroinfer_cache([0] * geo.batch, geo.layers, geo.batch, geo.context + max_new, geo.kv_heads, geo.q_heads,
                                     128, torch.bfloat16, mapping, max_new, num_gpus=1, model_size=8, kv_on_host=True,
                                     miss_path=path, use_cluster_estimation=path == "pull", **cfg.as_kwargs())
            for l in range(geo.layers):
                for b in range(geo.batch):
                    k, v = make_kv(geo.kv_heads, geo.context, 128, seed=(rank * 131 + l) * 1000 + b, theta=geo.rope_theta, device=device)
                    cache.prefill_update_kv_cache(None, k, v, l, b)
            cache.prepare_cache()
            built = path
            log(f"host tier set-up: {geo.layers} layers indexed, miss path {path}")
        g = torch.Generator(device=device).manual_seed(5 + rank)
        rnd = lambda h: torch.randn((geo.batch, 1, h, 128), generator=g, device=device).to(torch.bfloat16)   # noqa: E731
        results[mode] = {}
        for name, keep in (("fresh queries", 0.0), ("drifting queries", 0.95)):
            q = [rnd(geo.q_heads).float() for _ in range(geo.layers)]
            pages = [0, 0]

            def step(count):
                qs = []
                for l in range(geo.layers):
                    q[l] = keep * q[l] + (1 - keep * keep) ** 0.5 * rnd(geo.q_heads).float()
                    qs.append(q[l].to(torch.bfloat16))
                for l in range(geo.layers):
                    cache.decode_update_kv_cache(rnd(geo.kv_heads), rnd(geo.kv_heads), l)
                    cache.compute(qs[l], l, qs[l + 1] if ahead and l + 1 < geo.layers else None)
                    if count:
                        pages[0] += int(cache.page_lists[l][3].sum())
                        pages[1] += int(cache.page_lists[l][7].sum())
            for _ in range(warm):
                step(False)
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                step(True)
            torch.cuda.synchronize()
            sec = time.perf_counter() - t0
            hit, miss = pages
            if dist is not None:          # the slowest rank's time, everybody's pages
                t = torch.tensor([sec], dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                pg = torch.tensor([hit, miss], dtype=torch.int64)
                dist.all_reduce(pg)
                sec, hit, miss = float(t[0]), int(pg[0]), int(pg[1])
            results[mode][name] = {"tok_s": round(geo.batch * world * steps / sec, 1), "ms_per_step": round(sec / steps * 1e3, 3),
                                   "ms_per_layer": round(sec / steps / geo.layers * 1e3, 3),
                                   "page_hit_rate": round(hit / max(hit + miss, 1), 4),
                                   "missed_page_gbs": round(miss * 8 * 128 * 2 * 2 / sec / 1e9, 2)}
            log(f"{mode}, {name}: {results[mode][name]}")
    cache = None
    torch.cuda.empty_cache()
    return results


def run_host_tier(geo, args, log, rank=0, world=1, local_rank=0):
    """``--kv-on-host``: the configuration's geometry with the cluster store in pinned host memory and an LRU page cache
    on the GPU (the reference's tiers), ``--layers`` of its layers (pinned memory is the limit), eager stepping.
    Reports tokens/s, the page cache's hit rate and the host-to-device bytes of the missed pages per second, for every
    way of bringing the missed pages up (``--miss-path`` picks one): the side-stream pull with the next layer searched
    and pulled one layer ahead (the next layer's query handed over as ``queries_next``: the best any estimate can do),
    the same without looking ahead, the host-staged copy, and the reference's own pattern."""
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        # several GPUs: the batch is split over the ranks, which do not exchange anything (every rank has its own
        # PCIe link, host threads and page caches); gloo carries the barriers and the sums
        import torch.distributed as dist
        dist.init_process_group("gloo")
        if geo.batch % world:
            raise SystemExit(f"batch {geo.batch} does not split over {world} ranks")
        geo = replace(geo, batch=geo.batch // world)
    cfg = geo.index()
    steps, warm = args.steps, max(args.warmup, 3)
    modes = dict(HOST_TIER_MODES)
    if args.miss_path:
        modes = {k: v for k, v in modes.items() if v[0] == args.miss_path}
    results = host_tier_measure(geo, modes, steps, warm, device, log, rank, world, dist)
    if rank != 0:
        return
    first = next(iter(results))
    main = results[first]["drifting queries"]
    print(json.dumps({
        "metric": METRIC, "value": main["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{geo.name}: host tier (cluster store in pinned host memory, GPU page cache of "
                               f"{cfg.cache_cluster_num} clusters per group), {geo.layers} layers, batch {geo.batch} per GPU, ctx {geo.context}, "
                               f"{cfg.n_centroids} centroids, nprobe {cfg.nprobe}; value: drifting queries, missed pages by '{first}'",
                   "timing": "wall clock around eager steps (the host takes part in every layer)"},
        "host_tier": results}), flush=True)


def host_tier_summary(args, log):
    """The host tier in short, for the default line: configuration 3's geometry (Qwen2.5-7B, context 262144, batch 8) with
    2 of its layers, the side-stream pull one layer ahead and the reference's own pattern beside it."""
    geo = replace(GEOMETRIES["cfg3"], layers=2, name=GEOMETRIES["cfg3"].name + "-2layers")
    modes = {k: HOST_TIER_MODES[k] for k in ("pull, one layer ahead", "uva (the reference's pattern)")}
    res = host_tier_measure(geo, modes, 8, 3, torch.device("cuda", 0), log)
    cfg = geo.index()
    return {"workload": f"{geo.name}: cluster store in pinned host memory, GPU page cache of {cfg.cache_cluster_num} clusters per "
                        f"group, batch {geo.batch}, ctx {geo.context}, {cfg.n_centroids} centroids, nprobe {cfg.nprobe}; eager steps, "
                        "wall clock; fresh queries = no temporal locality, drifting = q_t = 0.95 q_(t-1) + noise",
            "results": res}


def reference_arm(geo, args, log):
    """The reference's own arithmetic for this path on the host cores (oracle port): each step is one
    layer of the workload (all groups), scaled to a full decode step."""
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "set-up of the synthetic index needs the GPU box"}))
        return
    warm = max(args.warmup, 1)
    wl = Workload(replace(geo, layers=1), torch.device("cuda", 0), warm + args.steps + 2, args.kmeans_iters, 0, log)
    secs = [cpu_layer_seconds(wl, 0, st, 1) for st in range(warm + args.steps)][warm:]
    sec = sum(secs) / len(secs)
    val = round(geo.batch / (sec * geo.layers), 3)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(sec * geo.layers * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{geo.name}: wave-index decode attention hot path on host cores"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": f"each step = layer 0 of the workload (all {geo.groups} groups), scaled by "
                                   f"{geo.layers} layers"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ----------------------------------------------------------------------------------------------
# clustering benchmark (config 2)
# ----------------------------------------------------------------------------------------------
def kmeans_inputs(geo, device):
    ks, vs = [], []
    for b in range(geo.batch):
        k, v = make_kv(geo.kv_heads, geo.context, 128, seed=b, theta=geo.rope_theta, device=device)
        ks.append(k[0].transpose(0, 1)); vs.append(v[0].transpose(0, 1))
    return torch.cat(ks, 0).contiguous(), torch.cat(vs, 0).contiguous()


def sustained_and_burst_tflops():
    _, burst, kind = measured_peaks()
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            sustained = json.load(f).get("bf16_tflops_sustained")
        if sustained:
            return float(sustained), burst, kind + " (sustained)"
    return burst, burst, kind


def kmeans_summary(geo, args, log):
    """Configuration 2 in short, for the default line: two warm builds, three timed (reference schedule).  Two,
    because a build's outputs are new tensors and the previous result is released only when the next one is bound:
    the allocator needs both sets before the timed builds stop calling cudaMalloc."""
    from retrievalattention_b200.cache_hub.kmeans import build_index

    device = torch.device("cuda", 0)
    cfg = geo.index()
    keys, values = kmeans_inputs(geo, device)
    for _ in range(2):
        r = build_index(keys, values, cfg.n_centroids, cfg.n_segment, args.kmeans_iters)
    torch.cuda.synchronize()
    assert int(r["error"]) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        r = build_index(keys, values, cfg.n_centroids, cfg.n_segment, args.kmeans_iters)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    it = args.kmeans_iters
    flop = 2.0 * geo.groups * geo.context * 128 * (cfg.n_centroids * (it - 1) / cfg.n_segment + cfg.n_centroids)
    sustained, burst, kind = sustained_and_burst_tflops()
    tf = flop / ms / 1e9
    log(f"k-means (cfg2): {ms:.2f} ms, {tf:.1f} TFLOP/s")
    return {"workload": f"ri_kmeans_build: {geo.groups} groups x {geo.context} keys x d128, {cfg.n_centroids} centroids, "
                        f"{cfg.n_segment} segments, {it} iterations, incl. centring, value sums and layout",
            "ms": round(ms, 3), "tflops": round(tf, 1), "bound": "tensor", "peak": sustained, "peak_kind": "of " + kind,
            "frac": round(tf / sustained, 4), "frac_of_burst_peak": round(tf / burst, 4)}


def prefill_summary(geo, log, seq=16384):
    """Dense causal prefill attention of one request at the model's head geometry: this library's tcgen05 kernel
    (through ``retroinfer_prefill_attn``) and, beside it, the flash-attn library call the reference makes
    (attn_hub/retroinfer_attn.py:4-13), on the same tensors.  TFLOP/s over 4*S^2*d*Hq/2 flops."""
    from retrievalattention_b200.attn_hub import retroinfer_attn as ra

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(7)
    mk = lambda h: torch.randn((1, seq, h, 128), generator=g, device=dev).to(torch.bfloat16)   # noqa: E731
    q, k, v = mk(geo.q_heads), mk(geo.kv_heads), mk(geo.kv_heads)
    flop = 4.0 * seq * seq * 128 * geo.q_heads / 2

    def timed(fn, reps=5):
        for _ in range(2):
            out = fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, out

    ms, out = timed(lambda: ra.retroinfer_prefill_attn(q, k, v, True))
    ra.check_prefill_errors()
    _, burst, kind = measured_peaks()
    res = {"workload": f"causal attention over one prompt of {seq} tokens, {geo.q_heads}q/{geo.kv_heads}kv heads, d128, bf16 "
                       "(V transposed inside the call)",
           "ms": round(ms, 3), "tflops": round(flop / ms / 1e9, 1), "bound": "tensor", "peak": burst,
           "peak_kind": "of " + kind, "frac": round(flop / ms / 1e9 / burst, 4)}
    try:
        from flash_attn import flash_attn_with_kvcache
        ms_lib, out_lib = timed(lambda: flash_attn_with_kvcache(q=q, k_cache=k, v_cache=v, causal=True))
        res["flash_attn_library_ms"] = round(ms_lib, 3)
        res["flash_attn_library_tflops"] = round(flop / ms_lib / 1e9, 1)
        res["max_abs_diff_to_library"] = round(float((out.float() - out_lib.float()).abs().max()), 5)
    except Exception as exc:      # noqa: BLE001 — the comparison is optional
        res["flash_attn_library"] = "unavailable: " + repr(exc)[:120]
    log(f"prefill attention: {res}")
    return res


def run_kmeans(geo, args, log):
    from retrievalattention_b200.cache_hub.kmeans import build_index

    device = torch.device("cuda", 0)
    cfg = geo.index()
    n = geo.context
    keys, values = kmeans_inputs(geo, device)
    results = {}
    schedules = (("reference schedule", cfg.n_segment),) if args.quick else \
        (("reference schedule", cfg.n_segment), ("plain Lloyd", 1))
    for label, segs in schedules:
        warm = max(args.warmup, 3) if segs > 1 else 1
        reps = min(args.steps, 5) if segs > 1 else 2
        if args.quick:
            warm, reps = 1, 1
        for _ in range(warm):
            r = build_index(keys, values, cfg.n_centroids, segs, args.kmeans_iters)
        torch.cuda.synchronize()
        assert int(r["error"]) == 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            r = build_index(keys, values, cfg.n_centroids, segs, args.kmeans_iters)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        g, c, it = geo.groups, cfg.n_centroids, args.kmeans_iters
        flop = 2.0 * g * n * 128 * (c * (it - 1) / segs + c)
        results[label] = {"segments": segs, "ms": round(ms, 3), "tflops": round(flop / ms / 1e9, 1), "flop": flop}
        log(f"{label}: {ms:.2f} ms, {flop / ms / 1e9:.1f} TFLOP/s")
    # builds run back to back for tens of milliseconds: the sustained matmul figure is the denominator
    peak_tf, burst_tf, kind = sustained_and_burst_tflops()
    main = results["reference schedule"]
    print(json.dumps({
        "metric": "prefill k-means clustering time (config 2)", "value": main["ms"], "unit": "ms", "n_gpus": 1,
        "steps": min(args.steps, 5), "warmup": max(args.warmup, 3), "ms_per_step": main["ms"], "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"ri_kmeans_build: {geo.groups} groups x {n} keys x d128, {cfg.n_centroids} centroids, "
                               f"{args.kmeans_iters} iterations, centring + value sums + cluster-contiguous layout",
                   "l2": "inputs larger than L2 (1.07 GB of keys)"},
        "roofline": {"bound": "tensor", "achieved": main["tflops"], "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": round(main["tflops"] / peak_tf, 4), "peak_kind": "of " + kind,
                     "frac_of_burst_peak": round(main["tflops"] / burst_tf, 4),
                     "note": "whole build (centring, assignment, bucket, update, layout) over the assignment GEMM's flops",
                     "traffic": None, "schedules": results},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="cfg1", choices=sorted(GEOMETRIES))
    ap.add_argument("--layers", type=int, default=0, help="override layer count (profiling on a small case only)")
    ap.add_argument("--kmeans-iters", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-model", action="store_true",
                    help="skip the whole-model decode step (projections, MLP, vocabulary head with random weights around "
                         "the same caches; key decode_model, single GPU)")
    ap.add_argument("--no-kmeans", action="store_true", help="skip the short clustering run (key kmeans, single GPU)")
    ap.add_argument("--kv-on-host", action="store_true",
                    help="time the host tier of --config (cluster store in pinned host memory, GPU page cache), --layers layers")
    ap.add_argument("--miss-path", default="", choices=["", "pull", "staged", "uva"],
                    help="with --kv-on-host: only this way of bringing missed pages up (default: all, one after the other)")
    ap.add_argument("--no-host-tier", action="store_true", help="skip the short host-tier run (key host_tier, single GPU)")
    ap.add_argument("--no-cfg4", action="store_true",
                    help="several GPUs: skip the run of configuration 4 (72B geometry, heads sharded) after the main one")
    ap.add_argument("--quick", action="store_true", help="cfg2 only: one warm-up, one repetition (profiler captures)")
    ap.add_argument("--prefill-seq", type=int, default=0,
                    help="only the dense prefill attention of one prompt of this many tokens (profiler captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    log = (lambda m: print(f"[bench] {m}", file=sys.stderr, flush=True)) if rank == 0 else (lambda m: None)

    geo = GEOMETRIES[args.config]
    if args.layers:
        geo = replace(geo, layers=args.layers, name=geo.name + f"-{args.layers}layers")
    if args.impl == "reference":
        if rank == 0:
            reference_arm(geo, args, log)
        return
    if args.prefill_seq:
        if rank == 0:
            print(json.dumps({"prefill_attn": prefill_summary(geo, log, args.prefill_seq)}), flush=True)
        return
    if args.config == "cfg2":
        if rank == 0:
            run_kmeans(geo, args, log)
        return
    if args.kv_on_host:
        run_host_tier(geo, args, log, rank, world, local_rank)
        return
    run_decode(geo, args, rank, world, local_rank, log)
    if world > 1:
        # leave without tearing the NCCL communicator down (a teardown after graph-captured collectives
        # has been seen not to return); everything has been printed and flushed
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
