#!/usr/bin/env python
"""Decode-throughput benchmark of the wave-index attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1): Llama-3-8B decode-attention geometry — 32 layers, 32 q / 8 kv heads, head_dim
128, batch 4, context 131072, 8192 centroids per kv head, budget 0.018, estimate 0.232 —
on seeded synthetic bf16 K/V/q.  One step = one decode step of the hot path over all layers:
per layer the new token's K/V is appended to the steady zone and the wave-index attention
(centroid scan, cluster selection, weighted flash decoding) runs for every request.

Prints ONE JSON line (rank 0).  ``value`` is tokens/s with every input resident in HBM, the
whole step replayed as one CUDA graph; ``e2e`` is the same step with q/k/v starting in pinned
host memory and the attention output copied back to the host inside the timed region.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from retrievalattention_b200.config import GEOMETRIES  # noqa: E402
from retrievalattention_b200.synthetic import make_kv  # noqa: E402

SINK, RECENT = 4, 64
FALLBACK_HBM_GBS = 6650.0


# ----------------------------------------------------------------------------------------------
# set-up (untimed): synthetic KV and its wave index, built on the device
# ----------------------------------------------------------------------------------------------
def lloyd_assign(data, cent, chunk=8192):
    """argmax_c <x, c> with bf16 operands and fp32 accumulation; data [Z,N,d], cent [Z,C,d]."""
    z, n, _ = data.shape
    out = torch.empty((z, n), dtype=torch.int64, device=data.device)
    ct = cent.transpose(1, 2).float()
    for s in range(0, n, chunk):
        out[:, s:s + chunk] = torch.bmm(data[:, s:s + chunk].float(), ct).argmax(-1)
    return out


def lloyd_step(data, cent, normalize):
    z, n, d = data.shape
    c = cent.shape[1]
    idx = lloyd_assign(data, cent)
    flat = (idx + torch.arange(z, device=data.device)[:, None] * c).reshape(-1)
    sums = torch.zeros((z * c, d), dtype=torch.float32, device=data.device)
    sums.index_add_(0, flat, data.reshape(-1, d).float())
    cnt = torch.bincount(flat, minlength=z * c).reshape(z, c)
    x = sums.reshape(z, c, d) / cnt[..., None].float()
    if normalize:
        x = x / torch.sqrt((x * x).sum(-1, keepdim=True))
    return torch.where(cnt[..., None] > 0, x.to(cent.dtype), cent), idx, cnt


def build_index_setup(keys, values, n_centroids, n_segment, iters):
    """Set-up only (untimed): the reference's segmented Lloyd schedule
    (cache_hub/kmeans.py:224-259) with library GEMMs, producing the layout the decode kernels
    read.  keys/values [Z, N, d] (mid-context tokens of every group of the layer)."""
    z, n, d = keys.shape
    mean = keys.float().mean(1, keepdim=True).to(keys.dtype)
    x = keys - mean
    init = (torch.arange(n_centroids, dtype=torch.float32, device=keys.device) * (n / n_centroids)
            + n / n_centroids / 2).to(torch.int64)
    cent = x[:, init].contiguous()
    n_seg, c_seg = n // n_segment, n_centroids // n_segment
    data = x[:, :n_seg * n_segment].reshape(-1, n_seg, d)
    cent = cent.reshape(-1, c_seg, d)
    for _ in range(iters - 1):
        cent, _, _ = lloyd_step(data, cent, True)
    cent = cent.reshape(z, n_centroids, d)
    cent, idx, cnt = lloyd_step(x, cent, False)
    order = torch.argsort(idx, dim=1, stable=True)
    gather = order[..., None].expand(-1, -1, d)
    csr_k = torch.gather(keys, 1, gather)
    csr_v = torch.gather(values, 1, gather)
    flat = (idx + torch.arange(z, device=keys.device)[:, None] * n_centroids).reshape(-1)
    vsum = torch.zeros((z * n_centroids, d), dtype=torch.float32, device=keys.device)
    vsum.index_add_(0, flat, values.reshape(-1, d).float())
    offsets = torch.zeros((z, n_centroids + 1), dtype=torch.int32, device=keys.device)
    offsets[:, 1:] = torch.cumsum(cnt, 1).to(torch.int32)
    return dict(centroids=(cent + mean).contiguous(), value_sum=vsum.reshape(z, n_centroids, d).to(keys.dtype),
                cluster_size=cnt.to(keys.dtype), cluster_count=cnt.to(torch.int32), cluster_offset=offsets,
                keys=csr_k.contiguous(), values=csr_v.contiguous())


def build_layer_tensors(geo, idx_cfg, layer, device, max_new, kmeans_iters, rank=0):
    """All groups of one layer: synthetic K/V per request, index, steady zone."""
    ks, vs = [], []
    for b in range(geo.batch):
        k, v = make_kv(geo.kv_heads, geo.context, geo.head_dim, seed=(rank * 131 + layer) * 1000 + b,
                       theta=geo.rope_theta, device=device)
        ks.append(k[0].transpose(0, 1))
        vs.append(v[0].transpose(0, 1))
    k = torch.cat(ks, 0)      # [G, ctx, d]
    v = torch.cat(vs, 0)
    del ks, vs
    mid = slice(SINK, geo.context - RECENT)
    t = build_index_setup(k[:, mid].contiguous(), v[:, mid].contiguous(), idx_cfg.n_centroids, idx_cfg.n_segment,
                          kmeans_iters)
    stride = SINK + RECENT + max_new
    for name, src in (("steady_keys", k), ("steady_values", v)):
        s = torch.zeros((k.shape[0], stride, geo.head_dim), dtype=k.dtype, device=device)
        s[:, :SINK] = src[:, :SINK]
        s[:, SINK:SINK + RECENT] = src[:, geo.context - RECENT:]
        t[name] = s
    return t


class Workload:
    """The resident state of one rank: every layer's index and the per-step inputs."""

    def __init__(self, geo, device, total_steps, kmeans_iters=10, rank=0, log=None):
        from retrievalattention_b200 import wave

        self.geo, self.device = geo, device
        self.cfg = geo.index()
        cfg = self.cfg
        self.max_new = max(total_steps + 1, 8)
        n_mid = geo.context - SINK - RECENT
        pages_per_cluster = -(-(n_mid // cfg.n_centroids) // cfg.cache_unit_size)
        buffer_pages = max(cfg.nprobe * 4, 16) * pages_per_cluster    # retroinfer_cache.py:107-111
        self.shape = wave.WaveShape(geo.groups, geo.group_size, cfg.n_centroids, cfg.nprobe,
                                    cfg.max_compute_cluster_num - cfg.nprobe, cfg.cache_unit_size, buffer_pages,
                                    n_mid, SINK + RECENT + self.max_new, torch.bfloat16)
        self.scratch = wave.new_scratch(self.shape, device)
        self.static_len = torch.tensor([SINK + RECENT], dtype=torch.int32, device=device)
        self.append_pos = torch.tensor([SINK + RECENT], dtype=torch.int32, device=device)
        self.layers = []
        t0 = time.time()
        for l in range(geo.layers):
            t = build_layer_tensors(geo, cfg, l, device, self.max_new, kmeans_iters, rank)
            self.layers.append(wave.WaveIndexLayer(self.shape, static_len=self.static_len, scratch=self.scratch, **t))
            if log and (l % 8 == 7 or l == geo.layers - 1):
                torch.cuda.synchronize()
                log(f"set-up: {l + 1}/{geo.layers} layers indexed, {time.time() - t0:.1f}s, "
                    f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB")
        g = torch.Generator(device=device)
        g.manual_seed(12345 + rank)
        shp_q = (total_steps, geo.layers, geo.batch, 1, geo.q_heads, geo.head_dim)
        shp_kv = (total_steps, geo.layers, geo.batch, 1, geo.kv_heads, geo.head_dim)
        self.q_all = torch.randn(shp_q, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.k_all = torch.randn(shp_kv, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.v_all = torch.randn(shp_kv, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.q_in = torch.zeros(shp_q[1:], dtype=torch.bfloat16, device=device)
        self.k_in = torch.zeros(shp_kv[1:], dtype=torch.bfloat16, device=device)
        self.v_in = torch.zeros(shp_kv[1:], dtype=torch.bfloat16, device=device)
        self.out = torch.zeros(shp_q[1:], dtype=torch.bfloat16, device=device)
        self.graph = None

    def reset(self):
        self.static_len.fill_(SINK + RECENT)
        self.append_pos.fill_(SINK + RECENT)

    def step_body(self):
        """One decode step of the hot path over all layers, on the current stream.
        4 kernels of this library per layer: steady append, scan, select, attend."""
        from retrievalattention_b200 import wave

        self.static_len.add_(1)     # every layer of this step sees the token appended below (:559)
        for l, layer in enumerate(self.layers):
            wave.steady_append(self.k_in[l], self.v_in[l], layer.t["steady_keys"], layer.t["steady_values"],
                               self.append_pos)
            layer.compute(self.q_in[l], self.out[l])
        self.append_pos.add_(1)

    def capture(self):
        self.step_body()            # warm the kernels (function attributes, modules) outside capture
        torch.cuda.synchronize()
        self.reset()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_body()
        self.reset()

    def launches_per_step(self):
        return 4 * self.geo.layers


# ----------------------------------------------------------------------------------------------
# measurement helpers
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
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
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(wl, n_ret_rows, static_len):
    """Per layer-step, all groups: bytes that must move (bf16): centroids once, value sums of
    the estimation set, K and V of retrieved + steady rows, cluster sizes, q and out."""
    s, d = wl.shape, 128
    g = s.groups
    scan = g * (2 * d * s.n_centroids + 2 * s.group_size * d)
    select = g * 2 * s.n_centroids
    attend = 2 * d * (g * s.n_estimate + 2 * (n_ret_rows + g * static_len)) + g * 2 * 2 * s.group_size * d
    return {"scan": scan, "select": select, "attend": attend}


def time_stages(wl, steps):
    """Average device time of each kernel, CUDA events around every launch (eager pass)."""
    names = ("scan", "select", "attend")
    ev = {n: [] for n in names}
    n_ret = 0
    wl.reset()
    for st in range(steps):
        wl.q_in.copy_(wl.q_all[st]); wl.k_in.copy_(wl.k_all[st]); wl.v_in.copy_(wl.v_all[st])
        wl.static_len.add_(1)
        from retrievalattention_b200 import wave
        for l, layer in enumerate(wl.layers):
            wave.steady_append(wl.k_in[l], wl.v_in[l], layer.t["steady_keys"], layer.t["steady_values"], wl.append_pos)
            for n in names:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                layer.stage(n, wl.q_in[l], wl.out[l])
                b.record()
                ev[n].append((a, b))
            if st == steps - 1:
                n_ret += int(layer.views()["n_exact"].sum().item())
        wl.append_pos.add_(1)
    torch.cuda.synchronize()
    ms = {n: sum(a.elapsed_time(b) for a, b in ev[n]) / len(ev[n]) for n in names}
    return ms, n_ret / len(wl.layers), int(wl.static_len.item())


# ----------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle port of the reference's arithmetic on host cores
# ----------------------------------------------------------------------------------------------
def cpu_layer_seconds(wl, layer_idx, step, repeats):
    from oracle import attention as oat

    torch.set_num_threads(os.cpu_count())
    layer = wl.layers[layer_idx]
    cpu = {k: v.cpu() for k, v in layer.t.items() if k not in ("scratch", "static_len")}
    mask = cpu["cluster_count"] == 0
    q = wl.q_all[step, layer_idx].cpu()
    s = wl.shape
    times = []
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        oat.compute(q, cpu["centroids"], cpu["value_sum"], cpu["cluster_size"], mask, cpu["cluster_count"],
                    cpu["cluster_offset"], cpu["keys"], cpu["values"], cpu["steady_keys"], cpu["steady_values"],
                    SINK + RECENT + 1, s.nprobe, s.nprobe + s.n_estimate, s.page_size, s.buffer_pages)
        times.append(time.perf_counter() - t0)
    return statistics.median(times[1:])


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
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    log = (lambda m: print(f"[bench] {m}", file=sys.stderr, flush=True)) if rank == 0 else (lambda m: None)

    geo = GEOMETRIES[args.config]
    if args.layers:
        from dataclasses import replace
        geo = replace(geo, layers=args.layers, name=geo.name + f"-{args.layers}layers")

    if args.impl == "reference":
        if rank != 0:
            return
        return reference_arm(geo, args, log)

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    warm = max(args.warmup, 3)
    total = warm + args.steps
    wl = Workload(geo, device, total, args.kmeans_iters, rank, log)
    wl.capture()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- `value`: inputs resident in HBM, one graph replay per step ----
    def run_resident(first, count):
        for st in range(first, first + count):
            wl.q_in.copy_(wl.q_all[st]); wl.k_in.copy_(wl.k_all[st]); wl.v_in.copy_(wl.v_all[st])
            wl.graph.replay()

    run_resident(0, warm)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_resident(warm, args.steps)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    # ---- `e2e`: q/k/v start in pinned host memory, outputs end there ----
    wl.reset()
    q_host = wl.q_all.cpu().pin_memory(); k_host = wl.k_all.cpu().pin_memory(); v_host = wl.v_all.cpu().pin_memory()
    out_host = torch.empty(wl.out.shape, dtype=wl.out.dtype).pin_memory()

    def run_e2e(first, count):
        for st in range(first, first + count):
            wl.q_in.copy_(q_host[st], non_blocking=True)
            wl.k_in.copy_(k_host[st], non_blocking=True)
            wl.v_in.copy_(v_host[st], non_blocking=True)
            wl.graph.replay()
            out_host.copy_(wl.out, non_blocking=True)
            torch.cuda.current_stream().synchronize()    # the caller consumes this step's output

    run_e2e(0, warm)
    barrier()
    e0.record()
    run_e2e(warm, args.steps)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()

    # ---- per-kernel time and roofline (separate eager pass, events around each launch) ----
    stage_ms, n_ret_rows, static_len = time_stages(wl, min(args.steps, 8))
    if rank != 0:
        return
    peak, peak_kind = measured_peak()
    alg = algorithmic_bytes(wl, n_ret_rows, static_len)
    kernels = {n: {"ms": round(stage_ms[n], 5), "alg_bytes": int(alg[n]),
                   "gbs": round(alg[n] / stage_ms[n] / 1e6, 1), "frac": round(alg[n] / stage_ms[n] / 1e6 / peak, 4)}
               for n in stage_ms}
    top = max(stage_ms, key=stage_ms.get)
    step_alg = sum(alg.values()) * geo.layers
    tokens = geo.batch * world * args.steps
    result = {
        "metric": "decode tok/s at 128K ctx (Llama-3-8B geometry); attn kernel HBM GB/s vs peak",
        "value": round(tokens / (ms / 1e3), 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{geo.name}: wave-index decode attention hot path, {geo.layers} layers, "
                               f"{geo.q_heads}q/{geo.kv_heads}kv heads, d128, batch {geo.batch}/GPU, ctx {geo.context}, "
                               f"{wl.cfg.n_centroids} centroids, nprobe {wl.cfg.nprobe}, estimate "
                               f"{wl.shape.n_estimate}; per layer: steady append + scan + select + attend",
                   "l2": "inputs larger than L2 (each layer-step touches its own ~120 MB; 3.9 GB per step)",
                   "index": "set-up (untimed) clusters with library GEMMs on the device",
                   "graph": "one CUDA graph per decode step"},
        "e2e": {"value": round(tokens / (ms_e2e / 1e3), 2), "unit": "tok/s",
                "h2d_bytes_per_step": int(wl.q_in.numel() * 2 + wl.k_in.numel() * 2 + wl.v_in.numel() * 2),
                "d2h_bytes_per_step": int(wl.out.numel() * 2)},
        "gpu_launches": wl.launches_per_step() * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "wave_" + top + "_kernel", "achieved": kernels[top]["gbs"], "peak": peak,
                     "unit": "GB/s", "frac": kernels[top]["frac"], "peak_kind": "of " + peak_kind,
                     "traffic": None, "kernels": kernels,
                     "path": {"alg_bytes_per_step": int(step_alg), "gbs": round(step_alg / (ms / args.steps) / 1e6, 1),
                              "frac": round(step_alg / (ms / args.steps) / 1e6 / peak, 4)}},
    }
    if not args.no_cpu_baseline:
        sec = cpu_layer_seconds(wl, 0, warm, 2)
        result["cpu_baseline"] = {"value": round(geo.batch / (sec * geo.layers), 3), "unit": "tok/s",
                                  "cores": os.cpu_count(), "kind": "port",
                                  "sample": f"layer 0 of the same workload, all {geo.groups} groups, median of 2 "
                                            f"runs ({sec * 1e3:.1f} ms), scaled by {geo.layers} layers"}
    print(json.dumps(result), flush=True)


def reference_arm(geo, args, log):
    """The reference's own arithmetic for this path on the host cores (oracle port): each
    step is one layer of the workload, scaled to a full decode step."""
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    from dataclasses import replace
    small = replace(geo, layers=1)
    warm = max(args.warmup, 1)
    wl = Workload(small, dev, warm + args.steps, args.kmeans_iters, 0, log) if dev.type == "cuda" else None
    if wl is None:
        print(json.dumps({"impl": "reference", "unavailable": "set-up of the index needs the GPU box"}))
        return
    secs = [cpu_layer_seconds(wl, 0, st, 1) for st in range(warm + args.steps)][warm:]
    sec = sum(secs) / len(secs)
    val = round(geo.batch / (sec * geo.layers), 3)
    print(json.dumps({
        "impl": "reference", "metric": "decode tok/s at 128K ctx (Llama-3-8B geometry); attn kernel HBM GB/s vs peak",
        "value": val, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(sec * geo.layers * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{geo.name}: wave-index decode attention hot path on host cores"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": f"each step = layer 0 of the workload (all {geo.groups} groups), scaled by "
                                   f"{geo.layers} layers"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


if __name__ == "__main__":
    main()
