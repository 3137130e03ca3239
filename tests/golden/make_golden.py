"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <reference checkout> [all|kmeans|kmeans-missing|wave]
    (the checkout may also be named by RI_REFERENCE_ROOT in the environment)

* ``kmeans_*.pt`` — outputs of the reference's own ``cache_hub/kmeans.py``
  (``segment_k_means``) executed unmodified on CPU tensors under the Triton
  interpreter (``TRITON_INTERPRET=1``; atomics run sequentially, so the result is
  deterministic).  The fixtures are float16 — a dtype every reference kernel on the
  path dispatches on — because Triton 3.6's interpreter keeps bfloat16 tensors as raw
  uint16 and multiplies the bit patterns in ``tl.dot`` (interpreter.py ``create_dot``),
  so a bfloat16 run under the interpreter is not the reference's arithmetic.
  Inputs are regenerated from a seed by
  ``retrievalattention_b200.synthetic.make_kv``; their SHA-256 is stored so that a
  drifting generator is detected instead of silently comparing different data.
* ``wave_buffer_*.pt`` — hit/miss/update lists recorded from the reference's own
  ``WaveBufferCPU`` (``oracle/_ref``, built by ``oracle/build_ref.py``) over a
  sequence of decode steps.

The tests never import the reference; they only read these files.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from retrievalattention_b200.synthetic import make_kv  # noqa: E402

KMEANS_CASES = {
    # name: (kv_heads, tokens, centroids, segments, iterations, seed, planted)
    "kmeans_seg2_tail": (2, 1501, 64, 2, 4, 11, 0),
    "kmeans_seg1_full": (1, 1030, 32, 1, 10, 12, 0),
    "kmeans_seg4_planted": (2, 2048, 128, 4, 6, 13, 24),
    # planted < 0: only -planted distinct key rows, repeated -> duplicate initial
    # centroids, so many clusters stay empty (edge case: masked centroid store).
    "kmeans_duplicates_empty": (2, 700, 64, 1, 5, 14, -37),
    # one and two iterations: both sides start from the same centroids, so every assignment that differs
    # from the reference's has to be a tie (strict parity, no drift to allow for)
    "kmeans_iter1": (2, 1200, 64, 2, 1, 15, 0),
    "kmeans_iter2": (2, 1200, 64, 2, 2, 16, 0),
}


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def kmeans_inputs(heads, tokens, seed, planted, dtype=torch.float16):
    k, v = make_kv(heads, tokens, 128, seed=seed, planted_centres=max(planted, 0), dtype=dtype)
    k = k[0].transpose(0, 1).contiguous()     # [heads, tokens, d]
    v = v[0].transpose(0, 1).contiguous()
    if planted < 0:
        k = k[:, torch.arange(tokens) % (-planted)].contiguous()
    mean = torch.mean(k, dim=1, keepdim=True)
    return k, v, k - mean


def make_kmeans(reference_root: str, only_missing: bool = False):
    spec = importlib.util.spec_from_file_location(
        "ref_kmeans", os.path.join(reference_root, "cache_hub", "kmeans.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name, (heads, tokens, cents, segs, iters, seed, planted) in KMEANS_CASES.items():
        if only_missing and os.path.exists(os.path.join(HERE, name + ".pt")):
            continue
        k, v, centred = kmeans_inputs(heads, tokens, seed, planted)
        cen, vsum, clusters, sizes = ref.segment_k_means(centred, v, cents, num_iters=iters, num_segments=segs)
        assign = torch.full((heads, tokens), -1, dtype=torch.int32)
        for h in range(heads):
            for c in range(cents):
                m = int(sizes[h, c])
                assign[h, clusters[h, c, :m].long()] = c
        assert (assign >= 0).all()
        torch.save({
            "params": dict(heads=heads, tokens=tokens, centroids=cents, segments=segs, iters=iters,
                           seed=seed, planted=planted),
            "input_sha": {"centred": sha(centred), "value": sha(v)},
            "centroids": cen, "value_sum": vsum, "sizes": sizes.to(torch.int32),
            "assignments": assign.to(torch.int16),
        }, os.path.join(HERE, name + ".pt"))
        print(name, "sizes max", int(sizes.max()), "empty", int((sizes == 0).sum()))


def coded_rows(heads, n, dim, salt):
    """Rows whose bit patterns encode (head, token, column); the re-layout is a byte
    copy, so any pattern serves and nothing but column 0 needs storing."""
    h = torch.arange(heads, dtype=torch.int32)[:, None, None]
    t = torch.arange(n, dtype=torch.int32)[None, :, None]
    j = torch.arange(dim, dtype=torch.int32)[None, None, :]
    k = ((t * 7 + h * 3001 + salt * 11) % 16000 + j).to(torch.int16)
    v = ((t * 5 + h * 2003 + salt * 13) % 16000 + j).to(torch.int16)
    return k.view(torch.bfloat16).contiguous(), v.view(torch.bfloat16).contiguous()


def make_wave_buffer():
    from oracle import build_ref
    build_ref.build()
    wb = build_ref.load()
    torch.manual_seed(5)
    batch, heads, dim, nprobe, page, cents = 2, 2, 128, 6, 8, 40
    buffer_pages, capacity, threads = 20, 14, 2
    groups = batch * heads
    pool = wb.ThreadPool(threads)
    w = wb.WaveBufferCPU(batch, heads, dim, nprobe, page, cents, cents, buffer_pages, capacity, threads, pool.get())
    i32 = lambda *s: torch.zeros(s, dtype=torch.int32)
    lists = [i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups),
             i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups),
             i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups, buffer_pages), i32(groups)]
    searched = torch.zeros((groups, nprobe), dtype=torch.int64)
    w.set_indices(*lists, searched)
    # cluster sizes 1..30 (no empty cluster), per request (the reference wants equal totals per head)
    sizes = torch.randint(1, 31, (batch, heads, cents), dtype=torch.int32)
    for b in range(batch):
        sizes[b, 1] = sizes[b, 0][torch.randperm(cents)]
    n_tok = int(sizes[0, 0].sum().item())
    max_sz = int(sizes.max())
    list_k = torch.zeros((batch, heads, int(sizes.sum(-1).max()), dim), dtype=torch.bfloat16)
    list_v = torch.zeros_like(list_k)
    recs = {"params": dict(batch=batch, heads=heads, nprobe=nprobe, page=page, centroids=cents,
                           buffer_pages=buffer_pages, capacity=capacity),
            "sizes": sizes.clone(), "steps": [], "organize": []}
    for b in range(batch):
        n_b = int(sizes[b, 0].sum())
        keys, vals = coded_rows(heads, n_b, dim, b)
        clusters = torch.zeros((heads, cents, max_sz), dtype=torch.int32)
        for h in range(heads):
            perm = torch.randperm(n_b, dtype=torch.int32)
            s = 0
            for c in range(cents):
                m = int(sizes[b, h, c])
                clusters[h, c, :m] = perm[s:s + m]
                s += m
        w.set_kv(list_k, list_v, keys, vals)
        w.async_construction(clusters, sizes[b].contiguous(), b)
        w.construction_sync()
        # rows are bit-coded (see coded_rows), so the first column identifies the source row
        assert (list_k[b, :, :n_b].view(torch.int16)[..., 5] == list_k[b, :, :n_b].view(torch.int16)[..., 0] + 5).all()
        recs["organize"].append({"clusters": clusters.to(torch.int16),
                                 "list_keys_col0": list_k[b, :, :n_b].view(torch.int16)[..., 0].clone(),
                                 "list_values_col0": list_v[b, :, :n_b].view(torch.int16)[..., 0].clone()})
    for step in range(12):
        for g in range(groups):
            searched[g] = torch.randperm(cents)[:nprobe] if step % 3 else torch.arange(nprobe) + (step * 2) % 20
        w.batch_access()
        w.sync()
        recs["steps"].append({"searched": searched.clone(), "lists": [t.clone() for t in lists]})
    torch.save(recs, os.path.join(HERE, "wave_buffer_lru.pt"))
    print("wave buffer fixture:", len(recs["steps"]), "steps; tokens/head", n_tok)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RI_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py <reference checkout> [all|kmeans|kmeans-missing|wave]   (or set RI_REFERENCE_ROOT)")
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    if which in ("all", "kmeans", "kmeans-missing"):
        make_kmeans(root, only_missing=which == "kmeans-missing")
    if which in ("all", "wave"):
        make_wave_buffer()
