"""This library's operators and decode path against the REFERENCE'S OWN CUDA kernels, compiled for sm_100a from
where they lie in the reference checkout (``oracle/build_ref.py`` -> ``oracle/_ref``: modules ``gemm_softmax`` and
``Copy``, exactly what ``retroinfer_kernels`` builds).  Skipped where those modules were never built.

* ``batch_gemm_softmax`` (CUTLASS GEMM with the softmax epilogue visitor): scores ``D`` and probabilities
  ``Softmax`` of ``ri_batch_gemm_softmax`` against the reference kernel's; then what the reference ranks by,
  ``bf16(sum over the GQA group of Softmax)`` (cache_hub/retroinfer_cache.py:569-573), against the 16-bit distance
  keys the single decode kernel and the stage kernels compute — this pins the rounding chain of the scores —
  and the reference's ``topk`` sets against the kernel's sets with the 1e-3 tie rule;
* the three copy operators: bit-exact against the reference kernels on the reference test's shapes and edge cases.
"""
import math

import numpy as np
import pytest
import torch

from helpers import Case, build_cpu_index, queries, to_gpu_layer, SINK, RECENT
from oracle import build_ref
from oracle import score_select as oss

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


def ref_module(name):
    mod = build_ref.load(name)
    if mod is None:
        pytest.skip(f"oracle/_ref/{name} was not built (needs the reference checkout at build time)")
    return mod


def ordered_key(dist):
    bits = dist.view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where(bits >= 0x8000, (~bits) & 0xFFFF, bits | 0x8000)


def ref_gemm_softmax(mod, A, B):
    batch, m, _ = A.shape
    n = B.shape[1]
    D = torch.zeros((batch, m, n), device="cuda", dtype=A.dtype)
    S = torch.zeros_like(D)
    blocks = (n + 255) // 256
    norm = torch.zeros((batch, m, blocks), device="cuda", dtype=torch.float32)
    ssum = torch.zeros_like(norm)
    mod.batch_gemm_softmax(A, B, D, norm, ssum, S, batch, m, n, 128, 1 / math.sqrt(128), 0)
    torch.cuda.synchronize()
    return D, S


@pytest.mark.parametrize("batch,m,n,dtype", [
    (16, 4, 8200, torch.bfloat16),     # the reference test's shape (scaled-down batch)
    (32, 4, 8192, torch.bfloat16),     # configuration 1
    (4, 8, 1024, torch.float16),
])
def test_operator_against_the_reference_cutlass_kernel(batch, m, n, dtype):
    from retrievalattention_b200 import kernels

    mod = ref_module("gemm_softmax")
    g = torch.Generator(device="cuda").manual_seed(n + m)
    A = torch.randn((batch, m, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    B = torch.randn((batch, n, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    ref_d, ref_s = ref_gemm_softmax(mod, A, B)
    D, S = torch.zeros_like(ref_d), torch.zeros_like(ref_s)
    blocks = (n + 255) // 256
    norm = torch.zeros((batch, m, blocks), device="cuda", dtype=torch.float32)
    kernels.batch_gemm_softmax(A, B, D, norm, norm.clone(), S, batch, m, n, 128, 1 / math.sqrt(128), 0)
    torch.cuda.synchronize()
    # both round one fp32 product per score; the accumulation orders differ, so a score may land on the
    # neighbouring 16-bit value — never further
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert (D.view(torch.int16) != ref_d.view(torch.int16)).float().mean() < 0.02
    assert ((D.float() - ref_d.float()).abs() <= ulp * ref_d.float().abs().clamp_min(2.0 ** -6)).all()
    assert torch.allclose(S.float(), ref_s.float(), atol=1e-3)          # the reference test's own tolerance
    assert (S.view(torch.int16) != ref_s.view(torch.int16)).float().mean() < 0.05


@pytest.mark.parametrize("form", ["single_kernel", "staged"])
def test_distance_keys_and_sets_against_the_reference_kernel(form):
    """Configuration 0's geometry: what the reference ranks by, computed by its own kernel, against the decode path."""
    mod = ref_module("gemm_softmax")
    case = Case(1, 8, 4, 8192, 512, 1, 9, 118, seed=0, iters=3)
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    q = queries(case).cuda()
    if form == "staged":
        layer.compute_staged(q)
    else:
        layer.compute(q)
    torch.cuda.synchronize()
    A = q.reshape(case.groups, case.group_size, 128).contiguous()
    _, S = ref_gemm_softmax(mod, A, layer.t["centroids"])
    dist = torch.sum(S, dim=1)                                          # cache_hub/retroinfer_cache.py:572
    dist = dist.masked_fill(cpu["mask"].cuda(), torch.finfo(DT).min)    # :573
    keys = layer.views()["dist_keys"].to(torch.int32) & 0xFFFF
    ref_keys = ordered_key(dist)
    assert (keys != ref_keys).float().mean() < 0.02                      # a flipped rounding of one probability
    assert ((keys - ref_keys).abs() <= 1).all()
    k = case.nprobe + case.n_estimate
    ret, est = layer.retrieved_ids.cpu(), layer.estimated_ids.cpu()
    assert oss.selection_matches(dist.cpu(), ret, case.nprobe)
    assert oss.selection_matches(dist.cpu(), torch.cat((ret, est), 1), k)
    # the reference's own selection (:574-575): its sets are admissible under the same rule, and outside the tie
    # band the two selections are the same sets
    top = torch.topk(dist.float(), k, dim=-1).indices.cpu()
    assert oss.selection_matches(dist.cpu(), top[:, :case.nprobe], case.nprobe)
    for g in range(case.groups):
        d = dist[g].float().cpu()
        cut = torch.topk(d, case.nprobe).values[-1]
        clear = set(torch.nonzero(d > cut + 1e-3).flatten().tolist())
        assert clear <= set(ret[g].tolist()) and clear <= set(top[g, :case.nprobe].tolist())


def page_lists(rng, rows, cols, n_used, max_index, unit, boundary=None):
    idx = rng.integers(0, 100, size=(rows, cols)).astype(np.int32)
    size = rng.integers(1, unit + 1, size=(rows, cols)).astype(np.int32)
    dst = rng.integers(0, 100, size=(rows, cols)).astype(np.int32)
    for g in range(rows):
        n = n_used[g]
        idx[g, :n] = rng.choice(max_index, n, replace=False)
        cum = 0
        for j in range(n):
            size[g, j] = rng.integers(0, unit + 1)
            dst[g, j] = cum
            cum += size[g, j]
        if boundary is not None and n > 0:
            x = rng.integers(0, n)
            idx[g, x] = boundary - size[g, x]
    pin = lambda a: torch.from_numpy(a).pin_memory()  # noqa: E731
    return pin(idx), pin(size), pin(dst), pin(np.asarray(n_used, dtype=np.int32))


def test_copy_operators_against_the_reference_kernels():
    from retrievalattention_b200 import kernels

    mod = ref_module("Copy")
    rng = np.random.default_rng(4)
    torch.manual_seed(4)
    # ---- gather_copy_vectors ----
    groups, rows, nprobe, isize = 8, 8192, 150, 2048
    n = isize - nprobe
    ks, vs = (torch.randn((groups, rows, 128), device="cuda").to(DT) for _ in range(2))
    ms = torch.randn((groups, rows), device="cuda").to(DT)
    idx = torch.stack([torch.randperm(rows)[:isize] for _ in range(groups)]).to(torch.int64).cuda()
    outs = []
    for fn in (mod.gather_copy_vectors, kernels.gather_copy_vectors):
        kd, vd = (torch.zeros((groups, n, 128), device="cuda", dtype=DT) for _ in range(2))
        md = torch.zeros((groups, n), device="cuda", dtype=DT)
        fn(ks, kd, vs, vd, ms, md, idx, groups, rows, n, isize, nprobe, n)
        torch.cuda.synchronize()
        outs.append((kd, vd, md))
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # ---- gather_copy_and_concat ----
    groups, n1, n2, units3, buf_units, ilen, unit, copy1 = 8, 1769, 12397, 1000, 400, 400, 8, 1602
    buf_rows = buf_units * unit + n1
    k1, v1 = (torch.randn((groups, n1, 128), device="cuda").to(DT) for _ in range(2))
    k2, v2 = (torch.randn((groups, n2, 128)).to(DT).pin_memory() for _ in range(2))
    k3, v3 = (torch.randn((groups, units3, unit, 128), device="cuda").to(DT) for _ in range(2))
    used = rng.integers(int(0.4 * ilen), int(0.5 * ilen), size=groups)
    n_a = [int(rng.integers(0, u)) for u in used]
    n_a[1], n_a[5] = 0, int(used[5])
    n_b = [int(u - a) for u, a in zip(used, n_a)]
    i2, s2, d2, c2 = page_lists(rng, groups, ilen, n_a, n2 - unit, unit, boundary=n2)
    i3, s3, d3, c3 = page_lists(rng, groups, ilen, n_b, units3, unit)
    base_k = torch.randn((groups, buf_rows, 128), device="cuda").to(DT)
    outs = []
    for fn in (mod.gather_copy_and_concat, kernels.gather_copy_and_concat):
        kd, vd = base_k.clone(), base_k.clone()
        valid = torch.zeros((groups,), dtype=torch.int32).pin_memory()
        fn(k1, k2, k3, kd, v1, v2, v3, vd, i2, s2, d2, c2, i3, s3, d3, c3, valid, groups, n1, n2, units3, buf_rows,
           ilen, copy1)
        torch.cuda.synchronize()
        outs.append((kd, vd, valid.clone()))
    assert torch.equal(outs[0][2], outs[1][2])
    for g in range(groups):            # rows beyond the valid length are nobody's business
        m = int(outs[0][2][g])
        assert torch.equal(outs[0][0][g, :m].view(torch.int16), outs[1][0][g, :m].view(torch.int16))
        assert torch.equal(outs[0][1][g, :m].view(torch.int16), outs[1][1][g, :m].view(torch.int16))
    # ---- gather_copy_and_scatter ----
    groups, src_units, dst_units, ilen, unit, start = 8, 400, 1000, 400, 8, 97
    src_rows = src_units * unit
    ks, vs = (torch.randn((groups, src_rows, 128), device="cuda").to(DT) for _ in range(2))
    base = torch.randn((groups, dst_units, unit, 128), device="cuda").to(DT)
    limit = src_rows - start
    si = rng.integers(0, 100, size=(groups, ilen)).astype(np.int32)
    sz = rng.integers(1, unit + 1, size=(groups, ilen)).astype(np.int32)
    di = rng.integers(0, 100, size=(groups, ilen)).astype(np.int32)
    cnt = np.zeros(groups, dtype=np.int32)
    for g in range(groups):
        if g == 1:
            continue
        m = int(rng.integers(int(0.2 * ilen), int(0.8 * ilen)))
        si[g, :m] = rng.choice(limit, m, replace=False)
        di[g, :m] = rng.choice(dst_units, m, replace=False)
        for j in range(m):
            sz[g, j] = min(int(rng.integers(0, unit + 1)), limit - si[g, j])
        cnt[g] = m
    pin = lambda a: torch.from_numpy(a).pin_memory()  # noqa: E731
    si, sz, di, cnt = pin(si), pin(sz), pin(di), pin(cnt)
    outs = []
    for fn in (mod.gather_copy_and_scatter, kernels.gather_copy_and_scatter):
        kd, vd = base.clone(), base.clone()
        fn(ks, kd, vs, vd, si, sz, di, cnt, groups, src_rows, dst_units, ilen, start)
        torch.cuda.synchronize()
        outs.append((kd, vd))
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
