"""The three gather/copy operators (through the C ABI) against the slicing-loop oracle, bit-exact.
Shapes and edge cases follow the reference's own kernel tests
(library/retroinfer/test/test_gather_copy.py): a group with no page from the host list, a group with
no page from the GPU cache, a page that ends exactly at the end of the source, partially filled
pages (0..8 rows), a pinned-host second source and pinned index arrays."""
import numpy as np
import pytest
import torch

from oracle import gather as og

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


def page_lists(rng, rows, cols, n_used, max_index, unit, boundary=None):
    idx = rng.integers(-1, 100, size=(rows, cols)).astype(np.int32)        # junk beyond the used part
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
            idx[g, x] = boundary - size[g, x]       # this page ends exactly at the end of the source
    pin = lambda a: torch.from_numpy(a).pin_memory()  # noqa: E731
    return pin(idx), pin(size), pin(dst), pin(np.asarray(n_used, dtype=np.int32))


def test_gather_copy_and_concat():
    from retrievalattention_b200.kernels import gather_copy_and_concat

    rng = np.random.default_rng(1)
    torch.manual_seed(1)
    groups, n1, n2, units3, buf_units, ilen, unit, copy1 = 8, 1769, 12397, 1000, 400, 400, 8, 1602
    buf_rows = buf_units * unit + n1
    k1, v1 = (torch.randn((groups, n1, 128), device="cuda").to(DT) for _ in range(2))
    k2, v2 = (torch.randn((groups, n2, 128)).to(DT).pin_memory() for _ in range(2))
    k3, v3 = (torch.randn((groups, units3, unit, 128), device="cuda").to(DT) for _ in range(2))
    kd = torch.randn((groups, buf_rows, 128), device="cuda").to(DT)
    vd = torch.randn((groups, buf_rows, 128), device="cuda").to(DT)
    kd_ref, vd_ref = kd.cpu().clone(), vd.cpu().clone()
    used = rng.integers(int(0.4 * ilen), int(0.5 * ilen), size=groups)
    n_a = [int(rng.integers(0, u)) for u in used]
    n_a[1], n_a[5] = 0, int(used[5])                         # no host pages / no cache pages
    n_b = [int(u - a) for u, a in zip(used, n_a)]
    i2, s2, d2, c2 = page_lists(rng, groups, ilen, n_a, n2 - unit, unit, boundary=n2)
    i3, s3, d3, c3 = page_lists(rng, groups, ilen, n_b, units3, unit)
    valid = torch.empty((groups,), dtype=torch.int32).pin_memory()
    gather_copy_and_concat(k1, k2, k3, kd, v1, v2, v3, vd, i2, s2, d2, c2, i3, s3, d3, c3, valid, groups, n1, n2,
                           units3, buf_rows, ilen, copy1)
    torch.cuda.synchronize()
    valid_ref = torch.zeros((groups,), dtype=torch.int32)
    og.gather_copy_and_concat(k1.cpu(), k2, k3.cpu(), kd_ref, v1.cpu(), v2, v3.cpu(), vd_ref, i2, s2, d2, c2, i3, s3,
                              d3, c3, valid_ref, copy1)
    assert torch.equal(valid, valid_ref)
    assert torch.equal(kd.cpu().view(torch.int16), kd_ref.view(torch.int16))
    assert torch.equal(vd.cpu().view(torch.int16), vd_ref.view(torch.int16))


def test_gather_copy_and_scatter():
    from retrievalattention_b200.kernels import gather_copy_and_scatter

    rng = np.random.default_rng(2)
    torch.manual_seed(2)
    groups, src_units, dst_units, ilen, unit, start = 8, 400, 1000, 400, 8, 97
    src_rows = src_units * unit
    ks, vs = (torch.randn((groups, src_rows, 128), device="cuda").to(DT) for _ in range(2))
    kd, vd = (torch.randn((groups, dst_units, unit, 128), device="cuda").to(DT) for _ in range(2))
    kd_ref, vd_ref = kd.cpu().clone(), vd.cpu().clone()
    limit = src_rows - start
    si = rng.integers(-1, 100, size=(groups, ilen)).astype(np.int32)
    sz = rng.integers(1, unit + 1, size=(groups, ilen)).astype(np.int32)
    di = rng.integers(0, 100, size=(groups, ilen)).astype(np.int32)
    n = np.zeros(groups, dtype=np.int32)
    for g in range(groups):
        if g == 1:
            continue                                          # a group with nothing to admit
        m = int(rng.integers(int(0.2 * ilen), int(0.8 * ilen)))
        si[g, :m] = rng.choice(limit, m, replace=False)
        di[g, :m] = rng.choice(dst_units, m, replace=False)
        for j in range(m):
            sz[g, j] = min(int(rng.integers(0, unit + 1)), limit - si[g, j])
        n[g] = m
    pin = lambda a: torch.from_numpy(a).pin_memory()  # noqa: E731
    si, sz, di, n = pin(si), pin(sz), pin(di), pin(n)
    gather_copy_and_scatter(ks, kd, vs, vd, si, sz, di, n, groups, src_rows, dst_units, ilen, start)
    torch.cuda.synchronize()
    og.gather_copy_and_scatter(ks.cpu(), kd_ref, vs.cpu(), vd_ref, si, sz, di, n, start)
    assert torch.equal(kd.cpu().view(torch.int16), kd_ref.view(torch.int16))
    assert torch.equal(vd.cpu().view(torch.int16), vd_ref.view(torch.int16))


def test_gather_copy_vectors():
    from retrievalattention_b200.kernels import gather_copy_vectors

    torch.manual_seed(3)
    groups, rows, nprobe, isize = 8, 8192, 150, 2048
    n = isize - nprobe
    ks, vs = (torch.randn((groups, rows, 128), device="cuda").to(DT) for _ in range(2))
    kd, vd = (torch.randn((groups, n, 128), device="cuda").to(DT) for _ in range(2))
    ms = torch.randn((groups, rows), device="cuda").to(DT)
    md = torch.empty((groups, n), device="cuda", dtype=DT)
    kd_ref, vd_ref, md_ref = kd.cpu().clone(), vd.cpu().clone(), md.cpu().clone()
    idx = torch.stack([torch.randperm(rows)[:isize] for _ in range(groups)]).to(torch.int64).cuda()
    gather_copy_vectors(ks, kd, vs, vd, ms, md, idx, groups, rows, n, isize, nprobe, n)
    torch.cuda.synchronize()
    og.gather_copy_vectors(ks.cpu(), kd_ref, vs.cpu(), vd_ref, ms.cpu(), md_ref, idx.cpu(), nprobe, n)
    assert torch.equal(kd.cpu().view(torch.int16), kd_ref.view(torch.int16))
    assert torch.equal(vd.cpu().view(torch.int16), vd_ref.view(torch.int16))
    assert torch.equal(md.cpu().view(torch.int16), md_ref.view(torch.int16))


def test_bad_ranges_are_rejected():
    from retrievalattention_b200 import _lib

    rc = _lib.lib.ri_gather_copy_vectors(16, 16, 16, 16, 16, 16, 16, 1, 8, 8, 4, 2, 4, None)
    assert rc == -1 and b"outside the index" in _lib.lib.ri_last_error()
