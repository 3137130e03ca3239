"""The C++ wave buffer (through the C ABI) against the step-by-step record of the reference's own
WaveBufferCPU (tests/golden/wave_buffer_lru.pt).  Page ids are arbitrary in the reference, so they
are checked for consistency; every other list must match exactly."""
import os

import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make(p, sizes):
    from retrievalattention_b200.kernels import ThreadPool, WaveBufferCPU

    groups = p["batch"] * p["heads"]
    pool = ThreadPool(2)
    wb = WaveBufferCPU(p["batch"], p["heads"], 128, p["nprobe"], p["page"], p["centroids"], p["centroids"],
                       p["buffer_pages"], p["capacity"], 2, pool.get())
    i32 = lambda *s: torch.zeros(s, dtype=torch.int32)  # noqa: E731
    bp = p["buffer_pages"]
    lists = [i32(groups, bp), i32(groups, bp), i32(groups, bp), i32(groups), i32(groups, bp), i32(groups, bp),
             i32(groups, bp), i32(groups), i32(groups, bp), i32(groups, bp), i32(groups, bp), i32(groups)]
    searched = torch.zeros((groups, p["nprobe"]), dtype=torch.int64)
    wb.set_indices(*lists, searched)
    for b in range(p["batch"]):
        wb.async_construction(None, sizes[b], b)
        wb.construction_sync()
    return wb, lists, searched


def test_matches_reference_record():
    rec = torch.load(os.path.join(GOLDEN, "wave_buffer_lru.pt"))
    p = rec["params"]
    groups = p["batch"] * p["heads"]
    wb, lists, searched = make(p, rec["sizes"])
    pages = [[(int(s) + p["page"] - 1) // p["page"] for s in row] for row in rec["sizes"].reshape(groups, -1)]
    ours = [dict() for _ in range(groups)]      # cluster -> page ids as this library assigned them
    saw_overflow = False
    for step in rec["steps"]:
        searched.copy_(step["searched"])
        saw_overflow |= wb.batch_access() > 0
        wb.sync()
        r = step["lists"]
        (hit_ids, hit_sizes, hit_cum, hit_n, miss_ids, miss_sizes, miss_cum, miss_n, upd_buf, upd_sizes, upd_cache,
         upd_n) = lists
        assert torch.equal(hit_n, r[3]) and torch.equal(miss_n, r[7]) and torch.equal(upd_n, r[11])
        for g in range(groups):
            nh, nm, nu = int(hit_n[g]), int(miss_n[g]), int(upd_n[g])
            assert torch.equal(hit_sizes[g, :nh], r[1][g, :nh]) and torch.equal(hit_cum[g, :nh], r[2][g, :nh])
            assert torch.equal(miss_ids[g, :nm], r[4][g, :nm]) and torch.equal(miss_sizes[g, :nm], r[5][g, :nm])
            assert torch.equal(miss_cum[g, :nm], r[6][g, :nm])
            assert torch.equal(upd_sizes[g, :nu], r[9][g, :nu]) and torch.equal(upd_buf[g, :nu], r[8][g, :nu])
            # page ids: a hit returns the pages the cluster was admitted to; live clusters never share one
            starts = {}
            row = 0
            for c, s in enumerate(rec["sizes"].reshape(groups, -1)[g].tolist()):
                starts[row] = c
                row += s
            pos = 0
            hit_list = hit_ids[g, :nh].tolist()
            hit_clusters = []
            while pos < nh:
                owner = [c for c, ids in ours[g].items() if ids and ids[0] == hit_list[pos]]
                assert len(owner) == 1, "hit page does not belong to exactly one cached cluster"
                n = pages[g][owner[0]]
                assert ours[g][owner[0]] == hit_list[pos:pos + n]
                hit_clusters.append(owner[0])
                pos += n
            ids = upd_cache[g, :nu].tolist()
            assert len(set(ids)) == nu and all(0 <= i < p["capacity"] for i in ids)
            # admitted clusters are a prefix of the missed ones, in order
            miss_clusters, pos = [], 0
            while pos < nm:
                c = starts[int(miss_ids[g, pos])]
                miss_clusters.append(c)
                pos += pages[g][c]
            pos = 0
            admitted = []
            for c in miss_clusters:
                if pos >= nu:
                    break
                ours[g][c] = ids[pos:pos + pages[g][c]]
                admitted.append(c)
                pos += pages[g][c]
            assert pos == nu
            # evict whatever now shares a page with a newly admitted cluster
            fresh = {i for c in admitted for i in ours[g][c]}
            for c in list(ours[g]):
                if c not in admitted and fresh & set(ours[g][c]):
                    del ours[g][c]
            live = [i for v in ours[g].values() for i in v]
            assert len(live) == len(set(live)) and len(live) <= p["capacity"]
    assert saw_overflow, "the fixture is meant to exercise the page-budget cut"


def test_rejects_bad_arguments():
    from retrievalattention_b200 import _lib

    assert not _lib.lib.ri_wb_create(0, 1, 1, 8, 8, 8, 8, 8, 1)
    assert b"positive" in _lib.lib.ri_last_error()
    assert _lib.lib.ri_wb_batch_access(None) < 0
