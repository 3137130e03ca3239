"""The CPU oracle against fixtures recorded from the reference itself
(``tests/golden/make_golden.py`` says how each file was made)."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import make_golden as mg  # noqa: E402
from oracle import kmeans as okm  # noqa: E402
from oracle import wave_buffer as owb  # noqa: E402

GOLDEN = os.path.join(HERE, "golden")


@pytest.mark.parametrize("name", sorted(mg.KMEANS_CASES))
def test_kmeans_matches_reference_run(name):
    heads, tokens, cents, segs, iters, seed, planted = mg.KMEANS_CASES[name]
    gold = torch.load(os.path.join(GOLDEN, name + ".pt"))
    k, v, centred = mg.kmeans_inputs(heads, tokens, seed, planted)
    assert mg.sha(centred) == gold["input_sha"]["centred"], "synthetic generator drifted"
    assert mg.sha(v) == gold["input_sha"]["value"]
    cen, vsum, clusters, sizes, assign = okm.segment_k_means(
        centred, v, cents, num_iters=iters, num_segments=segs, return_assignments=True)
    # integer outputs bit-exact; float outputs to one float16 ulp (the fp32 member sums
    # are accumulated in a different order than the interpreter's sequential atomics)
    assert torch.equal(assign, gold["assignments"].to(torch.int32))
    assert torch.equal(sizes, gold["sizes"])
    torch.testing.assert_close(cen.float(), gold["centroids"].float(), rtol=2 ** -10, atol=1e-6)
    torch.testing.assert_close(vsum.float(), gold["value_sum"].float(), rtol=2 ** -10, atol=1e-6)
    assert (cen.view(torch.int16) != gold["centroids"].view(torch.int16)).float().mean() < 1e-3
    # inverted lists hold exactly the members of each cluster
    for h in range(heads):
        for c in range(cents):
            members = clusters[h, c, :int(sizes[h, c])].long()
            assert (assign[h, members] == c).all()


def test_kmeans_fixture_has_empty_clusters():
    gold = torch.load(os.path.join(GOLDEN, "kmeans_duplicates_empty.pt"))
    assert int((gold["sizes"] == 0).sum()) > 0


def _check_page_consistency(state, g, hit_keys, hit_ids, pages, admitted):
    """Reference page ids are arbitrary (unordered_set); check what is not."""
    pos = 0
    for key in hit_keys:
        n = pages[key]
        assert state[g][key] == hit_ids[pos:pos + n], "cluster must hit on the pages it was admitted to"
        pos += n


def test_wave_buffer_matches_reference_run():
    rec = torch.load(os.path.join(GOLDEN, "wave_buffer_lru.pt"))
    p = rec["params"]
    groups = p["batch"] * p["heads"]
    sizes = rec["sizes"].reshape(groups, -1)
    bufs = [owb.GroupBuffer(p["capacity"], p["page"], p["buffer_pages"], sizes[g]) for g in range(groups)]
    ref_pages = [dict() for _ in range(groups)]   # cluster -> page ids, as the reference assigned them
    for step in rec["steps"]:
        (hit_ids, hit_sizes, hit_cum, hit_n, miss_ids, miss_sizes, miss_cum, miss_n,
         upd_buf, upd_sizes, upd_cache, upd_n) = step["lists"]
        for g in range(groups):
            acc = bufs[g].access(step["searched"][g])
            nh, nm = int(hit_n[g]), int(miss_n[g])
            assert nh == len(acc["hit_sizes"]) and nm == len(acc["miss_sizes"])
            assert hit_sizes[g, :nh].tolist() == acc["hit_sizes"]
            assert hit_cum[g, :nh].tolist() == acc["hit_cumsum"]
            assert miss_ids[g, :nm].tolist() == acc["miss_ids"]
            assert miss_sizes[g, :nm].tolist() == acc["miss_sizes"]
            assert miss_cum[g, :nm].tolist() == acc["miss_cumsum"]
            _check_page_consistency(ref_pages, g, acc["hit_keys"], hit_ids[g, :nh].tolist(), bufs[g].pages, None)
            miss_keys = acc["miss_keys"]
            upd = bufs[g].update()
            nu = int(upd_n[g])
            assert nu == len(upd["sizes"])
            assert upd_sizes[g, :nu].tolist() == upd["sizes"]
            assert upd_buf[g, :nu].tolist() == upd["buffer_offsets"]
            ids = upd_cache[g, :nu].tolist()
            assert len(set(ids)) == nu and all(0 <= i < p["capacity"] for i in ids)
            pos = 0
            for key in miss_keys[:upd["admitted"]]:
                n = bufs[g].pages[key]
                ref_pages[g][key] = ids[pos:pos + n]
                pos += n
            # evicted clusters leave the reference map too
            for key in list(ref_pages[g]):
                if key not in bufs[g].in_cache:
                    del ref_pages[g][key]
            live = [pid for pages in ref_pages[g].values() for pid in pages]
            assert len(live) == len(set(live)), "live clusters share a page"


def test_organize_kv_matches_reference_run():
    rec = torch.load(os.path.join(GOLDEN, "wave_buffer_lru.pt"))
    p = rec["params"]
    for b, org in enumerate(rec["organize"]):
        sizes = rec["sizes"][b]
        n_b = int(sizes[0].sum())
        keys, vals = mg.coded_rows(p["heads"], n_b, 128, b)
        lk, lv, starts = okm.organize_kv(keys, vals, org["clusters"].to(torch.int32), sizes)
        assert torch.equal(lk.view(torch.int16)[..., 0], org["list_keys_col0"])
        assert torch.equal(lv.view(torch.int16)[..., 0], org["list_values_col0"])
        assert int(starts[0, -1]) == n_b
