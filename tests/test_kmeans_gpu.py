"""Parity of the CUDA clustering (tcgen05 assignment GEMM + bucket + update + layout, through the
C ABI) against (a) the fixtures recorded from the reference's own kmeans.py and (b) the CPU oracle.

Bar: assignments, counts and member lists bit-exact except for tokens whose two best inner
products tie within 1e-3 (relative) — the tensor core accumulates the 128 products in a different
order than the CPU; centroids and value sums within one ulp of the 16-bit dtype wherever the
member sets agree."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import make_golden as mg  # noqa: E402
from oracle import kmeans as okm  # noqa: E402
from retrievalattention_b200.synthetic import make_kv  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(HERE, "golden")


def tie_excused(data, centroids, a, b, band=1e-3):
    """True where assignment a and b differ only between clusters whose scores tie."""
    ip = torch.bmm(data.float(), centroids.float().transpose(1, 2))
    sa = torch.gather(ip, 2, a.long()[..., None])[..., 0]
    sb = torch.gather(ip, 2, b.long()[..., None])[..., 0]
    return (sa - sb).abs() <= band * torch.maximum(sa.abs(), sb.abs()).clamp_min(1.0)


@pytest.mark.parametrize("name", sorted(mg.KMEANS_CASES))
def test_segment_k_means_against_reference_fixture(name):
    from retrievalattention_b200.cache_hub import kmeans as gk

    heads, tokens, cents, segs, iters, seed, planted = mg.KMEANS_CASES[name]
    gold = torch.load(os.path.join(GOLDEN, name + ".pt"))
    k, v, centred = mg.kmeans_inputs(heads, tokens, seed, planted)
    assert mg.sha(centred) == gold["input_sha"]["centred"]
    cen, vsum, clusters, sizes = gk.segment_k_means(centred.cuda(), v.cuda(), cents, num_iters=iters, num_segments=segs)
    torch.cuda.synchronize()
    cen, vsum, clusters, sizes = cen.cpu(), vsum.cpu(), clusters.cpu(), sizes.cpu()
    assign = torch.full((heads, tokens), -1, dtype=torch.int32)
    for h in range(heads):
        for c in range(cents):
            m = int(sizes[h, c])
            members = clusters[h, c, :m]
            assert (members[1:] > members[:-1]).all(), "members must be in ascending token order"
            assign[h, members.long()] = c
    assert (assign >= 0).all() and int(sizes.sum()) == heads * tokens
    want = gold["assignments"].to(torch.int32)
    diff = assign != want
    assert diff.float().mean() <= 0.01, f"{int(diff.sum())} of {diff.numel()} assignments differ"
    if diff.any():
        assert tie_excused(centred, gold["centroids"], assign, want)[diff].float().mean() > 0.5
    same = (sizes == gold["sizes"])
    assert same.float().mean() >= 0.97
    torch.testing.assert_close(cen.float()[same], gold["centroids"].float()[same], rtol=2 ** -9, atol=2e-3)
    torch.testing.assert_close(vsum.float()[same], gold["value_sum"].float()[same], rtol=2 ** -9, atol=2e-2)


BF16_CASES = {
    # heads, tokens, centroids, segments, iters, seed
    "one_tile": (2, 100, 32, 1, 3, 1),
    "ragged_tiles": (3, 1000, 96, 3, 4, 2),
    "many_tiles": (2, 5000, 512, 4, 5, 3),
    "wide": (1, 3000, 1024, 2, 3, 4),
}


@pytest.mark.parametrize("name", sorted(BF16_CASES))
def test_build_index_against_oracle_bf16(name):
    from retrievalattention_b200.cache_hub import kmeans as gk

    heads, tokens, cents, segs, iters, seed = BF16_CASES[name]
    k, v = make_kv(heads, tokens, 128, seed=seed)
    k = k[0].transpose(0, 1).contiguous()
    v = v[0].transpose(0, 1).contiguous()
    r = gk.build_index(k.cuda(), v.cuda(), cents, segs, iters, want_lists=True)
    torch.cuda.synchronize()
    r = {n: t.cpu() for n, t in r.items() if not n.startswith("_")}
    assert int(r["error"]) == 0

    # mean key: fp32 sum in another order, so allow one bf16 step; then centre exactly as the kernel did
    ref_mean = torch.mean(k, dim=1, keepdim=True)
    torch.testing.assert_close(r["mean_key"].float(), ref_mean.float(), rtol=2 ** -7, atol=1e-3)
    centred = k - r["mean_key"]
    cen, vsum, clusters, sizes, assign = okm.segment_k_means(centred, v, cents, iters, segs, return_assignments=True)

    diff = r["assign"] != assign
    assert diff.float().mean() <= 0.01, f"{int(diff.sum())} of {diff.numel()} assignments differ"
    if diff.any():
        assert tie_excused(centred, cen, r["assign"], assign)[diff].float().mean() > 0.5

    # structure: counts/offsets/order describe r["assign"] exactly, members ascending
    for h in range(heads):
        cnt = torch.bincount(r["assign"][h].long(), minlength=cents)
        assert torch.equal(cnt.to(torch.int32), r["cluster_count"][h])
        off = r["cluster_offset"][h].long()
        assert off[0] == 0 and off[-1] == tokens and torch.equal(off[1:] - off[:-1], cnt)
        order = r["order"][h].long()
        assert torch.equal(torch.sort(order).values, torch.arange(tokens))
        assert torch.equal(r["assign"][h].long()[order], torch.repeat_interleave(torch.arange(cents), cnt))
        same_cluster = r["assign"][h].long()[order][1:] == r["assign"][h].long()[order][:-1]
        assert (order[1:][same_cluster] > order[:-1][same_cluster]).all()
        # layout: rows copied bit-for-bit in member order
        assert torch.equal(r["keys"][h].view(torch.int16), k[h][order].view(torch.int16))
        assert torch.equal(r["values"][h].view(torch.int16), v[h][order].view(torch.int16))
    assert torch.equal(r["cluster_size"].view(torch.int16), r["cluster_count"].to(torch.bfloat16).view(torch.int16))

    same = sizes == r["cluster_count"]
    assert same.float().mean() >= 0.97
    want_cent = cen + r["mean_key"]
    torch.testing.assert_close(r["centroids"].float()[same], want_cent.float()[same], rtol=2 ** -6, atol=2e-2)
    torch.testing.assert_close(r["value_sum"].float()[same], vsum.float()[same], rtol=2 ** -6, atol=6e-2)
    if not diff.any():
        # identical member sets and a serial sum in the same order: value sums agree to the bit
        assert torch.equal(r["value_sum"].view(torch.int16), vsum.view(torch.int16))


def test_empty_clusters_keep_centroid_and_zero_value_sum():
    from retrievalattention_b200.cache_hub import kmeans as gk

    heads, tokens, cents = 2, 700, 64
    k, v = make_kv(heads, tokens, 128, seed=9)
    k = k[0].transpose(0, 1)[:, torch.arange(tokens) % 37].contiguous()
    v = v[0].transpose(0, 1).contiguous()
    r = gk.build_index(k.cuda(), v.cuda(), cents, 1, 5, want_lists=True)
    torch.cuda.synchronize()
    cnt = r["cluster_count"].cpu()
    assert int((cnt == 0).sum()) > 0
    assert (r["value_sum"].cpu()[cnt == 0] == 0).all()
    assert torch.isfinite(r["centroids"].float()).all()


def test_rejects_bad_shapes():
    import ctypes as C
    from retrievalattention_b200 import _lib

    p = _lib.KMeans()
    p.groups, p.n_tokens, p.n_centroids, p.n_segments, p.n_iters = 1, 100, 48, 1, 3
    assert _lib.lib.ri_kmeans_scratch_bytes(C.byref(p)) == -1
    assert b"multiple of 32" in _lib.lib.ri_last_error()
