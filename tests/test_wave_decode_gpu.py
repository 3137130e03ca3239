"""Parity of the fused decode path (scan -> select -> attend, through the C ABI) against the
CPU oracle on the same seeded inputs.

Bars: centroid scores within fp32 accumulation noise; distance keys and selected sets bit-exact
except where distances tie within 1e-3 of the cut; attention output max-abs <= 2e-2 and
mean-abs <= 2e-3 against the oracle's fp32 evaluation."""
import pytest
import torch

from helpers import Case, build_cpu_index, queries, to_gpu_layer, SINK, RECENT
from oracle import attention as oat
from oracle import score_select as oss

pytestmark = pytest.mark.gpu

CASES = {
    "small_gs4": Case(2, 2, 4, 2048 + 68, 128, 1, 6, 30),
    "qwen_gs7": Case(1, 2, 7, 1536 + 68, 96, 2, 5, 22, seed=3),
    "gs8_planted": Case(2, 1, 8, 2048 + 68, 128, 4, 6, 29, seed=4, planted=16),
    "gs1": Case(1, 3, 1, 1024 + 68, 64, 1, 4, 15, seed=5),
    "no_estimation": Case(1, 2, 4, 1024 + 68, 64, 1, 4, 0, seed=6),
    "tight_budget": Case(1, 2, 4, 2048 + 68, 64, 1, 8, 14, seed=7, buffer_pages=9),
    "empty_clusters": Case(1, 2, 4, 1024 + 68, 64, 1, 4, 15, seed=8, duplicate_rows=37),
    "cfg0_geometry": Case(1, 8, 4, 8192, 512, 1, 9, 118, seed=0, iters=3),
    # the cluster size follows the number of groups (the largest of 8 .. 4 CTAs with which all clusters are resident
    # at once; a B200 holds 15 clusters of 8 or 7 CTAs, 22 of 6, 26 of 5, 33 of 4): 20 and 21 groups run with 6
    "many_groups_gs8": Case(5, 4, 8, 1024 + 68, 64, 1, 4, 15, seed=9),
    "many_groups_gs3": Case(7, 3, 3, 1536 + 68, 96, 2, 5, 22, seed=10),
    # 16 groups (6 CTAs: slices of 8192 / 6 centroids that are not all alike — here some CTAs have no centroid at
    # all — and 640 or 384 output values shared out over 6 CTAs), 24 groups (5 CTAs), 30 groups (4 CTAs)
    "sixteen_groups_gs5": Case(2, 8, 5, 2048 + 68, 128, 2, 6, 29, seed=11),
    "sixteen_groups_gs3": Case(4, 4, 3, 1024 + 68, 64, 1, 4, 15, seed=12),
    "twentyfour_groups_gs7": Case(3, 8, 7, 1536 + 68, 96, 2, 5, 22, seed=13),
    "thirty_groups_gs4": Case(5, 6, 4, 1024 + 68, 64, 1, 4, 15, seed=14),
    # the fp16 instantiations (one small group count, one that runs with 6-CTA clusters)
    "fp16_gs4": Case(2, 2, 4, 2048 + 68, 128, 1, 6, 30, seed=15, dtype=torch.float16),
    "fp16_sixteen_groups": Case(4, 4, 2, 1024 + 68, 64, 1, 4, 15, seed=16, dtype=torch.float16),
}


def run_oracle(case, cpu, q, static_len):
    return oat.compute(q, cpu["centroids"], cpu["value_sum"], cpu["cluster_size"], cpu["mask"],
                       cpu["cluster_count"], cpu["cluster_offset"], cpu["keys"], cpu["values"],
                       cpu["steady_keys"], cpu["steady_values"], static_len, case.nprobe,
                       case.nprobe + case.n_estimate, case.page_size, case.pages(), return_parts=True)


def ordered_key(dist: torch.Tensor) -> torch.Tensor:
    bits = dist.view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where(bits >= 0x8000, (~bits) & 0xFFFF, bits | 0x8000)


@pytest.mark.parametrize("mode", ["single_kernel", "single_kernel_global_lists", "single_kernel_short_lists", "staged"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_fused_decode_matches_oracle(name, mode):
    case = CASES[name]
    cpu = build_cpu_index(case)
    static_len = SINK + RECENT + 1
    # one generated token already appended
    cpu["steady_keys"][:, SINK + RECENT] = torch.randn((case.groups, 128)).to(case.dtype)
    cpu["steady_values"][:, SINK + RECENT] = torch.randn((case.groups, 128)).to(case.dtype)
    layer = to_gpu_layer(case, cpu, static_len)
    q = queries(case)
    ref_out, parts = run_oracle(case, cpu, q, static_len)

    if mode == "staged":
        out = layer.compute_staged(q.cuda())
    elif mode == "single_kernel":
        out = layer.compute(q.cuda())
    else:   # no (or too little) room for estimation entries in shared memory: the kernel falls back to its
        # global lists — with 16 entries some CTAs have already started copies for the shared-memory form
        from retrievalattention_b200 import _lib
        _lib.lib.ri_wave_test_local_cap(0 if mode == "single_kernel_global_lists" else 16)
        try:
            out = layer.compute(q.cuda())
        finally:
            _lib.lib.ri_wave_test_local_cap(-1)
    torch.cuda.synchronize()
    v = layer.views()

    # scores: alpha * q.c in fp32
    ref_scores = torch.bmm(q.reshape(case.groups, case.group_size, 128).float(),
                           cpu["centroids"].float().transpose(1, 2)) / 128 ** 0.5
    torch.testing.assert_close(v["scores"].cpu(), ref_scores, rtol=1e-4, atol=1e-3)

    # 16-bit distance keys: bit-exact up to the rare rounding flip caused by fp32 summation order
    keys = (v["dist_keys"].cpu().to(torch.int32) & 0xFFFF)
    ref_keys = ordered_key(parts["dist"])
    assert (keys != ref_keys).float().mean() < 0.02
    assert ((keys - ref_keys).abs() <= 1).all()

    # selected sets, with the tie rule
    dist = parts["dist"]
    ret = layer.retrieved_ids.cpu()
    assert oss.selection_matches(dist, ret, case.nprobe)
    if case.n_estimate:
        both = torch.cat((ret, layer.estimated_ids.cpu()), dim=1)
        assert oss.selection_matches(dist, both, case.nprobe + case.n_estimate)
    # ranking of the retrieved clusters is descending
    d_ret = torch.gather(dist.float(), 1, ret)
    assert (d_ret[:, :-1] >= d_ret[:, 1:] - 1e-3).all()

    # page-budget rule on the kernel's own ranking
    kept = layer.retrieved_kept.cpu()
    for g in range(case.groups):
        expect = oat.surviving_clusters(ret[g], cpu["cluster_count"][g], case.page_size, case.pages())
        assert int(kept[g]) == expect
        rows = []
        for cid in ret[g, :expect].tolist():
            rows.extend(range(int(cpu["cluster_offset"][g, cid]), int(cpu["cluster_offset"][g, cid + 1])))
        assert int(v["n_exact"][g]) == len(rows)
        assert v["exact_rows"][g, :len(rows)].cpu().tolist() == rows

    # attention output
    err = (out.cpu().float() - ref_out.float()).abs()
    assert err.max() <= 2e-2, f"max abs err {err.max():.4f}"
    assert err.mean() <= 2e-3, f"mean abs err {err.mean():.5f}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_single_kernel_without_id_outputs(name):
    """The form a decode loop runs: no id outputs requested, so the kernel keeps its lists in shared
    memory, skips the ranking when every retrieved cluster fits the page budget, and writes nothing
    but the attention output.  Same tolerance against the oracle; and the output must agree with the
    id-producing form of the same kernel to summation-order noise."""
    case = CASES[name]
    cpu = build_cpu_index(case)
    static_len = SINK + RECENT
    q = queries(case)
    ref_out, _ = run_oracle(case, cpu, q, static_len)
    plain = to_gpu_layer(case, cpu, static_len, want_ids=False)
    out = plain.compute(q.cuda())
    with_ids = to_gpu_layer(case, cpu, static_len, want_ids=True).compute(q.cuda())
    torch.cuda.synchronize()
    err = (out.cpu().float() - ref_out.float()).abs()
    assert err.max() <= 2e-2, f"max abs err {err.max():.4f}"
    assert err.mean() <= 2e-3, f"mean abs err {err.mean():.5f}"
    assert (out.float() - with_ids.float()).abs().max() <= 1e-2


def test_tight_budget_actually_cuts():
    case = CASES["tight_budget"]
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    layer.compute(queries(case).cuda())
    torch.cuda.synchronize()
    assert (layer.retrieved_kept.cpu() < case.nprobe).any()


def test_empty_clusters_rank_last():
    case = CASES["empty_clusters"]
    cpu = build_cpu_index(case)
    assert int(cpu["mask"].sum()) > 0
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    layer.compute(queries(case).cuda())
    torch.cuda.synchronize()
    ret = layer.retrieved_ids.cpu()
    nonempty = (~cpu["mask"]).sum(1)
    for g in range(case.groups):
        if nonempty[g] >= case.nprobe:
            assert not cpu["mask"][g, ret[g]].any()


def test_repeatable_and_scratch_reusable():
    """Two calls in a row on the same scratch give bit-identical results (no stage depends on
    what the scratch held before, and the selection and the merge order are deterministic)."""
    case = CASES["small_gs4"]
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    q = queries(case).cuda()
    a = layer.compute(q).clone()
    b = layer.compute(q).clone()
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_steady_append_and_growing_static_len():
    from retrievalattention_b200 import wave

    case = CASES["small_gs4"]
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    pos = layer.t["static_len"]
    q = queries(case, seed=7)
    for step in range(3):
        k_new = torch.randn((case.batch, 1, case.kv_heads, 128)).to(case.dtype)
        v_new = torch.randn((case.batch, 1, case.kv_heads, 128)).to(case.dtype)
        wave.steady_append(k_new.cuda(), v_new.cuda(), layer.t["steady_keys"], layer.t["steady_values"], pos)
        cpu["steady_keys"][:, SINK + RECENT + step] = k_new.reshape(case.groups, 128)
        cpu["steady_values"][:, SINK + RECENT + step] = v_new.reshape(case.groups, 128)
        pos += 1
        static_len = SINK + RECENT + step + 1
        out = layer.compute(q.cuda())
        ref_out, _ = run_oracle(case, cpu, q, static_len)
        err = (out.cpu().float() - ref_out.float()).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3
    assert torch.equal(layer.t["steady_keys"].cpu(), cpu["steady_keys"])


@pytest.mark.parametrize("want_ids", [False, True])
def test_append_done_by_the_decode_kernel(want_ids):
    """The step's key/value rows handed to the decode call: the kernel stores them at row static_len - 1 of the
    steady zone before it attends — same steady zone and same output as a separate append followed by compute."""
    case = CASES["small_gs4"]
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT, want_ids=want_ids)
    pos = layer.t["static_len"]
    q = queries(case, seed=9)
    for step in range(3):
        k_new = torch.randn((case.batch, 1, case.kv_heads, 128)).to(case.dtype)
        v_new = torch.randn((case.batch, 1, case.kv_heads, 128)).to(case.dtype)
        cpu["steady_keys"][:, SINK + RECENT + step] = k_new.reshape(case.groups, 128)
        cpu["steady_values"][:, SINK + RECENT + step] = v_new.reshape(case.groups, 128)
        pos += 1                                   # the step attends static_len rows, the new one included
        layer.append_with_next_compute(k_new.cuda(), v_new.cuda())
        out = layer.compute(q.cuda())
        ref_out, _ = run_oracle(case, cpu, q, SINK + RECENT + step + 1)
        err = (out.cpu().float() - ref_out.float()).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3
        again = layer.compute(q.cuda())            # no rows pending: nothing is appended, same result
        assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    assert torch.equal(layer.t["steady_keys"].cpu(), cpu["steady_keys"])
    assert torch.equal(layer.t["steady_values"].cpu(), cpu["steady_values"])


def test_invalid_arguments_are_rejected():
    import ctypes as C
    from retrievalattention_b200 import _lib

    p = _lib.WaveLayer()
    assert _lib.lib.ri_wave_decode_layer(C.byref(p), None) == -1
    assert b"groups" in _lib.lib.ri_last_error()


def _random_case(seed: int) -> Case:
    """A geometry drawn at random: 1 .. 40 groups (every cluster size of the single kernel), every group size, centroid
    counts that do not divide evenly over 5, 6 or 7 CTAs."""
    rng = torch.Generator().manual_seed(1000 + seed)
    pick = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=rng))   # noqa: E731
    batch, kv_heads = pick(1, 8), pick(1, 5)
    n_segment = pick(1, 2)
    n_centroids = 8 * n_segment * pick(4, 12)
    nprobe = pick(2, 6)
    return Case(batch, kv_heads, pick(1, 8), 68 + 16 * n_centroids + 8 * pick(0, 40), n_centroids, n_segment, nprobe,
                pick(0, n_centroids // 3), seed=100 + seed)


@pytest.mark.parametrize("seed", range(16))
def test_random_geometries_single_kernel_against_oracle_and_stages(seed):
    case = _random_case(seed)
    cpu = build_cpu_index(case)
    static_len = SINK + RECENT
    q = queries(case)
    ref_out, parts = run_oracle(case, cpu, q, static_len)
    layer = to_gpu_layer(case, cpu, static_len)
    out = layer.compute(q.cuda()).clone()
    ret, est = layer.retrieved_ids.cpu().clone(), layer.estimated_ids.cpu().clone()
    staged = layer.compute_staged(q.cuda()).clone()
    plain = to_gpu_layer(case, cpu, static_len, want_ids=False).compute(q.cuda())
    torch.cuda.synchronize()
    what = (case.groups, case.group_size, case.n_centroids, case.nprobe, case.n_estimate)
    assert oss.selection_matches(parts["dist"], ret, case.nprobe), what
    if case.n_estimate:
        assert oss.selection_matches(parts["dist"], torch.cat((ret, est), dim=1), case.nprobe + case.n_estimate), what
    for name, o in (("single kernel", out), ("stages", staged), ("output only", plain)):
        err = (o.cpu().float() - ref_out.float()).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (name, what, float(err.max()), float(err.mean()))
    # the three forms sum in different orders: they may differ by a rounding step of the 16-bit output or two
    for other in (staged, plain):
        assert ((out.float() - other.float()).abs() <= 2.0 ** -6 * out.float().abs().clamp_min(0.5)).all(), what
