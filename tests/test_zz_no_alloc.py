"""The allocation-free entry point ``ri_wave_decode_layer_static`` against the regular one.

Some hosts cannot give the library scratch memory: a server that reserved all of HBM for its own
pool, or a decode loop that forbids cudaMalloc because it stalls the device.  For them the
library carries a fixed 16 MiB scratch inside its own image.  This file checks, through the C
ABI, that the result is the same as with caller-provided scratch — on two calls in a row, since
the second call finds the first one's leftovers in the shared array — and that a geometry too
large for the array is refused.  It is named to be collected last.
"""
import ctypes as C

import pytest
import torch

from helpers import Case, build_cpu_index, queries, to_gpu_layer, SINK, RECENT

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_caller_scratch_twice():
    case = Case(2, 2, 4, 2048 + 68, 128, 1, 6, 30, seed=21)
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    for call, seed in enumerate((31, 32)):
        q = queries(case, seed=seed).cuda()
        expect = layer.compute(q).clone()
        got = layer.compute_static(q).clone()
        torch.cuda.synchronize()
        err = (got.float() - expect.float()).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, f"call {call}: max {err.max():.4f} mean {err.mean():.5f}"
        # same kernels, same inputs, deterministic selection: the bits agree as well
        assert torch.equal(got.view(torch.int16), expect.view(torch.int16))


def test_static_scratch_three_stage_geometry_on_a_used_array():
    """More than 8192 centroids: the entry point runs the three stage kernels, whose intermediate results all go
    through the scratch.  Run right after a call of another geometry, so that the built-in array holds that
    call's leftovers; the result must equal the caller-scratch path to the bit."""
    from helpers import gpu_built_layer

    small = Case(1, 2, 4, 1024 + 68, 64, 1, 4, 15, seed=23)
    small_layer = to_gpu_layer(small, build_cpu_index(small), SINK + RECENT)
    (layer,), _, q = gpu_built_layer(1, 1, 4, 8256 * 16, 8256, 1, 148, 1915, seed=24)
    assert layer.shape.scratch_bytes() <= 16 << 20
    for call in range(2):
        small_layer.compute_static(queries(small, seed=40 + call).cuda())      # dirties the shared array
        expect = layer.compute(q).clone()
        got = layer.compute_static(q).clone()
        torch.cuda.synchronize()
        err = (got.float() - expect.float()).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3
        assert torch.equal(got.view(torch.int16), expect.view(torch.int16))


def test_static_scratch_ignores_caller_scratch_pointer():
    case = Case(1, 2, 4, 1024 + 68, 64, 1, 4, 15, seed=22)
    cpu = build_cpu_index(case)
    layer = to_gpu_layer(case, cpu, SINK + RECENT)
    q = queries(case, seed=33).cuda()
    expect = layer.compute(q).clone()
    saved = layer.params.d_scratch
    layer.params.d_scratch = None          # a caller that owns no scratch at all
    try:
        got = layer.compute_static(q).clone()
    finally:
        layer.params.d_scratch = saved
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), expect.view(torch.int16))


def test_static_scratch_refuses_oversized_geometry():
    from retrievalattention_b200 import _lib, wave

    shape = wave.WaveShape(groups=256, group_size=8, n_centroids=16384, nprobe=294, n_estimate=3801, page_size=8,
                           buffer_pages=2352, tokens_per_group=262076, steady_stride=324)
    assert shape.scratch_bytes() > 16 << 20
    p = _lib.WaveLayer()
    shape.fill(p)
    rc = _lib.lib.ri_wave_decode_layer_static(C.byref(p), None)
    assert rc == -1
    msg = _lib.lib.ri_last_error().decode()
    assert "built-in array" in msg and "ri_wave_decode_layer" in msg
