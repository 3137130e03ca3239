"""The output gather done by the decode kernel (ri_wave_decode_layer_gather / ri_wave_gather_wait).

One GPU stands in for a group of two ranks: both "ranks" are layers of this process, their gather
buffers and flag words are ordinary local tensors, and the launches run one after the other on one
stream — the wait kernel only ever waits for flags that earlier launches of the same stream have
already raised, or, in the time-out test, for a flag that nothing raises (it must give up after its
limit and report it, never hang)."""
import ctypes as C

import pytest
import torch

from helpers import Case, build_cpu_index, queries, to_gpu_layer, SINK, RECENT
from retrievalattention_b200 import _lib

pytestmark = pytest.mark.gpu

CASE = Case(2, 2, 4, 2048 + 68, 128, 1, 6, 30, seed=11)


def make_gather(rank, n, out_bufs, flag_bufs, epoch, error, limit_us, keep):
    slice_bytes = out_bufs[0][0].numel() * out_bufs[0].element_size()
    out_slots = torch.tensor([b.data_ptr() + rank * slice_bytes for b in out_bufs], dtype=torch.int64).cuda()
    flag_slots = torch.tensor([f.data_ptr() + rank * 4 for f in flag_bufs], dtype=torch.int64).cuda()
    keep += [out_slots, flag_slots]
    g = _lib.WaveGather()
    g.n_ranks, g.rank, g.wait_limit_us = n, rank, limit_us
    g.d_out_slots, g.d_flag_slots = out_slots.data_ptr(), flag_slots.data_ptr()
    g.d_flags = flag_bufs[rank].data_ptr()
    g.d_epoch, g.d_error = epoch.data_ptr(), error.data_ptr()
    return g


def test_two_ranks_on_one_gpu_fill_both_buffers_and_the_wait_returns():
    cpu = build_cpu_index(CASE)
    layers = [to_gpu_layer(CASE, cpu, SINK + RECENT, want_ids=False) for _ in range(2)]
    qs = [queries(CASE).cuda(), (queries(CASE) * 0.5).to(torch.bfloat16).cuda()]
    g_, gs = CASE.groups, CASE.group_size
    out_bufs = [torch.zeros((2, g_, gs, 128), dtype=torch.bfloat16, device="cuda") for _ in range(2)]   # per "rank"
    flag_bufs = [torch.zeros((2,), dtype=torch.int32, device="cuda") for _ in range(2)]
    epoch = torch.zeros((1,), dtype=torch.int32, device="cuda")
    error = torch.zeros((1,), dtype=torch.int32, device="cuda")
    keep = []
    gathers = [make_gather(r, 2, out_bufs, flag_bufs, epoch, error, 3000, keep) for r in range(2)]
    for step in range(3):
        epoch.add_(1)
        outs = [layers[r].compute(qs[r], gather=gathers[r]).clone() for r in range(2)]
        # "rank" 0 raises its flags and gives up waiting for rank 1's, which only the next call raises: on one
        # GPU the two calls cannot run side by side, so the first wait must run out (and must not hang)
        _lib.check(_lib.lib.ri_wave_gather_wait(C.byref(gathers[0]), _lib.current_stream()))
        torch.cuda.synchronize()
        assert int(error.item()) == 1
        error.zero_()
        _lib.check(_lib.lib.ri_wave_gather_wait(C.byref(gathers[1]), _lib.current_stream()))   # finds both flags
        torch.cuda.synchronize()
        assert int(error.item()) == 0
        for buf in out_bufs:                    # every rank's buffer holds both slices
            for r in range(2):
                assert torch.equal(buf[r].view(torch.int16), outs[r].reshape(g_, gs, 128).view(torch.int16))
        for f in flag_bufs:
            assert (f == step + 1).all()
    plain = layers[0].compute(qs[0])            # the gather form computes what the plain form computes
    torch.cuda.synchronize()
    assert torch.equal(plain.view(torch.int16), outs[0].view(torch.int16))


def test_gather_form_beyond_the_single_kernel():
    """8256 centroids (what configuration 1 has after one re-index of generated tokens): the gather entry point runs
    the three stage kernels and the attend stage stores the slice into every rank's buffer."""
    from helpers import gpu_built_layer

    layers, _, q = gpu_built_layer(1, 2, 4, 8256 * 16, 8256, 1, 148, 1915, seed=12, want_ids=False, n_layers=2)
    g_, gs = 2, 4
    out_bufs = [torch.zeros((2, g_, gs, 128), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flag_bufs = [torch.zeros((2,), dtype=torch.int32, device="cuda") for _ in range(2)]
    epoch = torch.ones((1,), dtype=torch.int32, device="cuda")
    error = torch.zeros((1,), dtype=torch.int32, device="cuda")
    keep = []
    gathers = [make_gather(r, 2, out_bufs, flag_bufs, epoch, error, 3000, keep) for r in range(2)]
    outs = [layers[r].compute(q, gather=gathers[r]).clone() for r in range(2)]
    plain = layers[0].compute(q).clone()
    torch.cuda.synchronize()
    assert torch.equal(plain.view(torch.int16), outs[0].view(torch.int16))
    for buf in out_bufs:
        for r in range(2):
            assert torch.equal(buf[r].view(torch.int16), outs[r].reshape(g_, gs, 128).view(torch.int16))


def test_wait_gives_up_after_its_limit_and_reports_it():
    flags = torch.zeros((2,), dtype=torch.int32, device="cuda")        # only this rank's own flag is ever raised
    mine = torch.zeros((2,), dtype=torch.int32, device="cuda")
    epoch = torch.ones((1,), dtype=torch.int32, device="cuda")
    error = torch.zeros((1,), dtype=torch.int32, device="cuda")
    slots = torch.tensor([flags.data_ptr(), mine.data_ptr()], dtype=torch.int64).cuda()   # own flag here, peer's elsewhere
    g = _lib.WaveGather()
    g.n_ranks, g.rank, g.wait_limit_us = 2, 0, 2000
    g.d_out_slots = g.d_flag_slots = slots.data_ptr()
    g.d_flags, g.d_epoch, g.d_error = flags.data_ptr(), epoch.data_ptr(), error.data_ptr()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    _lib.check(_lib.lib.ri_wave_gather_wait(C.byref(g), _lib.current_stream()))
    b.record()
    torch.cuda.synchronize()
    assert int(error.item()) == 1
    assert 1.0 <= a.elapsed_time(b) < 200.0     # about the 2 ms limit, and the context is still usable
    assert torch.zeros(4, device="cuda").sum().item() == 0.0


def test_invalid_gather_arguments_are_rejected():
    g = _lib.WaveGather()
    g.n_ranks, g.rank = 1, 0
    assert _lib.lib.ri_wave_gather_wait(C.byref(g), None) != 0
    g.n_ranks, g.rank = 2, 5
    assert _lib.lib.ri_wave_gather_wait(C.byref(g), None) != 0
