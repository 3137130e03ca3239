"""The weighted_flash_decoding operator against the CPU restatement of its call-site semantics
(oracle/attention.py — parity unpinned: the reference imports the operator from an external package that is
not in its tree).  Covers the reference's two uses: weighted rows with the log-sum-exp returned
(cache_hub/retroinfer_cache.py:611-617) and valid lengths with a previous partial result merged in (:666-674).
Tolerances: output max-abs 2e-2, mean-abs 2e-3; lse 2e-2."""
import pytest
import torch

from oracle import attention as oat
from retrievalattention_b200 import kernels

pytestmark = pytest.mark.gpu


def rand(shape, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("groups,gs,length,dtype", [(6, 4, 1900, torch.bfloat16), (3, 7, 333, torch.float16),
                                                    (2, 8, 16, torch.bfloat16), (4, 1, 5, torch.bfloat16)])
def test_weighted_rows_and_lse(groups, gs, length, dtype):
    q = rand((groups, 1, gs, 128), 1, dtype)
    k = rand((groups, length, 1, 128), 2, dtype)
    v = rand((groups, length, 1, 128), 3, dtype, 4.0)          # "value sums"
    w = torch.randint(1, 40, (groups, 1, 1, length), generator=torch.Generator().manual_seed(4)).to(dtype)
    ref_out, ref_lse = oat.weighted_flash_decoding(q, k, v, w, return_softmax_lse=True, out_dtype=torch.float32)
    out, lse = kernels.weighted_flash_decoding(q.cuda(), k.cuda(), v.cuda(), w.cuda(), return_softmax_lse=True)
    torch.cuda.synchronize()
    err = (out.cpu().float() - ref_out).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (float(err.max()), float(err.mean()))
    assert (lse.cpu() - ref_lse).abs().max() <= 2e-2


@pytest.mark.parametrize("groups,gs,stride,dtype", [(5, 4, 2500, torch.bfloat16), (2, 7, 700, torch.float16)])
def test_valid_lengths_and_merge_with_previous(groups, gs, stride, dtype):
    q = rand((groups, 1, gs, 128), 11, dtype)
    k = rand((groups, stride, 1, 128), 12, dtype)
    v = rand((groups, stride, 1, 128), 13, dtype)
    lens = torch.randint(1, stride, (groups,), generator=torch.Generator().manual_seed(14)).to(torch.int32)
    lens[0] = stride
    prev_out = rand((groups, 1, gs, 128), 15, dtype)
    prev_lse = rand((groups, gs, 1), 16, torch.float32, 2.0) + 3.0
    ref = oat.weighted_flash_decoding(q, k, v, previous_out=prev_out, previous_lse=prev_lse, cache_seqlens=lens,
                                      out_dtype=torch.float32)
    out = kernels.weighted_flash_decoding(q.cuda(), k.cuda(), v.cuda(), previous_out=prev_out.cuda(),
                                          previous_lse=prev_lse.cuda(), cache_seqlens=lens.cuda())
    torch.cuda.synchronize()
    err = (out.cpu().float() - ref).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (float(err.max()), float(err.mean()))


def test_the_two_calls_chained_equal_one_pass_over_everything():
    """Estimation zone first (weights, lse out), exact zone second (merge): the reference's sequence."""
    dtype, groups, gs = torch.bfloat16, 4, 4
    q = rand((groups, 1, gs, 128), 21, dtype)
    ke, ve = rand((groups, 96, 1, 128), 22, dtype), rand((groups, 96, 1, 128), 23, dtype, 3.0)
    w = torch.randint(1, 30, (groups, 1, 1, 96), generator=torch.Generator().manual_seed(24)).to(dtype)
    kx, vx = rand((groups, 640, 1, 128), 25, dtype), rand((groups, 640, 1, 128), 26, dtype)
    lens = torch.tensor([640, 17, 300, 1], dtype=torch.int32)
    es_out, es_lse = kernels.weighted_flash_decoding(q.cuda(), ke.cuda(), ve.cuda(), w.cuda(), return_softmax_lse=True)
    out = kernels.weighted_flash_decoding(q.cuda(), kx.cuda(), vx.cuda(), previous_out=es_out, previous_lse=es_lse,
                                          cache_seqlens=lens.cuda())
    r_out, r_lse = oat.weighted_flash_decoding(q, ke, ve, w, return_softmax_lse=True, out_dtype=torch.float32)
    ref = oat.weighted_flash_decoding(q, kx, vx, previous_out=r_out, previous_lse=r_lse, cache_seqlens=lens,
                                      out_dtype=torch.float32)
    torch.cuda.synchronize()
    err = (out.cpu().float() - ref).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (float(err.max()), float(err.mean()))
