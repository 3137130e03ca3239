"""The batch_gemm_softmax operator against the reference's own oracle for it (bmm -> scale -> softmax,
library/retroinfer/test/test_batch_gemm_softmax.py:9-18, tolerance atol 1e-3 as there), with seeds,
for the shape of that test (n = 8200, not a multiple of 256), the decode shapes and both dtypes."""
import math

import pytest
import torch

from retrievalattention_b200 import kernels

pytestmark = pytest.mark.gpu


def oracle(A, B):
    dist = torch.bmm(A.float(), B.float().transpose(1, 2)) / math.sqrt(A.size(-1))
    return dist, torch.softmax(dist.to(A.dtype).float(), dim=-1)


@pytest.mark.parametrize("batch,m,n,dtype", [
    (16, 4, 8200, torch.bfloat16),     # the reference test's shape (scaled-down batch)
    (32, 4, 8192, torch.bfloat16),     # config 1
    (3, 7, 1000, torch.float16),       # Qwen group size, ragged n
    (2, 8, 8, torch.bfloat16),         # one 8-column tile
    (5, 1, 520, torch.bfloat16),
])
def test_matches_bmm_softmax(batch, m, n, dtype):
    g = torch.Generator(device="cuda").manual_seed(n * 31 + m)
    A = torch.randn((batch, m, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    B = torch.randn((batch, n, 128), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    D = torch.zeros((batch, m, n), device="cuda", dtype=dtype)
    S = torch.zeros_like(D)
    blocks = (n + 255) // 256
    norm = torch.zeros((batch, m, blocks), device="cuda", dtype=torch.float32)
    ssum = torch.zeros_like(norm)
    kernels.batch_gemm_softmax(A, B, D, norm, ssum, S, batch, m, n, 128, 1 / math.sqrt(128), 0)
    torch.cuda.synchronize()
    ref_d, ref_s = oracle(A, B)
    # D is the fp32 product rounded once to the 16-bit type
    assert (D.float() - ref_d).abs().max() <= (0.04 if dtype == torch.bfloat16 else 0.01)
    assert torch.allclose(S.float(), ref_s, atol=1e-3), float((S.float() - ref_s).abs().max())
    assert torch.allclose(S.float().sum(-1), torch.ones((batch, m), device="cuda"), atol=2e-2)


def test_rejects_what_it_does_not_support():
    A = torch.zeros((1, 4, 128), device="cuda", dtype=torch.bfloat16)
    B = torch.zeros((1, 16, 128), device="cuda", dtype=torch.bfloat16)
    D = torch.zeros((1, 4, 16), device="cuda", dtype=torch.bfloat16)
    f = torch.zeros((1, 4, 1), device="cuda", dtype=torch.float32)
    with pytest.raises(RuntimeError):
        kernels.batch_gemm_softmax(A, B, D, f, f.clone(), D.clone(), 1, 4, 16, 128, 1.0, 0.5)     # beta != 0
    with pytest.raises(ValueError):
        kernels.batch_gemm_softmax(A, B, D, f, f.clone(), D.clone(), 1, 4, 24, 128, 1.0, 0.0)     # sizes do not match
