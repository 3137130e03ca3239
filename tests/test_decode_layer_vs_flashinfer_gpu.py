"""The element-wise kernels of the decode layer against the flashinfer calls the reference itself makes
(model_hub/llama.py:272 ``flashinfer.activation.silu_and_mul``, :307 ``flashinfer.rmsnorm``, :317
``flashinfer.rope.apply_rope_with_cos_sin_cache_inplace(..., is_neox=True)``), on the same tensors.  Both sides
compute in fp32 and round once to the 16-bit type, so the results may differ by the last place of that type, and
nearly all elements are bit-equal.  Skipped where flashinfer is absent or cannot build its kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


def flashinfer_or_skip():
    try:
        import flashinfer
        return flashinfer
    except Exception as exc:      # noqa: BLE001
        pytest.skip(f"flashinfer unavailable: {exc!r}"[:200])


def one_ulp(out, ref, frac_equal=0.97):
    a, b = out.float(), ref.float()
    assert ((a - b).abs() <= 2.0 ** -7 * b.abs().clamp_min(2.0 ** -10)).all(), float((a - b).abs().max())
    assert (out.view(torch.int16) == ref.view(torch.int16)).float().mean() >= frac_equal


@pytest.mark.parametrize("rows,dim", [(4, 4096), (16, 8192), (1, 3584)])
def test_rmsnorm_against_flashinfer(rows, dim):
    fi = flashinfer_or_skip()
    from retrievalattention_b200.decode_layer import rmsnorm

    g = torch.Generator(device="cuda").manual_seed(dim + rows)
    x = torch.randn((rows, dim), generator=g, device="cuda").to(DT)
    w = (1 + 0.1 * torch.randn((dim,), generator=g, device="cuda")).to(DT)
    try:
        ref = fi.rmsnorm(x, w, 1e-5)
    except Exception as exc:      # noqa: BLE001
        pytest.skip(f"flashinfer.rmsnorm could not run: {exc!r}"[:200])
    out = torch.empty_like(x)
    rmsnorm(x, w, 1e-5, out)
    torch.cuda.synchronize()
    one_ulp(out, ref)


@pytest.mark.parametrize("rows,inter", [(4, 14336), (8, 18944)])
def test_silu_and_mul_against_flashinfer(rows, inter):
    fi = flashinfer_or_skip()
    from retrievalattention_b200.decode_layer import silu_and_mul

    g = torch.Generator(device="cuda").manual_seed(inter)
    x = torch.randn((rows, 2 * inter), generator=g, device="cuda").to(DT)
    try:
        ref = fi.activation.silu_and_mul(x)
    except Exception as exc:      # noqa: BLE001
        pytest.skip(f"flashinfer silu_and_mul could not run: {exc!r}"[:200])
    out = torch.empty((rows, inter), dtype=DT, device="cuda")
    silu_and_mul(x, out)
    torch.cuda.synchronize()
    one_ulp(out, ref, frac_equal=0.95)


@pytest.mark.parametrize("rows,q_heads,kv_heads", [(4, 32, 8), (8, 28, 4)])
def test_rope_split_against_flashinfer(rows, q_heads, kv_heads):
    fi = flashinfer_or_skip()
    from retrievalattention_b200.decode_layer import cos_sin_cache, rope_split

    g = torch.Generator(device="cuda").manual_seed(rows)
    heads = q_heads + 2 * kv_heads
    qkv = torch.randn((rows, heads * 128), generator=g, device="cuda").to(DT)
    cache = cos_sin_cache(4096, 128, 5e5, "cuda")
    pos = torch.randint(0, 4096, (rows,), generator=g, device="cuda", dtype=torch.int64)
    q_ref = qkv[:, :q_heads * 128].clone()
    k_ref = qkv[:, q_heads * 128:(q_heads + kv_heads) * 128].clone()
    try:
        fi.rope.apply_rope_with_cos_sin_cache_inplace(pos, q_ref, k_ref, 128, cache, True)
    except Exception as exc:      # noqa: BLE001
        pytest.skip(f"flashinfer rope could not run: {exc!r}"[:200])
    q = torch.empty((rows, 1, q_heads, 128), dtype=DT, device="cuda")
    k = torch.empty((rows, 1, kv_heads, 128), dtype=DT, device="cuda")
    v = torch.empty((rows, 1, kv_heads, 128), dtype=DT, device="cuda")
    rope_split(qkv, cache, pos, q, k, v)
    torch.cuda.synchronize()
    one_ulp(q.view(rows, -1), q_ref)
    one_ulp(k.view(rows, -1), k_ref)
    assert torch.equal(v.view(rows, -1), qkv[:, (q_heads + kv_heads) * 128:])
