"""Dense prefill attention (``ri_prefill_attn`` behind ``retroinfer_prefill_attn``, the replacement of the reference's
flash-attn call, attn_hub/retroinfer_attn.py:4-13) against fp32 PyTorch attention.

Tolerance (bf16 probabilities and outputs, fp32 accumulation): max-abs <= 2e-2, mean-abs <= 2e-3."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(q, k, v, causal):
    b, s, hq, d = q.shape
    hk = k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)                                   # [B, Hq, S, d]
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(hq // hk, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(hq // hk, dim=1)
    out = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=bool(causal))
    return out.permute(0, 2, 1, 3)


@pytest.mark.parametrize("batch,seq,hq,hk,causal,dtype", [
    (1, 1024, 4, 1, True, torch.bfloat16),
    (2, 1000, 8, 2, True, torch.bfloat16),       # ragged: last tile partly empty, rows of the next request behind it
    (1, 128, 2, 2, True, torch.bfloat16),        # a single tile
    (1, 77, 4, 4, True, torch.float16),          # shorter than one tile
    (2, 640, 4, 2, False, torch.bfloat16),       # not causal
    (1, 4096, 8, 2, True, torch.bfloat16),
    (1, 16384, 2, 1, True, torch.bfloat16),
])
def test_prefill_attention_matches_fp32(batch, seq, hq, hk, causal, dtype):
    from retrievalattention_b200.attn_hub import retroinfer_attn as ra

    g = torch.Generator(device="cuda").manual_seed(seq + hq)
    mk = lambda h, scale: (torch.randn((batch, seq, h, 128), generator=g, device="cuda") * scale).to(dtype)   # noqa: E731
    q, k, v = mk(hq, 1.5), mk(hk, 1.5), mk(hk, 1.0)
    out = ra.retroinfer_prefill_attn(q, k, v, causal)
    ra.check_prefill_errors()
    ref = reference(q, k, v, causal)
    err = (out.float() - ref).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (float(err.max()), float(err.mean()))


def test_large_scores_move_the_reference_maximum():
    """Scores that keep growing along the sequence force the lazy reference maximum to move (the accumulator is
    rescaled in tensor memory) many times."""
    from retrievalattention_b200.attn_hub import retroinfer_attn as ra

    torch.manual_seed(3)
    seq = 1536
    q = torch.randn((1, seq, 2, 128), device="cuda")
    k = torch.randn((1, seq, 1, 128), device="cuda")
    ramp = torch.linspace(0.2, 6.0, seq, device="cuda")[None, :, None, None]
    k = (k * 0.3 + q[:, :, :1] * 0.05 * ramp)             # later keys score higher against every query
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    v = torch.randn((1, seq, 1, 128), device="cuda").to(torch.bfloat16)
    out = ra.retroinfer_prefill_attn(q, k, v, True)
    ra.check_prefill_errors()
    err = (out.float() - reference(q, k, v, True)).abs()
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (float(err.max()), float(err.mean()))


def test_bad_arguments_are_rejected():
    from retrievalattention_b200 import _lib

    assert _lib.lib.ri_prefill_attn(None, None, None, None, None, None, 1, 128, 4, 1, 1, 0, None) == -1
    assert _lib.lib.ri_prefill_attn_scratch_bytes(1, 0, 1) == -1
    assert _lib.lib.ri_prefill_attn_scratch_bytes(2, 1000, 2) == 2 * 2 * 128 * 1024 * 2
