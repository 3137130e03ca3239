"""Seeded synthetic keys, values and queries with the shapes of the benchmark
configurations.

Stands in for real prompts and checkpoints.  Keys are Gaussian with a
per-channel outlier scale and rotary position embedding applied (neox
half-split layout, as the reference applies it before the cache sees the keys,
model_hub/llama.py:304-310); values and queries are standard normal.
"""
from __future__ import annotations

import torch


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate ``x[..., n, d]`` (fp32) by position; first half / second half pairing."""
    d = x.shape[-1]
    half = d // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=x.device) / half))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def make_kv(kv_heads: int, n_tokens: int, head_dim: int, *, seed: int, theta: float = 5e5,
            device: str | torch.device = "cpu", dtype: torch.dtype = torch.bfloat16,
            outlier_std: float = 3.0, planted_centres: int = 0):
    """One request's K and V for one layer, shaped ``[1, n_tokens, kv_heads, head_dim]``
    like the tensors ``prefill_update_kv_cache`` receives.

    ``planted_centres > 0`` adds a per-head mixture centre to each key before the
    rotation (a more clusterable secondary distribution).
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    k0 = torch.randn((kv_heads, n_tokens, head_dim), generator=gen, device=device, dtype=torch.float32)
    sigma = (torch.randn((kv_heads, 1, head_dim), generator=gen, device=device, dtype=torch.float32)
             * outlier_std).abs()
    k0 = k0 * sigma
    if planted_centres > 0:
        centres = torch.randn((kv_heads, planted_centres, head_dim), generator=gen, device=device) * 4.0
        which = torch.randint(0, planted_centres, (kv_heads, n_tokens), generator=gen, device=device)
        k0 = k0 + torch.gather(centres, 1, which[..., None].expand(-1, -1, head_dim))
    pos = torch.arange(n_tokens, device=device)
    k = rope_neox(k0, pos, theta).to(dtype)
    v = torch.randn((kv_heads, n_tokens, head_dim), generator=gen, device=device, dtype=torch.float32).to(dtype)
    return k.transpose(0, 1).unsqueeze(0).contiguous(), v.transpose(0, 1).unsqueeze(0).contiguous()


def make_queries(batch: int, q_heads: int, head_dim: int, *, seed: int,
                 device: str | torch.device = "cpu", dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Decode-step queries ``[batch, 1, q_heads, head_dim]``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return torch.randn((batch, 1, q_heads, head_dim), generator=gen, device=device,
                       dtype=torch.float32).to(dtype)
