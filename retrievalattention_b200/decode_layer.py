"""The decode layer around the wave-index attention, with random-initialised weights.

Mirror of the reference's decode loop (model_hub/LLM.py:90-126 ``layer_decode``, :156-171
``decode_forward``) for measuring decode tokens/s with the projections and the MLP included.
There are no checkpoints here, so the weights are seeded Gaussians at the model's true shapes.
The projections are plain library GEMMs (``torch.nn.functional.linear``, as the reference); the
element-wise work between them runs in this package's kernels (``ri_rmsnorm`` with the residual
add folded in, ``ri_rope_split``, ``ri_silu_and_mul``); the attention is
``decode_update_kv_cache`` + ``compute`` of a ``retroinfer_cache``.

Every buffer is allocated once, positions live on the device, and nothing synchronises: one
decode step can be captured in a CUDA graph and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib


@dataclass
class ModelShape:
    hidden: int
    intermediate: int
    vocab: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int = 128
    rope_theta: float = 5e5
    rms_eps: float = 1e-5

    @property
    def qkv_dim(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


# published geometries of the models the benchmark configurations name
LLAMA3_8B = ModelShape(4096, 14336, 128256, 32, 32, 8, rope_theta=5e5, rms_eps=1e-5)
QWEN25_7B = ModelShape(3584, 18944, 152064, 28, 28, 4, rope_theta=1e6, rms_eps=1e-6)
QWEN25_72B = ModelShape(8192, 29568, 152064, 80, 64, 8, rope_theta=1e6, rms_eps=1e-6)


def rmsnorm(x, weight, eps, out, residual=None):
    """``out = rmsnorm(residual + x) * weight`` (``residual`` updated in place) or ``rmsnorm(x) * weight``."""
    rows, dim = x.shape
    _lib.check(_lib.lib.ri_rmsnorm(x.data_ptr(), _lib.ptr(residual), weight.data_ptr(), out.data_ptr(), rows, dim,
                                   float(eps), _lib.dtype_code(x.dtype), _lib.current_stream()), "ri_rmsnorm")
    return out


def rope_split(qkv, cos_sin, positions, q, k, v):
    """Rotate the query/key heads of ``qkv`` ``[rows, (Hq+2Hk)*128]`` at ``positions`` and split into ``q, k, v``."""
    rows, q_heads, kv_heads = q.shape[0], q.shape[-2], k.shape[-2]
    assert qkv.shape == (rows, (q_heads + 2 * kv_heads) * 128) and cos_sin.dtype == torch.float32
    assert cos_sin.shape[1] == 128 and positions.dtype == torch.int64 and positions.numel() == rows
    _lib.check(_lib.lib.ri_rope_split(qkv.data_ptr(), cos_sin.data_ptr(), positions.data_ptr(), q.data_ptr(),
                                      k.data_ptr(), v.data_ptr(), rows, q_heads, kv_heads, cos_sin.shape[0],
                                      _lib.dtype_code(qkv.dtype), _lib.current_stream()), "ri_rope_split")


def silu_and_mul(x, out):
    rows, two_inter = x.shape
    _lib.check(_lib.lib.ri_silu_and_mul(x.data_ptr(), out.data_ptr(), rows, two_inter // 2, _lib.dtype_code(x.dtype),
                                        _lib.current_stream()), "ri_silu_and_mul")
    return out


def cos_sin_cache(max_positions: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """fp32 ``[max_positions, head_dim]``: cosines then sines (model_hub/llama.py:81-84, :109)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    freqs = torch.outer(torch.arange(max_positions, dtype=torch.float32, device=device), inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous()


class SyntheticDecoder:
    """Decode-only model with seeded random weights over a prepared ``retroinfer_cache``."""

    def __init__(self, shape: ModelShape, cache, batch: int, max_positions: int, device, dtype=torch.bfloat16,
                 seed: int = 0, std: float = 0.02, layers: int | None = None):
        self.shape, self.cache, self.batch, self.device, self.dtype = shape, cache, batch, device, dtype
        self.n_layers = shape.layers if layers is None else layers
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)

        def w(*s):
            return (torch.randn(s, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)

        h, it = shape.hidden, shape.intermediate
        self.embed = w(shape.vocab, h)
        self.lm_head = w(shape.vocab, h)
        self.final_norm = torch.ones(h, dtype=dtype, device=device)
        self.layers = []
        for _ in range(self.n_layers):
            self.layers.append(dict(wqkv=w(shape.qkv_dim, h), wo=w(h, shape.q_heads * shape.head_dim),
                                    gate_up=w(2 * it, h), down=w(h, it),
                                    norm1=torch.ones(h, dtype=dtype, device=device),
                                    norm2=torch.ones(h, dtype=dtype, device=device)))
        self.cos_sin = cos_sin_cache(max_positions, shape.head_dim, shape.rope_theta, device)
        # the position of the token being decoded, per request (the reference slices position_ids at
        # kv_cache.context, model_hub/llama.py:330-337); advanced on the device after every step
        self.positions = torch.full((batch,), int(cache.context), dtype=torch.int64, device=device)
        z = lambda *s: torch.zeros(s, dtype=dtype, device=device)  # noqa: E731
        self.input_ids = torch.zeros((batch,), dtype=torch.int64, device=device)
        self.residual, self.normed = z(batch, h), z(batch, h)
        self.q = z(batch, 1, shape.q_heads, shape.head_dim)
        self.k = z(batch, 1, shape.kv_heads, shape.head_dim)
        self.v = z(batch, 1, shape.kv_heads, shape.head_dim)
        self.attn = z(batch, 1, shape.q_heads, shape.head_dim)
        self.act = z(batch, it)
        self.next_ids = torch.zeros((batch,), dtype=torch.int64, device=device)

    def layer_decode(self, ldx: int, x: torch.Tensor) -> torch.Tensor:
        """One layer (model_hub/LLM.py:90-126).  ``x`` is the previous block's output that has not been
        added to the residual stream yet (None for the first layer: the residual holds the embedding)."""
        s, L = self.shape, self.layers[ldx]
        rmsnorm(self.residual if x is None else x, L["norm1"], s.rms_eps, self.normed,
                residual=None if x is None else self.residual)
        qkv = F.linear(self.normed, L["wqkv"])
        rope_split(qkv, self.cos_sin, self.positions, self.q, self.k, self.v)
        self.cache.decode_update_kv_cache(self.k, self.v, ldx)
        # attn_hub.retroinfer_decode_attn is cache.compute; called directly to hand it the output buffer
        attn = self.cache.compute(self.q, ldx, out=self.attn)
        o = F.linear(attn.view(self.batch, -1), L["wo"])
        rmsnorm(o, L["norm2"], s.rms_eps, self.normed, residual=self.residual)
        silu_and_mul(F.linear(self.normed, L["gate_up"]), self.act)
        return F.linear(self.act, L["down"])

    def decode_forward(self) -> torch.Tensor:
        """One decode step for ``input_ids`` (model_hub/LLM.py:156-171): logits ``[batch, vocab]`` fp32;
        the greedy next ids are left in ``next_ids`` and become ``input_ids`` of the next step."""
        torch.index_select(self.embed, 0, self.input_ids, out=self.residual)
        x = None
        for ldx in range(self.n_layers):
            x = self.layer_decode(ldx, x)
        rmsnorm(x, self.final_norm, self.shape.rms_eps, self.normed, residual=self.residual)
        logits = F.linear(self.normed, self.lm_head).float()
        torch.argmax(logits, dim=-1, out=self.next_ids)
        self.input_ids.copy_(self.next_ids)
        self.positions.add_(1)
        return logits

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads (every matrix once; one embedding row per request)."""
        per_layer = sum(t.numel() * t.element_size() for t in self.layers[0].values())
        return per_layer * self.n_layers + self.lm_head.numel() * self.lm_head.element_size()
