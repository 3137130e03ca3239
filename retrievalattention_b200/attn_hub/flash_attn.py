"""Full attention over the dense cache, with the reference's interface (attn_hub/flash_attn.py:4-30): the comparator
of the wave-index path.  Decoding runs this library's split-K flash-decoding kernel (``ri_weighted_flash_decoding``
without weights) over the head-major cache of ``cache_hub.flash_attn_cache``."""
from __future__ import annotations

import torch

from ..kernels import weighted_flash_decoding
from .retroinfer_attn import retroinfer_prefill_attn


def prefill_full_flash_attn(query_states, key_states, value_states, causal):
    """attn_hub/flash_attn.py:4-13 — dense (causal) attention over the prompt."""
    return retroinfer_prefill_attn(query_states, key_states, value_states, causal)


def decode_full_flash_attn(query_states, key_states, value_states, layer_idx, full_attn_cache):
    """attn_hub/flash_attn.py:17-30.  query_states [batch, 1, heads, 128]; key/value_states: the cache tensors
    ``[batch, kv_heads, max_length, 128]`` that ``flash_attn_cache.decode_update_kv_cache`` returned."""
    c = full_attn_cache
    valid = c.valid_length + 1 if layer_idx < c.layer_num - 1 else c.valid_length        # :19
    b, _, hq, d = query_states.shape
    hk, length = key_states.shape[1], key_states.shape[2]
    g, gs = b * hk, hq // hk
    seqlens = valid.to(query_states.device).to(torch.int32).repeat_interleave(hk)
    out = weighted_flash_decoding(query_states.reshape(g, 1, gs, d), key_states.view(g, length, 1, d),
                                  value_states.view(g, length, 1, d), cache_seqlens=seqlens)
    return out.view(b, 1, hq, d)
