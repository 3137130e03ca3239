"""The two entry points of the reference's ``attn_hub/retroinfer_attn.py``."""
from __future__ import annotations


def retroinfer_prefill_attn(query_states, key_states, value_states, causal):
    """Dense prefill attention (attn_hub/retroinfer_attn.py:4-13).  Prefill is outside the decode
    hot path; like the reference this delegates to the flash-attn library kernel."""
    from flash_attn import flash_attn_with_kvcache

    return flash_attn_with_kvcache(q=query_states, k_cache=key_states, v_cache=value_states, causal=causal)


def retroinfer_decode_attn(query_states, key_states, value_states, layer_idx, retroinfer_cache, query_states_next=None):
    """attn_hub/retroinfer_attn.py:17-24 — decode attention is the cache's ``compute``."""
    return retroinfer_cache.compute(
        query_states.contiguous(), layer_idx,
        query_states_next.contiguous() if query_states_next is not None else None)
