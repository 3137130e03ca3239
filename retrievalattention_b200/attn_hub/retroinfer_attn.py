"""The two entry points of the reference's ``attn_hub/retroinfer_attn.py``."""
from __future__ import annotations

import torch

_errors = []        # status words of the prefill calls not yet checked (see ``check_prefill_errors``)


def retroinfer_prefill_attn(query_states, key_states, value_states, causal):
    """Dense prefill attention (attn_hub/retroinfer_attn.py:4-13: ``flash_attn_with_kvcache(q, k_cache, v_cache,
    causal)`` over the whole prompt), on this library's tcgen05 kernel ``ri_prefill_attn``.
    query_states [batch, seq_len, heads, 128]; key/value_states [batch, seq_len, kv_heads, 128].  Asynchronous on the
    current stream; ``check_prefill_errors()`` (which synchronises) raises if a device-side wait ever ran out."""
    from .. import _lib

    b, s, hq, d = query_states.shape
    hk = key_states.shape[2]
    if d != 128 or key_states.shape != (b, s, hk, d) or value_states.shape != key_states.shape or hq % hk:
        raise ValueError("retroinfer_prefill_attn: expected q [B,S,Hq,128] and k, v [B,S,Hk,128] with Hq a multiple of Hk")
    q, k, v = query_states.contiguous(), key_states.contiguous(), value_states.contiguous()
    out = torch.empty_like(q)
    need = _lib.lib.ri_prefill_attn_scratch_bytes(b, s, hk)
    scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    err = torch.zeros((1,), dtype=torch.int32, device=q.device)
    _lib.check(_lib.lib.ri_prefill_attn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                        err.data_ptr(), b, s, hq, hk, int(bool(causal)), _lib.dtype_code(q.dtype),
                                        _lib.current_stream()), "ri_prefill_attn")
    _errors.append(err)
    if len(_errors) > 64:
        check_prefill_errors()
    return out


def check_prefill_errors() -> None:
    """Raise if any prefill call since the last check gave up on a device-side wait (synchronises)."""
    bad = [int(e.item()) for e in _errors]
    _errors.clear()
    if any(bad):
        raise RuntimeError(f"ri_prefill_attn gave up on a device-side wait (codes {sorted(set(x for x in bad if x))})")


def retroinfer_decode_attn(query_states, key_states, value_states, layer_idx, retroinfer_cache, query_states_next=None):
    """attn_hub/retroinfer_attn.py:17-24 — decode attention is the cache's ``compute``."""
    return retroinfer_cache.compute(
        query_states.contiguous(), layer_idx,
        query_states_next.contiguous() if query_states_next is not None else None)
