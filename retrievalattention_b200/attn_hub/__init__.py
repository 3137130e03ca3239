from .retroinfer_attn import retroinfer_decode_attn, retroinfer_prefill_attn  # noqa: F401
