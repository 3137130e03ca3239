from .flash_attn import decode_full_flash_attn, prefill_full_flash_attn  # noqa: F401
from .retroinfer_attn import retroinfer_decode_attn, retroinfer_prefill_attn  # noqa: F401
