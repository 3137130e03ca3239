"""Base class holding the cache geometry (cache_hub/cache.py:4-59 of the reference)."""
from __future__ import annotations

import torch


class KV_Cache:
    def __init__(self, layer_num: int, batch_size: int, max_length: int, num_key_value_heads: int, num_heads: int,
                 head_dim: int, dtype: torch.dtype, layer_mapping: dict, num_gpus: int, model_size: int) -> None:
        self.layer_num = layer_num
        self.batch_size = batch_size
        self.max_length = max_length
        self.kv_head = num_key_value_heads
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.dtype = dtype
        self.layer_mapping = layer_mapping
        self.context = 0
        self.num_gpus = num_gpus
        self.model_size = model_size
        # free-memory estimate during prefill, GB (cache_hub/cache.py:47-58)
        gib = 1024 ** 3
        total = num_gpus * torch.cuda.get_device_properties(0).total_memory / gib
        per_token = num_heads * max_length * head_dim * 2 / gib
        prefill = per_token * 2 + (num_heads + 2 * num_key_value_heads) * max_length * head_dim * 2 / gib + 4 * per_token
        self.free_memory = total - model_size * 2 - prefill * num_gpus
