"""Dense KV cache with the reference's ``flash_attn_cache`` interface (cache_hub/flash_attn_cache.py:5-151): the
full-attention comparator of the wave index.

Same constructor, ``prefill_update_kv_cache`` / ``sync`` / ``decode_update_kv_cache`` / ``move_gpu`` and attributes
(``key_cache``, ``value_cache``, ``valid_length``, ``context``).  The cache is always resident on the layer's GPU (the
reference falls back to pinned host memory during prefill when HBM is short, :54-76), and it is kept head-major,
``[batch, kv_heads, max_length, head_dim]``, which is the layout this library's decode kernel streams; the tensors
``decode_update_kv_cache`` returns are meant for ``attn_hub.decode_full_flash_attn`` of this package only.
"""
from __future__ import annotations

import numpy as np
import torch

from .cache import KV_Cache


class flash_attn_cache(KV_Cache):
    def __init__(self, valid_start, layer_num: int, batch_size: int, max_length: int, num_key_value_heads: int,
                 num_heads: int, head_dim: int, dtype: torch.dtype, layer_mapping: dict, num_gpus: int,
                 model_size: int) -> None:
        super().__init__(layer_num, batch_size, max_length, num_key_value_heads, num_heads, head_dim, dtype,
                         layer_mapping, num_gpus, model_size)
        if head_dim != 128:
            raise ValueError("the decode kernel is built for head_dim 128")
        self.valid_start = valid_start
        self.valid_length = None            # [batch] int32 on the first layer's device, set by the first prefill call
        self.allocated = True
        mk = lambda ldx: torch.zeros((batch_size, self.kv_head, max_length, head_dim), dtype=dtype,   # noqa: E731
                                     device=layer_mapping[str(ldx)])
        self.key_cache = [mk(ldx) for ldx in range(layer_num)]
        self.value_cache = [mk(ldx) for ldx in range(layer_num)]
        self._rows = torch.arange(batch_size, device=layer_mapping[str(0)])

    def move_gpu(self):
        """The reference moves a host-resident cache to the GPUs here (:85-89); this one is already there."""
        return None

    def prefill_update_kv_cache(self, query_states, key_states, value_states, layer_idx, start_bdx):
        """One request, one layer (:92-127).  key/value_states: [1, seq_len, kv_heads, head_dim]."""
        bsz, seq_len, _, _ = key_states.shape
        assert bsz == 1, "Multi-batch prefilling only support prefill single batch one by one."
        assert seq_len <= self.max_length, f"Prefilling sequence length {seq_len} exceeds max length {self.max_length}."
        if self.valid_length is None:
            vs = np.asarray(self.valid_start)
            self.valid_length = torch.from_numpy(seq_len - vs).to(torch.int32).to(self.layer_mapping[str(0)])
        vs = int(self.valid_start[start_bdx])
        n = seq_len - vs
        self.key_cache[layer_idx][start_bdx, :, :n].copy_(key_states[0, vs:].transpose(0, 1))
        self.value_cache[layer_idx][start_bdx, :, :n].copy_(value_states[0, vs:].transpose(0, 1))
        if layer_idx == self.layer_num - 1 and start_bdx + bsz == self.batch_size:
            self.context += seq_len
        return key_states[:, vs:], value_states[:, vs:]

    def sync(self, layer_idx, start_bdx):
        """The reference waits for its side-stream copy (:129-130); the copy above is in stream order."""
        return None

    def decode_update_kv_cache(self, key_states, value_states, layer_idx):
        """Append one token per request (:133-151).  key/value_states: [batch, 1, kv_heads, head_dim]."""
        pos = self.valid_length.to(self.key_cache[layer_idx].device).long()
        self.key_cache[layer_idx][self._rows.to(pos.device), :, pos] = key_states[:, 0]
        self.value_cache[layer_idx][self._rows.to(pos.device), :, pos] = value_states[:, 0]
        if layer_idx == self.layer_num - 1:
            self.context += 1
            self.valid_length += 1
        return self.key_cache[layer_idx], self.value_cache[layer_idx]
