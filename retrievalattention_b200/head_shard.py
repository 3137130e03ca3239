"""Sharding of the wave-index path over the GPUs of one node: by KV head first, then by batch.

Every (request, kv-head) group is independent through clustering, selection and attention, so a
rank simply builds a ``retroinfer_cache`` for the heads and requests it owns.  The only exchange is
the gather of the per-rank head slices of the attention output before the output projection
(the reference has no multi-GPU mode for this path: its layer-wise placement, model_hub/llama.py:
123-128, moves whole layers, not heads).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    """Which heads and requests a rank owns.  ``world = head_shards * batch_shards``."""

    rank: int
    world: int
    kv_heads: int        # global
    q_heads: int         # global
    batch: int           # global

    def __post_init__(self):
        hs = self.head_shards
        if self.kv_heads % hs or self.world % hs or self.batch % self.batch_shards:
            raise ValueError(f"cannot shard {self.kv_heads} kv heads x batch {self.batch} over {self.world} ranks")

    @property
    def head_shards(self) -> int:
        return min(self.world, self.kv_heads)

    @property
    def batch_shards(self) -> int:
        return self.world // self.head_shards

    @property
    def head_index(self) -> int:
        return self.rank % self.head_shards

    @property
    def batch_index(self) -> int:
        return self.rank // self.head_shards

    @property
    def local_kv_heads(self) -> int:
        return self.kv_heads // self.head_shards

    @property
    def local_q_heads(self) -> int:
        return self.q_heads // self.head_shards

    @property
    def local_batch(self) -> int:
        return self.batch // self.batch_shards

    def kv_head_slice(self) -> slice:
        return slice(self.head_index * self.local_kv_heads, (self.head_index + 1) * self.local_kv_heads)

    def q_head_slice(self) -> slice:
        return slice(self.head_index * self.local_q_heads, (self.head_index + 1) * self.local_q_heads)

    def batch_slice(self) -> slice:
        return slice(self.batch_index * self.local_batch, (self.batch_index + 1) * self.local_batch)

    def head_group_ranks(self) -> list[int]:
        """Ranks that hold the other head slices of the same requests."""
        return [self.batch_index * self.head_shards + h for h in range(self.head_shards)]


class HeadGather:
    """All-gather of ``[B, 1, Hq_local, d]`` slices into ``[B, 1, Hq, d]`` over one process group."""

    def __init__(self, shard: HeadShard, group=None):
        self.shard = shard
        self.group = group
        self._buf = None

    @staticmethod
    def make_groups(shard: HeadShard):
        """One process group per batch shard (collective: every rank must call it).  Returns the
        group this rank belongs to, or None when a single group spans the world."""
        if shard.batch_shards == 1:
            return None
        mine = None
        for b in range(shard.batch_shards):
            ranks = [b * shard.head_shards + h for h in range(shard.head_shards)]
            g = dist.new_group(ranks)
            if b == shard.batch_index:
                mine = g
        return mine

    def __call__(self, out_local: torch.Tensor, gathered: torch.Tensor | None = None) -> torch.Tensor:
        """Returns a ``[B, 1, Hq, d]`` view (head-major inside each request) of the gathered buffer
        ``[shards, B, 1, Hq_local, d]``."""
        s = self.shard
        b, one, hl, d = out_local.shape
        if gathered is None:
            if self._buf is None or self._buf.shape[1:] != out_local.shape or self._buf.dtype != out_local.dtype:
                self._buf = torch.empty((s.head_shards, b, one, hl, d), dtype=out_local.dtype, device=out_local.device)
            gathered = self._buf
        if s.head_shards == 1:
            gathered[0].copy_(out_local)
        else:
            dist.all_gather_into_tensor(gathered.view(-1), out_local.contiguous().view(-1), group=self.group)
        return gathered.permute(1, 2, 0, 3, 4).reshape(b, one, s.head_shards * hl, d)
