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


class PeerGather:
    """The same gather without a collective: every rank's decode kernel stores its head slice straight
    into the gather buffer of every rank of its group (peer-mapped memory over NVLink); ``wait(layer)``
    enqueues, behind that kernel, a small one that writes the step's epoch into this rank's flag word on
    every rank and then waits — with a time limit — until all ranks' flag words of that layer hold it.

    Buffers come from ``torch.distributed._symmetric_memory`` (one allocation per rank, mapped into
    every rank of ``group``).  NVLink multicast is not used (plain peer stores), and it is switched off
    for the allocation so that no rank's memory is bound to a multicast object.

    A rank may overwrite layer l's slice on its peers as soon as their NEXT wait of any layer has passed, so a
    consumer must have read ``view(l)`` before its rank enqueues the wait after next — automatic with two or more
    layers consumed in order; a single-layer model needs two ``PeerGather`` objects used alternately.

    Per step: ``next_step()`` once (advances the epoch), then per layer ``compute(..., gather=self)``
    and ``wait(layer)``.  Layout per rank: ``gathered[layer, shard, B, 1, Hq_local, d]`` and
    ``flags[layer, shard]``; ``view(layer)`` is the ``[B, 1, Hq, d]`` view of a layer.
    """

    def __init__(self, shard: HeadShard, layers: int, batch: int, q_heads_local: int, head_dim: int,
                 dtype: torch.dtype, device: torch.device, group=None, wait_limit_us: int = 0):
        import ctypes as C
        import os

        from . import _lib

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.shard, self.layers = shard, layers
        n = shard.head_shards
        me = shard.head_index
        group = group if group is not None else dist.group.WORLD
        slice_elems = batch * q_heads_local * head_dim
        self.gathered = symm_mem.empty((layers, n, batch, 1, q_heads_local, head_dim), dtype=dtype, device=device)
        self.flags = symm_mem.empty((layers, n), dtype=torch.int32, device=device)
        self.gathered.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        h_out = symm_mem.rendezvous(self.gathered, group)
        h_flag = symm_mem.rendezvous(self.flags, group)
        if h_out.world_size != n or h_out.rank != me:
            raise RuntimeError("PeerGather: the process group does not match the head shards")
        self.epoch = torch.zeros((1,), dtype=torch.int32, device=device)
        self.error = torch.zeros((1,), dtype=torch.int32, device=device)
        # per layer: the wait kernel's timer readings (entry, flags raised, last flag seen) of its latest call
        self.stamps = torch.zeros((layers, 3), dtype=torch.int64, device=device)
        esz = self.gathered.element_size()
        out_slots = torch.tensor([[h_out.buffer_ptrs[p] + (l * n + me) * slice_elems * esz for p in range(n)]
                                  for l in range(layers)], dtype=torch.int64)
        flag_slots = torch.tensor([[h_flag.buffer_ptrs[p] + (l * n + me) * 4 for p in range(n)]
                                   for l in range(layers)], dtype=torch.int64)
        self._out_slots = out_slots.to(device)
        self._flag_slots = flag_slots.to(device)
        self._handles = (h_out, h_flag)          # keep the mappings alive
        self.params = []
        for l in range(layers):
            g = _lib.WaveGather()
            g.n_ranks, g.rank, g.wait_limit_us = n, me, wait_limit_us
            g.d_out_slots = self._out_slots[l].data_ptr()
            g.d_flag_slots = self._flag_slots[l].data_ptr()
            g.d_flags = self.flags[l].data_ptr()
            g.d_epoch = self.epoch.data_ptr()
            g.d_error = self.error.data_ptr()
            g.d_stamps = self.stamps[l].data_ptr()
            self.params.append(g)
        self._C, self._lib = C, _lib
        torch.cuda.synchronize(device)

    def next_step(self) -> None:
        """Advance the epoch (enqueued on the current stream): once per decode step, on every rank."""
        self.epoch.add_(1)

    def wait(self, layer: int) -> None:
        """Enqueue the bounded wait for ``layer``'s slices of this step on the current stream."""
        self._lib.check(self._lib.lib.ri_wave_gather_wait(self._C.byref(self.params[layer]), self._lib.current_stream()),
                        "ri_wave_gather_wait")

    def view(self, layer: int) -> torch.Tensor:
        n, b, one, hl, d = self.gathered.shape[1:]
        return self.gathered[layer].permute(1, 2, 0, 3, 4).reshape(b, one, n * hl, d)

    def wait_times_us(self) -> dict:
        """From the latest wait of every layer: microseconds spent raising the flags (fence + remote stores) and
        waiting for the last rank's flag, as mean and minimum over the layers.  The minimum of the wait is what the
        protocol itself costs (the peer was ready), the rest is waiting for a rank that finished its layer later."""
        st = self.stamps.cpu().double()
        signal = (st[:, 1] - st[:, 0]) / 1e3
        wait = (st[:, 2] - st[:, 1]) / 1e3
        return {"signal_mean": round(float(signal.mean()), 2), "wait_mean": round(float(wait.mean()), 2),
                "wait_min": round(float(wait.min()), 2), "wait_max": round(float(wait.max()), 2)}

    def timed_out(self) -> bool:
        """True when some wait gave up (reads one word from the device)."""
        return bool(self.error.item())
