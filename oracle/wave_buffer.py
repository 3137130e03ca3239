"""CPU restatement of the reference's host-side wave buffer (per-group LRU page
cache).  TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp:
``ClusterDescriptor`` :38-45, ``BufferManager::batch_access`` :190-257,
``BufferManager::batch_update`` :102-188, ``parse_clusters`` :513-542.

The reference hands out free GPU page ids from an ``unordered_set`` (:153-172), so
the ids themselves are arbitrary; this restatement hands out the lowest free id.
Tests compare everything except the concrete page ids, which are checked for
consistency instead (a cluster hits on exactly the pages it was admitted to; live
clusters never share a page).
"""
from __future__ import annotations

from collections import OrderedDict


class GroupBuffer:
    """One (batch, kv-head) group's LRU state."""

    def __init__(self, capacity: int, page_size: int, max_pages: int, sizes):
        self.capacity = capacity
        self.page_size = page_size
        self.max_pages = max_pages
        self.free = set(range(capacity))
        self.lru: OrderedDict[int, None] = OrderedDict()   # first = most recent
        self.in_cache: dict[int, list[int]] = {}
        self.set_clusters(sizes)
        self._miss: list[int] = []
        self._hit: list[int] = []

    def set_clusters(self, sizes, base_start: int = 0, first_id: int = 0):
        """parse_clusters: start = exclusive prefix sum, pages = ceil(size/page),
        last page holds ``size % page`` rows or a full page (:523-540)."""
        if first_id == 0:
            self.start, self.pages, self.last = [], [], []
        total = base_start
        for s in [int(x) for x in sizes]:
            self.start.append(total)
            self.pages.append((s + self.page_size - 1) // self.page_size)
            self.last.append(self.page_size if s % self.page_size == 0 else s % self.page_size)
            total += s
        return total

    def access(self, keys):
        """batch_access.  Returns dict of hit/miss page lists."""
        hit_ids, hit_sizes, hit_cum = [], [], []
        miss_ids, miss_sizes, miss_cum = [], [], []
        self._miss, self._hit = [], []
        h = m = 0
        considered = 0
        overflow = False
        for key in [int(k) for k in keys]:
            considered += self.pages[key]
            if considered > self.max_pages:
                overflow = True
                break
            n = self.pages[key]
            # An empty cluster has BlockNum 0, for which the reference writes GPUBlockIDs[-1]
            # (:167) — undefined.  Selection ranks empty clusters last, so none is ever accessed.
            assert n > 0, "empty cluster accessed"
            if key not in self.in_cache:
                self._miss.append(key)
                start = self.start[key]
                for j in range(n - 1):
                    miss_ids.append(start); miss_sizes.append(self.page_size); miss_cum.append(m)
                    m += self.page_size; start += self.page_size
                miss_ids.append(start); miss_sizes.append(self.last[key]); miss_cum.append(m)
                m += self.last[key]
            else:
                self._hit.append(key)
                pages = self.in_cache[key]
                hit_ids.extend(pages[:n])
                for j in range(n - 1):
                    hit_sizes.append(self.page_size); hit_cum.append(h); h += self.page_size
                hit_sizes.append(self.last[key]); hit_cum.append(h); h += self.last[key]
        return {"hit_ids": hit_ids, "hit_sizes": hit_sizes, "hit_cumsum": hit_cum,
                "miss_ids": miss_ids, "miss_sizes": miss_sizes, "miss_cumsum": miss_cum,
                "hit_keys": list(self._hit), "miss_keys": list(self._miss), "overflow": overflow}

    def update(self):
        """batch_update.  Returns (cache page ids, sizes, buffer offsets) per page."""
        for key in reversed(self._hit):
            self.lru.move_to_end(key, last=False)
        admit, need = 0, 0
        for key in self._miss:
            if need + self.pages[key] <= self.capacity:
                admit += 1
                need += self.pages[key]
            else:
                break
        ids, sizes, offs = [], [], []
        if admit:
            while len(self.free) < need:
                victim, _ = self.lru.popitem(last=True)
                self.free.update(self.in_cache.pop(victim))
            cum = 0
            for key in self._miss[:admit]:
                n = self.pages[key]
                got = []
                for j in range(n):
                    pid = min(self.free)
                    self.free.remove(pid)
                    got.append(pid)
                    sz = self.page_size if j < n - 1 else self.last[key]
                    ids.append(pid); sizes.append(sz); offs.append(cum)
                    cum += sz
                self.in_cache[key] = got
                self.lru[key] = None
                self.lru.move_to_end(key, last=False)
        self._miss, self._hit = [], []
        return {"cache_ids": ids, "sizes": sizes, "buffer_offsets": offs, "admitted": admit}
