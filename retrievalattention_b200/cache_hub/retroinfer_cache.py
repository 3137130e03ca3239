"""``retroinfer_cache`` with the reference's interface (cache_hub/retroinfer_cache.py:16-697), backed
by the CUDA kernels of this package and with the whole cluster-contiguous KV resident in HBM.

What is the same: constructor arguments, ``prefill_update_kv_cache`` / ``sync`` / ``prepare_cache`` /
``decode_update_kv_cache`` / ``compute`` and their return values, the attributes callers read
(``context``, ``layer_num``), the steady-zone bookkeeping (``static_pattern_total``), the index
parameters and the page budget ``buffer_size`` (:107-111).

What differs underneath: the index is built on the GPU by ``ri_kmeans_build`` (no pinned-host
offload, no CPU re-layout).  Two storage tiers:

* default (``kv_on_host=False``): the whole cluster-contiguous KV stays in HBM and one decode layer is
  one ``ri_wave_decode_layer`` call with no host synchronisation.  ``core`` and ``cache_cluster_num``
  are accepted but unused — nothing lives on the host, so there is no page cache to size.
* ``kv_on_host=True`` (not a reference argument): the reference's tiers — cluster-contiguous KV
  in pinned host memory (:264-274), an LRU page cache of ``cache_cluster_num`` clusters on the GPU
  (:204-211), a host-side wave buffer per layer (:117-121) and an execution buffer assembled per step
  (:642-648).  Three ways to bring the missed pages up (``miss_path``):

  - ``"pull"`` (default): the select stage writes the retrieved ids straight into pinned host memory and the host
    waits on an event (instead of the blocking copy of :575); while the host walks the LRU lists the GPU already
    attends the estimation zone and the steady zone; then ``gather_copy_and_concat`` runs on a SIDE stream and
    reads the missed pages from the pinned store itself (over PCIe) into one of two execution buffers, hit pages
    behind them; behind that kernel's event the second attention pass covers the pages and merges with the
    first by log-sum-exp; ``gather_copy_and_scatter`` admits the missed pages into the GPU cache (:682-690).
    With ``use_cluster_estimation=True`` the search, the list walk and the pull of layer l+1 are started inside
    layer l's call with ``queries_next``, so a layer's pages cross PCIe under the previous layer's work.
  - ``"staged"``: the host's worker threads copy the missed pages into a pinned staging area and one strided
    ``cudaMemcpy2DAsync`` per tensor sends them up on the side stream (measured slower: a second pass over
    the bytes on the host).
  - ``"uva"``: the reference's own pattern — blocking id copy, one copy kernel on the main stream, one
    attention pass, three host waits.

After every 1024 generated tokens ``decode_update_kv_cache`` folds them into the index (``_update_kv_cache``,
:462-524), provided ``max_new_length`` announced that many at construction.

``use_cluster_estimation=True``: ``compute(queries, l, queries_next)`` also searches layer ``l + 1``'s
clusters with ``queries_next`` (the caller's estimate of the next layer's query, model_hub/LLM.py:102-107), and a
layer whose clusters were searched ahead in this step attends those clusters with its real query instead of
searching again (:565, :582-595).  Layers without a search made for them (the first ones, or whenever the caller
passes no ``queries_next``) search with their own query — the reference instead reuses whatever an earlier step
left in its index buffer for layer 2, an off-by-one that is not reproduced.  The point of the feature in the
reference is to start the host wave buffer's work one layer early, which is what the host tier's ``"pull"`` path
does with it; with the cluster store in HBM there is nothing to hide, so there the mode exists for its results
(it is slower than the single kernel: five launches per layer).
"""
from __future__ import annotations

import math

import torch

from .. import wave
from .cache import KV_Cache
from .kmeans import build_index

THRESHOLD_LENGTH = 1024   # reference: re-index period in generated tokens (:13)


class retroinfer_cache(KV_Cache):
    def __init__(self, valid_start, layer_num: int, batch_size: int, max_length: int, num_key_value_heads: int,
                 num_heads: int, head_dim: int, dtype: torch.dtype, layer_mapping: dict, max_new_length: int,
                 static_pattern_start: int, static_pattern_end: int, core: int, n_centroids: int, n_segment: int,
                 nprobe: int, max_compute_cluster_num: int, cache_unit_size: int, cache_cluster_num: int,
                 num_gpus: int, model_size: int, use_cluster_estimation: bool = False,
                 kv_on_host: bool = False, fuse_append: bool = True, miss_path: str = "pull") -> None:
        super().__init__(layer_num, batch_size, max_length, num_key_value_heads, num_heads, head_dim, dtype,
                         layer_mapping, num_gpus, model_size)
        if head_dim != 128:
            raise ValueError("the wave-index kernels are built for head_dim 128 (as the reference's copy kernels are)")
        self.valid_start = valid_start
        # fuse_append (not in the reference): decode_update_kv_cache only hands the new rows to the layer and the
        # decode kernel of the following compute() stores them into the steady zone itself (one launch less per
        # layer).  The two calls always come in pairs (attn_hub.retroinfer_decode_attn); the rows passed must stay
        # unchanged until that compute().  HBM tier only.
        self.fuse_append = bool(fuse_append) and not kv_on_host and not use_cluster_estimation
        self.static_pattern_start = static_pattern_start
        self.static_pattern_end = static_pattern_end
        self.static_pattern_total = static_pattern_start + static_pattern_end
        self.group_size = num_heads // num_key_value_heads
        self.batch_groups = batch_size * num_key_value_heads
        self.page_size = cache_unit_size
        self.core = core
        self.use_cluster_estimation = use_cluster_estimation

        self.input_length = max_length - max_new_length
        self.max_new_length = min(max_new_length - 1, THRESHOLD_LENGTH)       # :64
        # re-indexing of generated tokens (:66-69): every THRESHOLD_LENGTH of them become 64 more clusters
        self.input_length_new = max(0, (max_new_length - 2) // THRESHOLD_LENGTH) * THRESHOLD_LENGTH
        self.n_centroids_per_update_segment = ((THRESHOLD_LENGTH // 16) // 32) * 32
        self.n_centroids_new = max(0, (max_new_length - 2) // THRESHOLD_LENGTH) * self.n_centroids_per_update_segment
        self.static_stride = self.static_pattern_total + self.max_new_length
        self.n_centroids = n_centroids
        self.n_segment = n_segment
        self.nprobe = nprobe
        self.max_compute_cluster_num = max_compute_cluster_num
        self.es_cluster_num = max_compute_cluster_num - nprobe
        avg_cluster_size = (self.input_length - self.static_pattern_total) // n_centroids
        pages_per_cluster = math.ceil(avg_cluster_size / self.page_size)
        self.cache_size = cache_cluster_num * pages_per_cluster
        self.buffer_size = max(int(nprobe * 4), 16) * pages_per_cluster      # :111, page budget per group
        # rows of the cluster store per group: the prompt's clustered tokens, then room for the re-indexed ones (:264-274)
        self.list_stride = self.input_length - self.static_pattern_total + self.input_length_new

        self.kv_on_host = bool(kv_on_host)
        if miss_path not in ("pull", "staged", "uva"):
            raise ValueError(f"miss_path must be 'pull', 'staged' or 'uva', got {miss_path!r}")
        self.miss_path = miss_path if self.kv_on_host else None
        self.stage_misses = self.miss_path == "staged"
        g, c, d = self.batch_groups, n_centroids, head_dim
        self.steady_zone_keys, self.steady_zone_values = [], []
        self.centroids, self.value_sum, self.cluster_size = [], [], []
        self.cluster_count, self.cluster_offset, self.centroids_mask = [], [], []
        self.list_keys, self.list_values = [], []
        self._error_flags = []
        for ldx in range(layer_num):
            dev = layer_mapping[str(ldx)]
            z = lambda *shape, dt=dtype: torch.zeros(shape, dtype=dt, device=dev)  # noqa: E731
            self.steady_zone_keys.append(z(batch_size, self.kv_head, self.static_stride, d))
            self.steady_zone_values.append(z(batch_size, self.kv_head, self.static_stride, d))
            self.centroids.append(z(g, c, d))
            self.value_sum.append(z(g, c, d))
            self.cluster_size.append(z(g, c))
            self.cluster_count.append(z(g, c, dt=torch.int32))
            self.cluster_offset.append(z(g, c + 1, dt=torch.int32))
            self.centroids_mask.append(z(g, c, dt=torch.bool))
            if not self.kv_on_host:
                self.list_keys.append(z(batch_size, self.kv_head, self.list_stride, d))
                self.list_values.append(z(batch_size, self.kv_head, self.list_stride, d))
            else:
                host = lambda: torch.zeros((batch_size, self.kv_head, self.list_stride, d), dtype=dtype,  # noqa: E731
                                           pin_memory=True)
                self.list_keys.append(host())
                self.list_values.append(host())

        self.shape = wave.WaveShape(g, self.group_size, c, nprobe, self.es_cluster_num, self.page_size,
                                    self.buffer_size, self.list_stride, self.static_stride, dtype)
        self.reindex_count = 0
        # per device: scratch shared by the layers of that device, and the device-side counters
        self._per_device = {}
        for dev in sorted(set(layer_mapping.values())):
            self._per_device[dev] = {
                "scratch": wave.new_scratch(self.shape, dev),
                "static_len": torch.tensor([self.static_pattern_total + 1], dtype=torch.int32, device=dev),
                "append_pos": torch.tensor([self.static_pattern_total], dtype=torch.int32, device=dev),
            }
        self._layers = [None] * layer_num
        # use_cluster_estimation: a search made one layer ahead lives in the layer's own scratch until it is used
        self._ahead = [False] * layer_num
        if self.use_cluster_estimation:
            if kv_on_host and miss_path != "pull":
                raise NotImplementedError("on the host tier use_cluster_estimation needs miss_path='pull'")
            for dev in self._per_device:
                self._per_device[dev]["layer_scratch"] = {}
        if self.kv_on_host:
            self._init_host_tier(cache_cluster_num)

    def _init_host_tier(self, cache_cluster_num):
        """GPU page cache, execution buffers, pinned page lists and the host wave buffers
        (cache_hub/retroinfer_cache.py:117-193, :204-211, :302-316)."""
        from ..kernels import ThreadPool, WaveBufferCPU

        g, d = self.batch_groups, self.head_dim
        if self.page_size != 8:
            raise ValueError("the host tier's copy kernels move pages of 8 rows (as the reference's, gather_copy.cu:11): "
                             f"cache_unit_size must be 8, got {self.page_size}")
        self.cache_size = max(self.cache_size, 1)
        self.execution_stride = self.buffer_size * self.page_size + self.static_stride
        self.thread_pool = ThreadPool(self.core)
        self.cache_keys, self.cache_values, self.wave_buffer = [], [], []
        self.page_lists, self.cluster_ids = [], []
        i32 = lambda *shape: torch.zeros(shape, dtype=torch.int32, pin_memory=True)  # noqa: E731
        for ldx in range(self.layer_num):
            dev = self.layer_mapping[str(ldx)]
            self.cache_keys.append(torch.zeros((g, self.cache_size, self.page_size, d), dtype=self.dtype, device=dev))
            self.cache_values.append(torch.zeros((g, self.cache_size, self.page_size, d), dtype=self.dtype, device=dev))
            wb = WaveBufferCPU(self.batch_size, self.kv_head, d, self.nprobe, self.page_size, self.n_centroids,
                               self.n_centroids + self.n_centroids_new, self.buffer_size, self.cache_size, self.core,
                               self.thread_pool.get())
            b = self.buffer_size
            lists = [i32(g, b), i32(g, b), i32(g, b), i32(g), i32(g, b), i32(g, b), i32(g, b), i32(g),
                     i32(g, b), i32(g, b), i32(g, b), i32(g)]
            ids = torch.zeros((g, self.nprobe), dtype=torch.int64, pin_memory=True)
            wb.set_indices(*lists, ids)
            self.wave_buffer.append(wb)
            self.page_lists.append(lists)
            self.cluster_ids.append(ids)
        for dev, per in self._per_device.items():
            per["exec_keys"] = torch.zeros((g, self.execution_stride, d), dtype=self.dtype, device=dev)
            per["exec_values"] = torch.zeros((g, self.execution_stride, d), dtype=self.dtype, device=dev)
            per["valid_lengths"] = torch.zeros((g,), dtype=torch.int32, device=dev)
            if self.miss_path in ("pull", "staged"):
                per["copy_stream"] = torch.cuda.Stream(device=dev)
                per["lse"] = torch.zeros((g, self.group_size), dtype=torch.float32, device=dev)
                per["part"] = torch.zeros((g, self.group_size, d), dtype=self.dtype, device=dev)
                per["steady_lengths"] = torch.zeros((g,), dtype=torch.int32, device=dev)
            if self.miss_path == "pull":
                # two execution buffers used by even and odd layers (a layer's pages may arrive while the layer
                # before it still reads its own), each with its page-row counts and two events
                per["exec"] = [(per["exec_keys"], per["exec_values"]),
                               (torch.zeros_like(per["exec_keys"]), torch.zeros_like(per["exec_values"]))]
                per["rest_lengths"] = [torch.zeros((g,), dtype=torch.int32, device=dev) for _ in range(2)]
                per["selected"] = [torch.cuda.Event() for _ in range(2)]
                per["pulled"] = [torch.cuda.Event() for _ in range(2)]
            if self.stage_misses:
                # two staging areas used alternately (the host refills one while the other's copy may still be running),
                # on the host (pinned) and on the device; one side stream and one event per area
                rows = self.buffer_size * self.page_size
                per["stage_rows"] = rows
                per["stage_host"] = [tuple(torch.zeros((g, rows, d), dtype=self.dtype, pin_memory=True) for _ in range(2))
                                     for _ in range(2)]
                per["stage_dev"] = [tuple(torch.zeros((g, rows, d), dtype=self.dtype, device=dev) for _ in range(2))
                                    for _ in range(2)]
                per["uploaded"] = [torch.cuda.Event() for _ in range(2)]
                per["selected"] = torch.cuda.Event()
                per["rest_lengths"] = torch.zeros((g,), dtype=torch.int32, device=dev)
                per["turn"] = 0
        self._keep_alive = []

    # ------------------------------------------------------------------ prefill
    def prefill_update_kv_cache(self, query_states, key_states, value_states, layer_idx, batch_idx):
        """One request, one layer (:368-441).  key/value_states: [1, seq_len, kv_heads, head_dim]."""
        bsz, seq_len, group_num, head_dim = key_states.shape
        assert bsz == 1, "Multi-batch prefilling only support prefill single batch one by one."
        assert seq_len <= self.input_length, f"seq_len({seq_len}) should less than input_length({self.input_length})"
        vs = int(self.valid_start[batch_idx])
        start, end, total = self.static_pattern_start, self.static_pattern_end, self.static_pattern_start + self.static_pattern_end
        valid_length = seq_len - total - vs

        temp_keys = key_states[0, vs + start:seq_len - end].transpose(0, 1).contiguous()      # [kv_heads, N_b, d]
        temp_values = value_states[0, vs + start:seq_len - end].transpose(0, 1).contiguous()

        sk, sv = self.steady_zone_keys[layer_idx], self.steady_zone_values[layer_idx]
        sk[batch_idx, :, :start] = key_states[0, vs:vs + start].transpose(0, 1)
        sk[batch_idx, :, start:total] = key_states[0, seq_len - end:seq_len].transpose(0, 1)
        sv[batch_idx, :, :start] = value_states[0, vs:vs + start].transpose(0, 1)
        sv[batch_idx, :, start:total] = value_states[0, seq_len - end:seq_len].transpose(0, 1)

        r = build_index(temp_keys, temp_values, self.n_centroids, self.n_segment)
        rows = slice(batch_idx * self.kv_head, (batch_idx + 1) * self.kv_head)
        self.centroids[layer_idx][rows].copy_(r["centroids"])
        self.value_sum[layer_idx][rows].copy_(r["value_sum"])
        self.cluster_size[layer_idx][rows].copy_(r["cluster_size"])
        self.cluster_count[layer_idx][rows].copy_(r["cluster_count"])
        self.cluster_offset[layer_idx][rows].copy_(r["cluster_offset"])
        self.centroids_mask[layer_idx][rows].copy_(r["cluster_count"] == 0)
        self._error_flags.append(r["error"])
        if self.kv_on_host:
            # the offload of this request-layer's laid-out rows runs on a side stream, under the clustering of the next
            # request-layer (the reference's offload <-> k-means overlap, :388-403); at most two laid-out copies are
            # kept on the device
            dev = key_states.device
            per = self._per_device[self.layer_mapping[str(layer_idx)]]
            if "offload_stream" not in per:
                per["offload_stream"] = torch.cuda.Stream(device=dev)
            off, done = per["offload_stream"], torch.cuda.Event()
            off.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(off):
                for h in range(self.kv_head):      # one contiguous run per head: a plain asynchronous copy each
                    self.list_keys[layer_idx][batch_idx, h, :valid_length].copy_(r["keys"][h], non_blocking=True)
                    self.list_values[layer_idx][batch_idx, h, :valid_length].copy_(r["values"][h], non_blocking=True)
                done.record(off)
            self._keep_alive.append((done, r))
            while len(self._keep_alive) > 2:
                self._keep_alive.pop(0)[0].synchronize()
            self.wave_buffer[layer_idx].async_construction(None, r["cluster_count"], batch_idx)
        else:
            self.list_keys[layer_idx][batch_idx, :, :valid_length].copy_(r["keys"])
            self.list_values[layer_idx][batch_idx, :, :valid_length].copy_(r["values"])

        if layer_idx == self.layer_num - 1 and batch_idx + bsz == self.batch_size:
            self.context += seq_len
        return key_states[:, vs:], value_states[:, vs:]

    def sync(self, layer_idx, batch_idx):
        """The reference waits here for its host offload and starts the CPU re-layout (:443-458).  The layout was
        already written by the clustering pass; the host tier's offload copies keep running on their side stream and
        ``prepare_cache`` waits for the last of them."""
        return None

    def prepare_cache(self):
        """Finish prefill (:336-365): check the clustering status words and bind every layer."""
        torch.cuda.synchronize()
        for flag in self._error_flags:
            if int(flag.item()) != 0:
                raise RuntimeError(f"clustering gave up on a device-side wait (code {int(flag.item())})")
        self._error_flags.clear()
        if self.kv_on_host:
            self._keep_alive.clear()
        g = self.batch_groups
        for ldx in range(self.layer_num):
            per = self._per_device[self.layer_mapping[str(ldx)]]
            if self.kv_on_host:
                shape = wave.WaveShape(g, self.group_size, self.n_centroids, self.nprobe, self.es_cluster_num,
                                       self.page_size, self.buffer_size, self.execution_stride, self.static_stride,
                                       self.dtype)
                store_k, store_v = per["exec_keys"], per["exec_values"]
            else:
                shape = self.shape
                store_k = self.list_keys[ldx].view(g, self.list_stride, self.head_dim)
                store_v = self.list_values[ldx].view(g, self.list_stride, self.head_dim)
            self._layers[ldx] = wave.WaveIndexLayer(
                shape, centroids=self.centroids[ldx], value_sum=self.value_sum[ldx],
                cluster_size=self.cluster_size[ldx], cluster_count=self.cluster_count[ldx],
                cluster_offset=self.cluster_offset[ldx], keys=store_k, values=store_v,
                want_ids=self.kv_on_host, host_tier=self.kv_on_host,
                steady_keys=self.steady_zone_keys[ldx].view(g, self.static_stride, self.head_dim),
                steady_values=self.steady_zone_values[ldx].view(g, self.static_stride, self.head_dim),
                static_len=per["static_len"], scratch=self._scratch_for(ldx, per))
            if self.miss_path in ("pull", "staged"):
                # the select stage stores the ranked ids straight into the pinned array the host wave buffer reads
                self._layers[ldx].retrieved_ids = self.cluster_ids[ldx]
                self._layers[ldx].params.d_retrieved_ids = self.cluster_ids[ldx].data_ptr()

    def _scratch_for(self, ldx, per):
        """One scratch per device; with ``use_cluster_estimation`` one per layer (a search made ahead must survive
        the other layers' work)."""
        if not self.use_cluster_estimation:
            return per["scratch"]
        need = self.shape.scratch_bytes()
        old = per["layer_scratch"].get(ldx)
        if old is None or old.numel() < need:
            per["layer_scratch"][ldx] = wave.new_scratch(self.shape, per["static_len"].device)
        return per["layer_scratch"][ldx]

    # ------------------------------------------------------------------ re-index
    def _update_kv_cache(self):
        """Fold the THRESHOLD_LENGTH oldest tokens of the steady zone's tail into the wave index (:462-524):
        cluster them per group into ``n_centroids_per_update_segment`` more clusters (one segment, keys
        centred on their own mean), append centroids / value sums / sizes to the meta index and the
        members, cluster-contiguous, to the cluster store, then move the last ``static_pattern_end`` rows
        down behind the sink tokens.  The clustering and the re-layout run on the device (the reference offloads
        the rows to the host and re-lays them out there); on the host tier the laid-out members are then copied
        into the pinned cluster store.  Tensors of the meta index are replaced by longer ones, so a
        CUDA graph captured before this call no longer describes the cache and has to be captured again."""
        if (self.reindex_count + 1) * THRESHOLD_LENGTH > self.input_length_new:
            raise RuntimeError("the cluster store has no room left for re-indexed tokens (max_new_length too small)")
        start, end, total = self.static_pattern_start, self.static_pattern_end, self.static_pattern_total
        g, d, extra = self.batch_groups, self.head_dim, self.n_centroids_per_update_segment
        for ldx in range(self.layer_num):
            dev = self.layer_mapping[str(ldx)]
            with torch.cuda.device(dev):
                sk, sv = self.steady_zone_keys[ldx], self.steady_zone_values[ldx]
                # copies, not views (:465-466): with one group the slice is already contiguous and the window move
                # below would overwrite its first rows before the clustering reads them
                update_keys = sk[:, :, start:total - end].reshape(g, THRESHOLD_LENGTH, d).clone()
                update_values = sv[:, :, start:total - end].reshape(g, THRESHOLD_LENGTH, d).clone()
                tail_k, tail_v = sk[:, :, total - end:total].clone(), sv[:, :, total - end:total].clone()
                sk[:, :, start:start + end] = tail_k        # move the local window (:469-472)
                sv[:, :, start:start + end] = tail_v
                r = build_index(update_keys, update_values, extra, 1)
                self._error_flags.append(r["error"])
                old_off = self.cluster_offset[ldx]
                first = old_off[:, -1:].long()               # rows already used by each group
                self.centroids[ldx] = torch.cat((self.centroids[ldx], r["centroids"]), dim=1)
                self.value_sum[ldx] = torch.cat((self.value_sum[ldx], r["value_sum"]), dim=1)
                self.cluster_size[ldx] = torch.cat((self.cluster_size[ldx], r["cluster_size"]), dim=1)
                self.cluster_count[ldx] = torch.cat((self.cluster_count[ldx], r["cluster_count"]), dim=1)
                self.centroids_mask[ldx] = torch.cat((self.centroids_mask[ldx], r["cluster_count"] == 0), dim=1)
                self.cluster_offset[ldx] = torch.cat((old_off, (first + r["cluster_offset"][:, 1:].long()).to(torch.int32)),
                                                     dim=1)
                if self.kv_on_host:
                    # cluster store in pinned host memory: the members go behind each group's rows there, and the
                    # host wave buffer learns the new clusters' sizes (wave_buffer_cpu.cpp:635-720 `update_kv`)
                    lk = self.list_keys[ldx].view(g, self.list_stride, d)
                    lv = self.list_values[ldx].view(g, self.list_stride, d)
                    for grp, n0 in enumerate(first.view(-1).tolist()):
                        lk[grp, n0:n0 + THRESHOLD_LENGTH].copy_(r["keys"][grp])
                        lv[grp, n0:n0 + THRESHOLD_LENGTH].copy_(r["values"][grp])
                    self.wave_buffer[ldx].update_kv(None, None, None, r["cluster_count"])
                else:
                    rows = first + torch.arange(THRESHOLD_LENGTH, device=dev)[None, :]
                    pick = torch.arange(g, device=dev)[:, None]
                    self.list_keys[ldx].view(g, self.list_stride, d)[pick, rows] = r["keys"]
                    self.list_values[ldx].view(g, self.list_stride, d)[pick, rows] = r["values"]
        self.n_centroids += extra                            # :509
        self.reindex_count += 1
        self.static_pattern_total = start + end              # :522
        self.shape = wave.WaveShape(g, self.group_size, self.n_centroids, self.nprobe, self.es_cluster_num,
                                    self.page_size, self.buffer_size, self.list_stride, self.static_stride, self.dtype)
        for dev, per in self._per_device.items():
            per["scratch"] = wave.new_scratch(self.shape, dev)
            per["static_len"].fill_(self.static_pattern_total + 1)
            per["append_pos"].fill_(self.static_pattern_total)
        self.prepare_cache()

    # ------------------------------------------------------------------ decode
    def decode_update_kv_cache(self, key_states, value_states, layer_idx):
        """Append the new token's K/V ([bs, 1, kv_heads, d]) to the steady zone (:527-546)."""
        if self.static_pattern_total == self.static_pattern_start + self.static_pattern_end + THRESHOLD_LENGTH:
            self._update_kv_cache()
        per = self._per_device[self.layer_mapping[str(layer_idx)]]
        g = self.batch_groups
        if self.fuse_append:
            self._layers[layer_idx].append_with_next_compute(key_states.contiguous(), value_states.contiguous())
        else:
            wave.steady_append(key_states.contiguous(), value_states.contiguous(),
                               self.steady_zone_keys[layer_idx].view(g, self.static_stride, self.head_dim),
                               self.steady_zone_values[layer_idx].view(g, self.static_stride, self.head_dim),
                               per["append_pos"])
        if layer_idx == self.layer_num - 1:
            self.context += 1
            self.static_pattern_total += 1
            for p in self._per_device.values():
                p["append_pos"].add_(1)
        return None, None

    def compute(self, queries, layer_idx, queries_next=None, out=None, gather=None):
        """Wave-index attention for one layer (:549-697).  queries: [batch, 1, heads, d].
        ``out`` (optional, not in the reference) receives the result instead of a new tensor.
        ``gather`` (optional, several GPUs): a ``head_shard.PeerGather``; the decode kernel then also
        stores this rank's head slice into every rank's gather buffer (no collective afterwards)."""
        if self.kv_on_host:
            if gather is not None:
                raise NotImplementedError("the peer-store gather is built for the HBM tier only")
            if self.miss_path == "pull":
                out = self._compute_host_tier_pull(queries.contiguous(), layer_idx, queries_next, out)
            else:
                out = self._compute_host_tier(queries.contiguous(), layer_idx, out)
        elif self.use_cluster_estimation:
            if gather is not None:
                raise NotImplementedError("the peer-store gather is not combined with use_cluster_estimation")
            out = self._compute_with_estimation(queries.contiguous(), layer_idx, queries_next, out)
        else:
            out = self._layers[layer_idx].compute(queries.contiguous(), out,
                                                  gather=None if gather is None else gather.params[layer_idx])
        if layer_idx == self.layer_num - 1:
            # every layer of a step attends static_pattern_total(+1) rows (:559); advance for the next step
            for p in self._per_device.values():
                p["static_len"].add_(1)
        return out.view(self.batch_size, 1, self.num_heads, self.head_dim)

    def _compute_with_estimation(self, queries, layer_idx, queries_next, out):
        """``use_cluster_estimation`` (:565, :582-595): attend the clusters searched one layer ahead if there are
        any, else search now; then search the next layer's clusters with ``queries_next``."""
        layer = self._layers[layer_idx]
        if out is None:
            out = torch.empty_like(queries)
        if self._ahead[layer_idx]:
            self._ahead[layer_idx] = False
            layer.stage("rescore", queries, out)      # the estimation entries' scores for the real query
            layer.stage("attend", queries, out)
        else:
            layer.compute(queries, out)
        if queries_next is not None and layer_idx + 1 < self.layer_num:
            nxt = self._layers[layer_idx + 1]
            q_next = queries_next.contiguous()
            self._q_next_alive = q_next
            sink = torch.empty_like(q_next)           # the stages take an output pointer; scan and select do not write it
            nxt.stage("scan", q_next, sink)
            nxt.stage("select", q_next, sink)
            self._ahead[layer_idx + 1] = True
        return out

    def _compute_host_tier(self, queries, layer_idx, out):
        """One layer with the cluster store in pinned host memory (the reference's steps 1-10,
        cache_hub/retroinfer_cache.py:558-697)."""
        from ..kernels import gather_copy_and_concat, gather_copy_and_scatter

        layer, wb = self._layers[layer_idx], self.wave_buffer[layer_idx]
        per = self._per_device[self.layer_mapping[str(layer_idx)]]
        g, d = self.batch_groups, self.head_dim
        if out is None:
            out = torch.empty_like(queries)
        static_len = self.static_pattern_total if layer_idx == self.layer_num - 1 else self.static_pattern_total + 1
        layer.stage("scan", queries, out)
        layer.stage("select", queries, out)
        if self.stage_misses:
            return self._finish_host_tier_staged(queries, layer_idx, out, static_len)
        self.cluster_ids[layer_idx].copy_(layer.retrieved_ids)          # blocking device-to-host copy (:575)
        wb.batch_access()                                                # hit/miss page lists; LRU update in background
        (hit_ids, hit_sizes, hit_cum, hit_n, miss_ids, miss_sizes, miss_cum, miss_n,
         upd_buf, upd_sizes, upd_cache, upd_n) = self.page_lists[layer_idx]
        sk = self.steady_zone_keys[layer_idx].view(g, self.static_stride, d)
        sv = self.steady_zone_values[layer_idx].view(g, self.static_stride, d)
        lk = self.list_keys[layer_idx].view(g, self.list_stride, d)
        lv = self.list_values[layer_idx].view(g, self.list_stride, d)
        ek, ev, lens = per["exec_keys"], per["exec_values"], per["valid_lengths"]
        gather_copy_and_concat(sk, lk, self.cache_keys[layer_idx], ek, sv, lv, self.cache_values[layer_idx], ev,
                               miss_ids, miss_sizes, miss_cum, miss_n, hit_ids, hit_sizes, hit_cum, hit_n, lens, g,
                               self.static_stride, self.list_stride, self.cache_size, self.execution_stride,
                               self.buffer_size, static_len)
        layer.attend_buffer(queries, out, ek, ev, lens)
        wb.sync()                                                        # update lists are final (:682)
        gather_copy_and_scatter(ek, self.cache_keys[layer_idx], ev, self.cache_values[layer_idx], upd_buf, upd_sizes,
                                upd_cache, upd_n, g, self.execution_stride, self.cache_size, self.buffer_size,
                                static_len)
        return out

    def _finish_host_tier_staged(self, queries, layer_idx, out, static_len):
        """The rest of a host-tier layer with the missed pages staged by the host and sent up on a side stream (what the
        reference does with UVA reads inside its copy kernel, :642-648), overlapped with the first attention pass."""
        import ctypes as C

        from .. import _lib
        from ..kernels import gather_copy_and_concat, gather_copy_and_scatter

        layer, wb = self._layers[layer_idx], self.wave_buffer[layer_idx]
        dev = self.layer_mapping[str(layer_idx)]
        per = self._per_device[dev]
        g, d, gs = self.batch_groups, self.head_dim, self.group_size
        main = torch.cuda.current_stream(dev)
        per["selected"].record(main)
        (hit_ids, hit_sizes, hit_cum, hit_n, miss_ids, miss_sizes, miss_cum, miss_n,
         upd_buf, upd_sizes, upd_cache, upd_n) = self.page_lists[layer_idx]
        sk = self.steady_zone_keys[layer_idx].view(g, self.static_stride, d)
        sv = self.steady_zone_values[layer_idx].view(g, self.static_stride, d)
        lk = self.list_keys[layer_idx].view(g, self.list_stride, d)
        lv = self.list_values[layer_idx].view(g, self.list_stride, d)
        ek, ev, lens = per["exec_keys"], per["exec_values"], per["valid_lengths"]
        # 1. nothing of this needs the host: the steady rows into the execution buffer (a concat without pages), then the
        #    estimation zone + steady zone attention, with its log-sum-exp
        zero = self._zero_counts(dev, g)
        gather_copy_and_concat(sk, per["stage_dev"][0][0], self.cache_keys[layer_idx], ek, sv, per["stage_dev"][0][1],
                               self.cache_values[layer_idx], ev, miss_cum, miss_sizes, miss_cum, zero, hit_ids, hit_sizes,
                               hit_cum, zero, per["steady_lengths"], g, self.static_stride, per["stage_rows"],
                               self.cache_size, self.execution_stride, self.buffer_size, static_len)
        layer._bind(queries, per["part"].view_as(queries))
        _lib.check(_lib.lib.ri_wave_attend_buffer_lse(C.byref(layer.params), ek.data_ptr(), ev.data_ptr(), ek.shape[1],
                                                      per["steady_lengths"].data_ptr(), per["lse"].data_ptr(),
                                                      _lib.current_stream()), "ri_wave_attend_buffer_lse")
        # 2. host: ids are in pinned memory once the select stage is done; LRU walk; worker threads stage the missed pages
        per["selected"].synchronize()
        wb.batch_access()
        turn = per["turn"]
        per["turn"] = turn ^ 1
        per["uploaded"][turn].synchronize()          # the area's previous copy (two layers ago) is long done
        hk, hv = per["stage_host"][turn]
        dk, dv = per["stage_dev"][turn]
        rows = C.c_int32(0)
        _lib.check(_lib.lib.ri_wb_stage_misses(wb._h, lk.data_ptr(), lv.data_ptr(), self.list_stride, hk.data_ptr(),
                                               hv.data_ptr(), per["stage_rows"], d * 2, C.byref(rows)), "ri_wb_stage_misses")
        with torch.cuda.stream(per["copy_stream"]):
            _lib.check(_lib.lib.ri_stage_upload(dk.data_ptr(), dv.data_ptr(), hk.data_ptr(), hv.data_ptr(), g,
                                                per["stage_rows"], rows.value, d * 2, per["copy_stream"].cuda_stream),
                       "ri_stage_upload")
            per["uploaded"][turn].record(per["copy_stream"])
        # 3. behind the copy: missed pages (from the device staging area) and hit pages behind the steady rows, the second
        #    attention pass over them, merged with the first by log-sum-exp
        main.wait_event(per["uploaded"][turn])
        gather_copy_and_concat(sk, dk, self.cache_keys[layer_idx], ek, sv, dv, self.cache_values[layer_idx], ev,
                               miss_cum, miss_sizes, miss_cum, miss_n, hit_ids, hit_sizes, hit_cum, hit_n, lens, g,
                               self.static_stride, per["stage_rows"], self.cache_size, self.execution_stride,
                               self.buffer_size, static_len)
        torch.sub(lens, static_len, out=per["rest_lengths"])
        off = static_len * d * ek.element_size()
        _lib.check(_lib.lib.ri_weighted_flash_decoding(
            queries.data_ptr(), ek.data_ptr() + off, ev.data_ptr() + off, None, per["rest_lengths"].data_ptr(),
            per["part"].data_ptr(), per["lse"].data_ptr(), out.data_ptr(), None, g, gs, self.execution_stride,
            _lib.dtype_code(self.dtype), _lib.current_stream()), "ri_weighted_flash_decoding")
        wb.sync()                                     # update lists are final (:682)
        gather_copy_and_scatter(ek, self.cache_keys[layer_idx], ev, self.cache_values[layer_idx], upd_buf, upd_sizes,
                                upd_cache, upd_n, g, self.execution_stride, self.cache_size, self.buffer_size, static_len)
        return out

    def _compute_host_tier_pull(self, queries, layer_idx, queries_next, out):
        """One host-tier layer with the missed pages pulled over PCIe by a copy kernel on a side stream.

        First pass (main stream): estimation zone + steady zone, with its log-sum-exp.  Second pass, behind the
        pull's event: the retrieved pages, merged with the first.  With ``use_cluster_estimation`` and a
        ``queries_next`` the NEXT layer's search is enqueued in front of this layer's own work and its list walk and
        pull are started before this call returns: the host walks the lists while the GPU attends this layer, and the
        next layer's pages cross PCIe under this layer's second pass and the next layer's first."""
        import ctypes as C

        from .. import _lib
        from ..kernels import gather_copy_and_scatter

        layer, wb = self._layers[layer_idx], self.wave_buffer[layer_idx]
        dev = self.layer_mapping[str(layer_idx)]
        per = self._per_device[dev]
        g, gs = self.batch_groups, self.group_size
        main = torch.cuda.current_stream(dev)
        if out is None:
            out = torch.empty_like(queries)
        static_len = self.static_pattern_total if layer_idx == self.layer_num - 1 else self.static_pattern_total + 1
        par = layer_idx & 1
        # 1. searches first: the host needs their ids soonest.  The next layer's (with the caller's estimate of its
        #    query), then this layer's own unless it was searched one layer ahead
        ahead = (self.use_cluster_estimation and queries_next is not None and layer_idx + 1 < self.layer_num
                 and self.layer_mapping[str(layer_idx + 1)] == dev)
        if ahead:
            self._q_next_alive = queries_next.contiguous()
            self._search(layer_idx + 1, self._q_next_alive, par ^ 1)
        searched_before = self._ahead[layer_idx]
        if searched_before:
            self._ahead[layer_idx] = False
            layer.stage("rescore", queries, out)          # the estimation entries' scores for the real query
        else:
            self._search(layer_idx, queries, par)
        # 2. nothing of this needs a page: estimation zone + steady zone, read where they lie
        per["steady_lengths"].fill_(static_len)
        layer._bind(queries, per["part"].view_as(queries))
        _lib.check(_lib.lib.ri_wave_attend_buffer_lse(
            C.byref(layer.params), self.steady_zone_keys[layer_idx].data_ptr(), self.steady_zone_values[layer_idx].data_ptr(),
            self.static_stride, per["steady_lengths"].data_ptr(), per["lse"].data_ptr(), _lib.current_stream()),
            "ri_wave_attend_buffer_lse")
        if not searched_before:
            self._lists_and_pull(layer_idx, par)          # the host walks the lists while the first pass runs
        # 3. behind the pull: the second pass over the pages, merged with the first by log-sum-exp
        ek, ev = per["exec"][par]
        rest = per["rest_lengths"][par]
        main.wait_event(per["pulled"][par])
        _lib.check(_lib.lib.ri_weighted_flash_decoding(
            queries.data_ptr(), ek.data_ptr(), ev.data_ptr(), None, rest.data_ptr(), per["part"].data_ptr(),
            per["lse"].data_ptr(), out.data_ptr(), None, g, gs, self.execution_stride, _lib.dtype_code(self.dtype),
            _lib.current_stream()), "ri_weighted_flash_decoding")
        torch.add(rest, static_len, out=per["valid_lengths"])
        if ahead:
            self._lists_and_pull(layer_idx + 1, par ^ 1)
            self._ahead[layer_idx + 1] = True
        # 4. admit the missed pages (they lie in the execution buffer from row 0)
        upd_buf, upd_sizes, upd_cache, upd_n = self.page_lists[layer_idx][8:12]
        wb.sync()                                     # update lists are final (:682)
        gather_copy_and_scatter(ek, self.cache_keys[layer_idx], ev, self.cache_values[layer_idx], upd_buf, upd_sizes,
                                upd_cache, upd_n, g, self.execution_stride, self.cache_size, self.buffer_size, 0)
        return out

    def _search(self, layer_idx, q, par):
        """scan + select of one layer on the main stream; the ranked ids land in pinned memory."""
        layer = self._layers[layer_idx]
        per = self._per_device[self.layer_mapping[str(layer_idx)]]
        sink = per["part"].view_as(q)                 # the stages take an output pointer; these two do not write it
        layer.stage("scan", q, sink)
        layer.stage("select", q, sink)
        per["selected"][par].record(torch.cuda.current_stream(sink.device))

    def _lists_and_pull(self, layer_idx, par):
        """Host: wait for the ids, walk the LRU lists.  Side stream: missed pages from the pinned store (read by the
        copy kernel over PCIe) and hit pages from the GPU cache into execution buffer ``par`` from row 0."""
        from ..kernels import gather_copy_and_concat

        wb = self.wave_buffer[layer_idx]
        dev = self.layer_mapping[str(layer_idx)]
        per = self._per_device[dev]
        g, d = self.batch_groups, self.head_dim
        per["selected"][par].synchronize()
        wb.batch_access()
        (hit_ids, hit_sizes, hit_cum, hit_n, miss_ids, miss_sizes, miss_cum, miss_n) = self.page_lists[layer_idx][:8]
        ek, ev = per["exec"][par]
        side = per["copy_stream"]
        # this buffer's readers of two layers ago were enqueued before the search whose event this is
        side.wait_event(per["selected"][par])
        sk = self.steady_zone_keys[layer_idx].view(g, self.static_stride, d)
        sv = self.steady_zone_values[layer_idx].view(g, self.static_stride, d)
        lk = self.list_keys[layer_idx].view(g, self.list_stride, d)
        lv = self.list_values[layer_idx].view(g, self.list_stride, d)
        with torch.cuda.stream(side):
            gather_copy_and_concat(sk, lk, self.cache_keys[layer_idx], ek, sv, lv, self.cache_values[layer_idx], ev,
                                   miss_ids, miss_sizes, miss_cum, miss_n, hit_ids, hit_sizes, hit_cum, hit_n,
                                   per["rest_lengths"][par], g, self.static_stride, self.list_stride, self.cache_size,
                                   self.execution_stride, self.buffer_size, 0)
        per["pulled"][par].record(side)

    def _zero_counts(self, dev, g):
        per = self._per_device[dev]
        if "zero_counts" not in per:
            per["zero_counts"] = torch.zeros((g,), dtype=torch.int32, pin_memory=True)
        return per["zero_counts"]
