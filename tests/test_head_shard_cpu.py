"""Multi-rank host logic on CPU (gloo, world size 2): KV-head sharding and the head gather give
exactly the single-rank result, because every (request, kv-head) group is independent."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _full_problem():
    from helpers import Case, build_cpu_index, queries

    case = Case(2, 4, 2, 512 + 68, 32, 1, 3, 8, seed=17)
    return case, build_cpu_index(case), queries(case, seed=5)


def _attend(case, cpu, q, groups, heads_q):
    from oracle import attention as oat

    sel = lambda t: t[groups]  # noqa: E731
    return oat.compute(q, sel(cpu["centroids"]), sel(cpu["value_sum"]), sel(cpu["cluster_size"]), sel(cpu["mask"]),
                       sel(cpu["cluster_count"]), sel(cpu["cluster_offset"]), sel(cpu["keys"]), sel(cpu["values"]),
                       sel(cpu["steady_keys"]), sel(cpu["steady_values"]), 68, case.nprobe,
                       case.nprobe + case.n_estimate, case.page_size, case.pages())


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from retrievalattention_b200.head_shard import HeadGather, HeadShard

    case, cpu, q = _full_problem()
    shard = HeadShard(rank, world, case.kv_heads, case.q_heads, case.batch)
    hs = shard.kv_head_slice()
    groups = [b * case.kv_heads + h for b in range(case.batch) for h in range(hs.start, hs.stop)]
    q_local = q[:, :, shard.q_head_slice()].contiguous()
    out_local = _attend(case, cpu, q_local, groups, shard.local_q_heads)
    gathered = HeadGather(shard)(out_local)
    if rank == 0:
        full = _attend(case, cpu, q, list(range(case.groups)), case.q_heads)
        ret["equal"] = bool(torch.equal(gathered.contiguous().view(torch.int16), full.view(torch.int16)))
        ret["shape"] = tuple(gathered.shape)
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_attention_equals_single_rank():
    world, port = 2, _free_port()
    with mp.get_context("spawn").Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert ret["equal"], "gathered head slices differ from the single-rank result"
        assert ret["shape"] == (2, 1, 8, 128)


def test_shard_arithmetic():
    from retrievalattention_b200.head_shard import HeadShard

    s = HeadShard(5, 8, 8, 64, 16)
    assert (s.head_shards, s.batch_shards, s.local_kv_heads, s.local_q_heads, s.local_batch) == (8, 1, 1, 8, 16)
    assert s.kv_head_slice() == slice(5, 6) and s.q_head_slice() == slice(40, 48)
    s = HeadShard(5, 8, 4, 28, 8)            # more ranks than kv heads: the rest shards the batch
    assert (s.head_shards, s.batch_shards, s.head_index, s.batch_index, s.local_batch) == (4, 2, 1, 1, 4)
    assert s.head_group_ranks() == [4, 5, 6, 7] and s.batch_slice() == slice(4, 8)
    with pytest.raises(ValueError):
        HeadShard(0, 3, 8, 32, 4)
