"""Multi-rank host logic on CPU: two gloo ranks shard heads, run a per-head
function on their shards and reproduce the single-rank result bit for bit; the
timing reduction takes the slowest rank."""
from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
from fhob.sharding import head_shard, max_over_ranks, sharded_call


def test_head_shard_partitions():
    for total in (0, 1, 7, 32, 64, 512, 513):
        for world in (1, 2, 3, 4, 8):
            spans = [head_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert spans[-1][0] + spans[-1][1] == total
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    assert head_shard(512, 8, 3) == (192, 64)       # the scaling configuration: 64 heads per GPU
    assert head_shard(32, 8, 7) == (28, 4)          # long-context configuration: 4 heads per GPU
    with pytest.raises(ValueError):
        head_shard(8, 2, 2)


def _per_head(q, k):
    """Stand-in for the operator on CPU: any function that treats heads independently."""
    return torch.einsum("hqd,hkd->hq", q, k).contiguous()


def _worker(rank, world, port, out_dir):
    for p in (str(ROOT), str(ROOT / "flash-hob_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(6, 16, 8, generator=g)
    k = torch.randn(6, 24, 8, generator=g)
    start, count, res = sharded_call(_per_head, (q, k), 6, world, rank)
    slowest = max_over_ranks(10.0 + rank)           # pretend rank r took 10+r ms
    gathered = [None] * world
    dist.all_gather_object(gathered, (start, count, res))
    if rank == 0:
        full = torch.cat([g[2] for g in sorted(gathered, key=lambda g: g[0])])
        torch.save(dict(full=full, slowest=slowest, want=_per_head(q, k)), os.path.join(out_dir, "r0.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_single_rank(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = torch.load(tmp_path / "r0.pt")
    assert torch.equal(r["full"], r["want"])
    assert r["slowest"] == 11.0
