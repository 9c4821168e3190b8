"""Multi-rank host logic on CPU: shard plans and the all-gather + interleave plumbing with two
gloo ranks (no GPU, no NCCL)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pluto_b200 import PlutoStatusError
from pluto_b200.sharding import allgather_heads, shard_heads


def test_shard_plan_covers_heads_exactly():
    for world in (1, 2, 4, 8):
        shards = [shard_heads(40, 8, world, r) for r in range(world)]
        assert [s.kv_begin for s in shards] == [r * 8 // world for r in range(world)]
        assert sum(s.q_heads for s in shards) == 40 and sum(s.kv_heads for s in shards) == 8
        for s in shards:
            for h in range(s.q_begin, s.q_end):
                assert s.kv_begin <= h // 5 < s.kv_end
    with pytest.raises(PlutoStatusError):
        shard_heads(40, 8, 3, 0)
    with pytest.raises(PlutoStatusError):
        shard_heads(40, 7, 1, 0)
    with pytest.raises(PlutoStatusError):
        shard_heads(40, 8, 2, 2)


def _worker(rank, world, port, rows, cols):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(rows * world * cols, dtype=torch.float32).view(rows, world * cols)
        local = full[:, rank * cols:(rank + 1) * cols].contiguous()
        out = allgather_heads(local)
        assert torch.equal(out, full)
        shard = shard_heads(12, 4, world, rank)
        owned = torch.zeros(12)
        owned[shard.q_begin:shard.q_end] = 1
        dist.all_reduce(owned)
        assert torch.equal(owned, torch.ones(12))  # every head owned exactly once
    finally:
        dist.destroy_process_group()


def test_allgather_heads_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, 6, 10), nprocs=2, join=True)
