"""Multi-rank host logic on CPU: shard plans and the all-gather + interleave plumbing with two
gloo ranks (no GPU, no NCCL)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pluto_b200 import PlutoStatusError
from pluto_b200.sharding import (allgather_heads, projection_rows, reduce_row_parallel, shard_heads,
                                 shard_input_columns, shard_output_major)


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


def test_projection_shards_tile_the_matrices_and_their_scale_blocks():
    hq, hkv, d, hidden = 8, 4, 128, 384
    wq = torch.arange(hq * 2 * d * hidden, dtype=torch.float32).view(hq * 2 * d, hidden)
    sq = torch.arange((hq * 2 * d // 128) * (hidden // 128), dtype=torch.float32)
    wo = torch.arange(hidden * hq * d, dtype=torch.float32).view(hidden, hq * d)
    so = torch.arange((hidden // 128) * (hq * d // 128), dtype=torch.float32)
    for world in (1, 2, 4):
        q_parts, q_scales, o_parts, o_scales, kv_rows = [], [], [], [], []
        for rank in range(world):
            shard = shard_heads(hq, hkv, world, rank)
            begin, end = projection_rows(shard, d, values_per_head=2)
            w, sc = shard_output_major(wq, sq, begin, end)
            assert w.data_ptr() == wq[begin:].data_ptr()          # a view, not a copy
            q_parts.append(w); q_scales.append(sc.view(-1, hidden // 128))
            kv_rows.append(projection_rows(shard, d, kv=True))
            cb, ce = projection_rows(shard, d)                    # the heads' columns of W_o
            w, sc = shard_input_columns(wo, so, cb, ce)
            assert w.is_contiguous()
            o_parts.append(w); o_scales.append(sc.view(hidden // 128, -1))
        assert torch.equal(torch.cat(q_parts), wq)
        assert torch.equal(torch.cat(q_scales).reshape(-1), sq)
        assert torch.equal(torch.cat(o_parts, dim=1), wo)
        assert torch.equal(torch.cat(o_scales, dim=1).reshape(-1), so)
        assert kv_rows[0][0] == 0 and kv_rows[-1][1] == hkv * d
        assert all(a[1] == b[0] for a, b in zip(kv_rows, kv_rows[1:]))
    with pytest.raises(PlutoStatusError):
        shard_output_major(wq, sq, 64, 256)                       # not on a scale-block boundary
    with pytest.raises(PlutoStatusError):
        shard_input_columns(wo, None, 0, hq * d + 1)


def _projection_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hkv, d, hidden = 4, 2, 8, 24
        gen = torch.Generator().manual_seed(5)
        x = torch.randn(3, hidden, generator=gen)
        wq = torch.randn(hq * d, hidden, generator=gen)           # output-major, as imported
        wo = torch.randn(hidden, hq * d, generator=gen)
        shard = shard_heads(hq, hkv, world, rank)
        begin, end = projection_rows(shard, d)
        local_q, _ = shard_output_major(wq, None, begin, end)
        heads = x @ local_q.t()                                   # column-parallel: no communication
        assert torch.allclose(heads, (x @ wq.t())[:, begin:end])
        local_o, _ = shard_input_columns(wo, None, begin, end)
        out = reduce_row_parallel(heads @ local_o.t())            # row-parallel + one reduction
        assert torch.allclose(out, (x @ wq.t()) @ wo.t(), atol=1e-4)
    finally:
        dist.destroy_process_group()


def test_column_then_row_parallel_projection_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_projection_worker, args=(2, port), nprocs=2, join=True)
