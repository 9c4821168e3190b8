"""Head sharding across the GPUs of one box.

Attention is independent per (sequence, head) and per KV-head group, so the engine scales by
giving each rank a contiguous range of KV heads together with the query heads that read them;
nothing crosses NVLink inside the operator.  Only a caller that wants the concatenated
[rows, E] output pays for one all-gather (NCCL over NVLink/NVSwitch through torch.distributed)
followed by a local interleave kernel.  The reference has no multi-GPU path to mirror
(src/cuda/thread_pool.h:19-22).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import _capi
from ._capi import PlutoStatusError, check


@dataclass(frozen=True)
class HeadShard:
    """Heads owned by one rank: KV heads [kv_begin, kv_end) and query heads [q_begin, q_end)."""
    rank: int
    world: int
    kv_begin: int
    kv_end: int
    q_begin: int
    q_end: int

    @property
    def kv_heads(self) -> int:
        return self.kv_end - self.kv_begin

    @property
    def q_heads(self) -> int:
        return self.q_end - self.q_begin


def shard_heads(q_heads: int, kv_heads: int, world: int, rank: int) -> HeadShard:
    """Contiguous, equal KV-head ranges; a rank's query heads are exactly those of its KV heads
    (query head h reads KV head h // (q_heads // kv_heads), cached_attention_ops.cc:92)."""
    if q_heads <= 0 or kv_heads <= 0 or q_heads % kv_heads != 0:
        raise PlutoStatusError("InvalidArgument", "invalid full-attention dimensions or parameters", -1)
    if world <= 0 or not 0 <= rank < world:
        raise PlutoStatusError("InvalidArgument", "rank outside the process group", -1)
    if kv_heads % world != 0:
        raise PlutoStatusError("InvalidArgument",
                               f"{kv_heads} KV heads do not divide over {world} ranks", -1)
    per = kv_heads // world
    group = q_heads // kv_heads
    return HeadShard(rank, world, rank * per, (rank + 1) * per, rank * per * group,
                     (rank + 1) * per * group)


def allgather_heads(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """local [rows, E/G] (this rank's heads, same shape on every rank) -> [rows, E] on every rank,
    columns ordered by rank.  One all-gather plus a local interleave."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    local = local.contiguous()
    rows, cols = local.shape
    gathered = torch.empty((world * rows, cols), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered, local, group=group)  # rank-major [world][rows][cols]
    out = torch.empty((rows, world * cols), dtype=local.dtype, device=local.device)
    if local.is_cuda:
        check(_capi.lib().pluto_interleave_heads(torch.cuda.current_stream().cuda_stream,
                                                 gathered.data_ptr(), out.data_ptr(), world, rows,
                                                 cols * local.element_size()))
    else:
        # host tensors (gloo, used by the CPU tests of this plumbing): a plain strided copy
        out.view(rows, world, cols).copy_(gathered.view(world, rows, cols).permute(1, 0, 2))
    return out
