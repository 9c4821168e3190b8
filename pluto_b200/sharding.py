"""Head sharding across the GPUs of one box, and the matching split of the projections either side.

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


# -------------------------------------------------------------------------------------------------
# Projections either side of a head-sharded attention layer (src/llm/qwen/model.cc:192-227 calls
# them in this order: q/gate, k, v projections -> attention -> output projection).
#   * The q/gate, k and v projections are split by OUTPUT (column-parallel): an output-major
#     matrix [rows, hidden] gives each rank the contiguous rows of its own heads, so a rank's
#     shard is a view and its projection needs no communication.
#   * The output projection is split by INPUT (row-parallel): a rank multiplies its heads'
#     columns of W_o and the partial results are summed over the ranks (one all-reduce).
# -------------------------------------------------------------------------------------------------
def projection_rows(shard: HeadShard, head_dim: int, values_per_head: int = 1, kv: bool = False):
    """Row range [begin, end) of an output-major projection matrix that produces this rank's heads.
    values_per_head = 2 for Qwen's fused query + gate projection ([Hq, 2, D] outputs)."""
    if head_dim <= 0 or values_per_head <= 0:
        raise PlutoStatusError("InvalidArgument", "invalid projection dimensions", -1)
    per_head = head_dim * values_per_head
    if kv:
        return shard.kv_begin * per_head, shard.kv_end * per_head
    return shard.q_begin * per_head, shard.q_end * per_head


def shard_output_major(weights: torch.Tensor, scales: Optional[torch.Tensor], begin: int, end: int):
    """Rows [begin, end) of an output-major matrix [rows, cols] as a view, with the matching rows
    of its 128x128 block scales (fully_connected.cc:267-293) when it has them; the range must
    then start and end on a multiple of 128 rows (or at the matrix end)."""
    rows, cols = weights.shape
    if not 0 <= begin < end <= rows:
        raise PlutoStatusError("InvalidArgument", "projection shard outside the matrix", -1)
    if scales is None:
        return weights[begin:end], None
    if begin % 128 != 0 or (end % 128 != 0 and end != rows):
        raise PlutoStatusError("InvalidArgument",
                               "FP8 projection shards must cover whole 128-row scale blocks", -1)
    scale_cols = (cols + 127) // 128
    table = scales.view((rows + 127) // 128, scale_cols)
    return weights[begin:end], table[begin // 128:(end + 127) // 128].reshape(-1)


def shard_input_columns(weights: torch.Tensor, scales: Optional[torch.Tensor], begin: int, end: int):
    """Columns [begin, end) of an output-major matrix (the row-parallel split of the output
    projection), copied once at load time into a contiguous matrix, with the matching columns of
    its block scales; FP8 ranges must cover whole 128-column scale blocks."""
    rows, cols = weights.shape
    if not 0 <= begin < end <= cols:
        raise PlutoStatusError("InvalidArgument", "projection shard outside the matrix", -1)
    part = weights[:, begin:end].contiguous()
    if scales is None:
        return part, None
    if begin % 128 != 0 or (end % 128 != 0 and end != cols):
        raise PlutoStatusError("InvalidArgument",
                               "FP8 projection shards must cover whole 128-column scale blocks", -1)
    table = scales.view((rows + 127) // 128, (cols + 127) // 128)
    return part, table[:, begin // 128:(end + 127) // 128].contiguous().reshape(-1)


def reduce_row_parallel(partial: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sum of the ranks' partial output-projection results, returned in the input's dtype.  The
    partials are summed at fp32 (bf16 partials get one final rounding whatever the number of
    ranks).  This is NCCL's all-reduce over NVLink / NVSwitch as it stands: the projection kernel
    and the reduction are separate steps, not one fused kernel over peer memory."""
    if dist.get_world_size(group) == 1:
        return partial
    total = partial.float()
    dist.all_reduce(total, group=group)
    return total.to(partial.dtype)
