"""Head sharding across the GPUs of one box, and the matching split of the projections either side.

Attention is independent per (sequence, head) and per KV-head group, so the engine scales by
giving each rank a contiguous range of KV heads together with the query heads that read them;
nothing crosses NVLink inside the operator.  Only a caller that wants the concatenated
[rows, E] output pays for one all-gather (NCCL over NVLink/NVSwitch through torch.distributed)
followed by a local interleave kernel.  The reference has no multi-GPU path to mirror
(src/cuda/thread_pool.h:19-22).
"""
from __future__ import annotations

import ctypes as C
import os
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


class NcclCommunicator:
    """An ncclComm_t over the ranks of a torch.distributed group, for the C entry point
    pluto_allgather_heads (a C++ host owns such a communicator anyway; this is the Python
    stand-in).  It is created with ctypes on the NCCL library torch itself loads, made globally
    visible so that the engine binds the same copy; the unique id travels through the group's
    own broadcast.  The calling thread's current CUDA device is the rank's GPU."""

    class _UniqueId(C.Structure):
        _fields_ = [("internal", C.c_byte * 128)]

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._nccl = C.CDLL(self._library_path(), mode=C.RTLD_GLOBAL)
        self._nccl.ncclGetErrorString.restype = C.c_char_p
        uid = self._UniqueId()
        if self.rank == 0:
            self._check(self._nccl.ncclGetUniqueId(C.byref(uid)))
        box = [bytes(uid.internal)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group else 0, group=group)
        C.memmove(C.byref(uid), box[0], 128)
        self.handle = C.c_void_p()
        self._nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, self._UniqueId, C.c_int]
        self._check(self._nccl.ncclCommInitRank(C.byref(self.handle), self.world, uid, self.rank))

    @staticmethod
    def _library_path() -> str:
        bundled = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia", "nccl", "lib",
                               "libnccl.so.2")
        return bundled if os.path.exists(bundled) else "libnccl.so.2"

    def _check(self, code: int) -> None:
        if code != 0:
            raise PlutoStatusError("Internal", "NCCL: " + self._nccl.ncclGetErrorString(code).decode(), code)

    def close(self) -> None:
        if self.handle:
            self._nccl.ncclCommDestroy.argtypes = [C.c_void_p]
            self._nccl.ncclCommDestroy(self.handle)
            self.handle = C.c_void_p()


def allgather_heads(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                    comm: Optional[NcclCommunicator] = None, out: Optional[torch.Tensor] = None,
                    scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """local [rows, E/G] (this rank's heads, same shape on every rank) -> [rows, E] on every rank,
    columns ordered by rank.  One all-gather plus a local interleave.  With `comm` both happen
    inside the C entry point pluto_allgather_heads (NCCL on the current stream); without it the
    gather goes through torch.distributed.  `out` / `scratch` ([world*rows, cols]) let a caller
    reuse buffers."""
    world = comm.world if comm is not None else dist.get_world_size(group)
    if world == 1:
        return local
    local = local.contiguous()
    rows, cols = local.shape
    gathered = scratch if scratch is not None else torch.empty((world * rows, cols), dtype=local.dtype,
                                                              device=local.device)
    if comm is not None:
        if out is None:
            out = torch.empty((rows, world * cols), dtype=local.dtype, device=local.device)
        check(_capi.lib().pluto_allgather_heads(torch.cuda.current_stream().cuda_stream, comm.handle,
                                                local.data_ptr(), gathered.data_ptr(), out.data_ptr(),
                                                world, rows, cols * local.element_size()))
        return out
    dist.all_gather_into_tensor(gathered, local, group=group)  # rank-major [world][rows][cols]
    if out is None:
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
