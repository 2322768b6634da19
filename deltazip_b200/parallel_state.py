"""Tensor-parallel group and the collectives the delta layers need.

Role of serving/vllm/model_executor/parallel_utils/parallel_state.py:22-87 and
communication_op.py:17-105 for this path: one tensor-parallel group spanning
all ranks (one process per GPU, torch.distributed; NCCL on GPUs, gloo in the
CPU tests), all-reduce after row-parallel layers (the library's peer-memory
all-reduce when the message qualifies, else the backend's), all-gather for
gather_output column layers.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

_TP_GROUP: Optional[dist.ProcessGroup] = None
_TP_SIZE = 1
_TP_RANK = 0


def initialize_model_parallel(tensor_model_parallel_size: int = 1,
                              disable_custom_all_reduce: bool = False) -> None:
    """All ranks of the default group form the tensor-parallel group.  On an NCCL group of up
    to 8 ranks the peer-memory all-reduce is set up too (collective call) unless disabled, as
    the reference does in its worker (serving/vllm/worker/worker.py: init_custom_ar)."""
    global _TP_GROUP, _TP_SIZE, _TP_RANK
    if tensor_model_parallel_size == 1 or not dist.is_initialized():
        _TP_GROUP, _TP_SIZE, _TP_RANK = None, 1, 0
        return
    world = dist.get_world_size()
    if world != tensor_model_parallel_size:
        raise ValueError(f"world size {world} != tensor parallel size {tensor_model_parallel_size}")
    _TP_GROUP = dist.group.WORLD
    _TP_SIZE = world
    _TP_RANK = dist.get_rank()
    if not disable_custom_all_reduce and dist.get_backend() == "nccl" and world <= 8:
        from . import custom_all_reduce
        custom_all_reduce.init_custom_ar(_TP_RANK, world, group=_TP_GROUP)


def destroy_model_parallel() -> None:
    global _TP_GROUP, _TP_SIZE, _TP_RANK
    from . import custom_all_reduce
    custom_all_reduce.destroy_custom_ar()
    _TP_GROUP, _TP_SIZE, _TP_RANK = None, 1, 0


def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE


def get_tensor_model_parallel_rank() -> int:
    return _TP_RANK


def tensor_model_parallel_all_reduce(x: torch.Tensor) -> torch.Tensor:
    """Sum over the tensor-parallel ranks (no-op for one rank).  May or may not work in
    place: always use the return value (same contract as communication_op.py:17-40)."""
    if _TP_SIZE == 1:
        return x
    from .custom_all_reduce import custom_all_reduce
    out = custom_all_reduce(x)
    if out is not None:
        return out
    dist.all_reduce(x, group=_TP_GROUP)
    return x


def tensor_model_parallel_all_gather(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if _TP_SIZE == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(_TP_SIZE)]
    dist.all_gather(parts, x.contiguous(), group=_TP_GROUP)
    return torch.cat(parts, dim=dim)


def tensor_model_parallel_gather(x: torch.Tensor, dst: int = 0, dim: int = -1,
                                 sizes: Optional[list] = None) -> Optional[torch.Tensor]:
    """Concatenation of every rank's `x` along `dim` on rank `dst`, None elsewhere (contract of
    communication_op.py:74-104).  `sizes` gives every rank's extent along `dim` when the shards
    are uneven (vocabulary rows cut at 128-row units): the pieces travel padded to the widest
    and are trimmed on arrival."""
    if _TP_SIZE == 1:
        return x
    if dim < 0:
        dim += x.dim()
    widest = max(sizes) if sizes else x.shape[dim]
    piece = x
    if x.shape[dim] != widest:
        pad = list(x.shape)
        pad[dim] = widest - x.shape[dim]
        piece = torch.cat([x, x.new_zeros(pad)], dim=dim)
    piece = piece.contiguous()
    parts = [torch.empty_like(piece) for _ in range(_TP_SIZE)] if _TP_RANK == dst else None
    dist.gather(piece, parts, dst=dst, group=_TP_GROUP)
    if _TP_RANK != dst:
        return None
    if sizes:
        parts = [p.narrow(dim, 0, n) for p, n in zip(parts, sizes)]
    return torch.cat(parts, dim=dim)


# Tensor-parallel cuts are made at whole 128-wide units on both sides of a column-parallel /
# row-parallel pair (128 output rows of qkv / gate / up = 128 input columns of o_proj /
# down_proj), so that a producer's shard is exactly its consumer's K range for every rank
# count, also when the unit count does not divide evenly (Llama-2-7B: 11008 = 86 units).
SHARD_UNIT = 128


def shard_range(total: int, unit: int, rank: int, size: int):
    """[lo, hi) of `total` for `rank`, cut at multiples of `unit` (use SHARD_UNIT for model
    dimensions)."""
    if total % unit:
        raise ValueError(f"{total} is not a multiple of {unit}")
    units = total // unit
    return units * rank // size * unit, units * (rank + 1) // size * unit
