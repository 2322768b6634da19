"""Tensor-parallel group and the collectives the delta layers need.

Role of serving/vllm/model_executor/parallel_utils/parallel_state.py:22-87 and
communication_op.py:17-105 for this path: one tensor-parallel group spanning
all ranks (one process per GPU, torch.distributed; NCCL on GPUs, gloo in the
CPU tests), all-reduce after row-parallel layers, all-gather for
gather_output column layers.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

_TP_GROUP: Optional[dist.ProcessGroup] = None
_TP_SIZE = 1
_TP_RANK = 0


def initialize_model_parallel(tensor_model_parallel_size: int = 1) -> None:
    """All ranks of the default group form the tensor-parallel group."""
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


def destroy_model_parallel() -> None:
    global _TP_GROUP, _TP_SIZE, _TP_RANK
    _TP_GROUP, _TP_SIZE, _TP_RANK = None, 1, 0


def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE


def get_tensor_model_parallel_rank() -> int:
    return _TP_RANK


def tensor_model_parallel_all_reduce(x: torch.Tensor) -> torch.Tensor:
    """In-place sum over the tensor-parallel ranks (no-op for one rank)."""
    if _TP_SIZE == 1:
        return x
    dist.all_reduce(x, group=_TP_GROUP)
    return x


def tensor_model_parallel_all_gather(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if _TP_SIZE == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(_TP_SIZE)]
    dist.all_gather(parts, x.contiguous(), group=_TP_GROUP)
    return torch.cat(parts, dim=dim)


def shard_range(total: int, unit: int, rank: int, size: int):
    """[lo, hi) of `total` for `rank`, cut at multiples of `unit` (whole 128-row tiles for
    column-parallel layers, whole 64-column blocks for row-parallel ones)."""
    if total % unit:
        raise ValueError(f"{total} is not a multiple of {unit}")
    units = total // unit
    return units * rank // size * unit, units * (rank + 1) // size * unit
