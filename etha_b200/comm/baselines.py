"""Comparison method: gather the whole tensor, broadcast it to everybody, re-slice locally.

Kept only as the slow yardstick of the benchmarks (reference: `gather_broadcast_comm`,
src/etha/comm/comm_methods.py:16-50).
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
from torch.distributed.tensor import DTensor
from torch.distributed.tensor._utils import _compute_local_shape_and_global_offset
from torch.distributed.tensor.placement_types import Placement

from .planner import mesh_tensor_of

__all__ = ["gather_broadcast_comm", "local_slice_of"]


def local_slice_of(full: torch.Tensor, mesh, placements: Sequence[Placement], rank: int) -> torch.Tensor:
    """The local shard `rank` holds of `full` under `(mesh, placements)` (Shard/Replicate only)."""
    m = mesh_tensor_of(mesh)
    coord = (m == rank).nonzero()[0].tolist()
    shape, offset = _compute_local_shape_and_global_offset(tuple(full.shape), tuple(m.shape), coord, tuple(placements))
    index = tuple(slice(o, o + n) for o, n in zip(offset, shape))
    return full[index]


def gather_broadcast_comm(
    target_mesh,
    target_specs: Sequence[Placement],
    local_tensor: DTensor | None,
    origin_tensor: torch.Tensor,
    source_world_size: int,
) -> torch.Tensor | None:
    """Ranks `[0, source_world_size)` hold `local_tensor`; every later rank returns its target shard.

    `origin_tensor` only supplies shape, dtype and device of the full tensor.
    """
    rank = dist.get_rank()
    with torch.profiler.record_function("gather_broadcast::gather"):
        full = local_tensor.full_tensor() if rank < source_world_size else None
    with torch.profiler.record_function("gather_broadcast::broadcast"):
        if full is None:
            full = torch.empty(origin_tensor.shape, dtype=origin_tensor.dtype, device=origin_tensor.device)
        dist.broadcast(full, src=0)
        dist.barrier()
    with torch.profiler.record_function("gather_broadcast::reslice"):
        if rank < source_world_size:
            return None
        return local_slice_of(full, target_mesh, target_specs, rank).clone()
