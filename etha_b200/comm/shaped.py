"""Shape-aware planning for tensors whose dimensions do not divide evenly over the meshes.

The pair-level `M2MMap` is shape independent: it cuts every local shard into equal cells of an lcm grid,
which only exists when all sharded dimensions divide evenly (the reference silently drops the remainder,
src/etha/comm/utils.py:53-55, src/etha/comm/get_chunks.py:18).  DTensor itself shards unevenly like
`torch.chunk` (pieces of ceil(n/k), the last ones shorter or empty).  `plan_for_shape` handles that
case: it computes every rank's box of the global tensor with DTensor's own arithmetic and intersects
consumer boxes with producer boxes.  The result is a list of explicit transfers with the same semantics
as the lcm plan (same replica-choice rule: consumer number j reads from the family of producer number
`j mod S`; same Partial families), and for evenly divisible shapes it moves exactly the same bytes.

It is also the planner for `_StridedShard` placements (the FSDP-over-TP layout the reference's CPU test and
benchmark use as a target, tests/test_communication_cpu.py:43, bench/transfer_benchmark.py:386-390): whenever the
strided shard is matched by later mesh dims of its split factor, every rank's shard is one box and is planned like
any other.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Any, Sequence

import torch
from torch.distributed.tensor._utils import _compute_local_shape_and_global_offset
from torch.distributed.tensor.placement_types import Partial, Placement, Replicate, Shard

from .ir import Chunk, PartialFamily, Transport, partial_family
from .planner import _check_placements, is_strided_shard, mesh_tensor_of, shards_dim

__all__ = ["BOX_PLAN_ONLY", "ShapedRoute", "ShapedPlan", "plan_for_shape", "shaped_to_chunks", "infer_global_shape", "needs_shaped_plan"]

class _BoxPlanOnly:
    """Stands in for an `M2MMap` where a layout has no shape-independent plan (`_StridedShard`): the pair is valid,
    its transfers are planned per tensor from explicit boxes."""

    def __repr__(self) -> str:
        return "BOX_PLAN_ONLY"


BOX_PLAN_ONLY = _BoxPlanOnly()

Box = tuple[tuple[int, int], ...]  # per dim (start, stop) in LOCAL coordinates of the owning rank


@dataclass(frozen=True)
class ShapedRoute:
    src_rank: int
    src_box: Box
    dsts: tuple[tuple[int, Box], ...]  # (consumer rank, box in the consumer's local tensor)

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(b - a for a, b in self.src_box)


@dataclass
class ShapedPlan:
    routes: list[ShapedRoute]
    global_shape: tuple[int, ...]
    source_partial_reductions: list[tuple[int, str]]


def _boxes(mesh: torch.Tensor, placements: Sequence[Placement], shape: Sequence[int]):
    eff = tuple(Replicate() if isinstance(p, Partial) else p for p in placements)
    out = {}
    for coord in itertools.product(*[range(n) for n in mesh.shape]):
        lshape, off = _compute_local_shape_and_global_offset(tuple(shape), tuple(mesh.shape), list(coord), eff)
        out[coord] = (tuple(lshape), tuple(off))
    return out


def needs_shaped_plan(mesh: Any, placements: Sequence[Placement], global_shape: Sequence[int]) -> bool:
    """True if some sharded dim of `global_shape` does not divide evenly over the mesh dims that shard it."""
    m = mesh_tensor_of(mesh)
    counts: dict[int, int] = {}
    for size, p in zip(m.shape, placements):
        if shards_dim(p) is not None:
            counts[p.dim] = counts.get(p.dim, 1) * int(size)
    return any(is_strided_shard(p) for p in placements) or any(global_shape[d] % c for d, c in counts.items())


def plan_for_shape(source_mesh: Any, source_placements: Sequence[Placement], target_mesh: Any,
                   target_placements: Sequence[Placement], global_shape: Sequence[int]) -> ShapedPlan:
    smesh, tmesh = mesh_tensor_of(source_mesh), mesh_tensor_of(target_mesh)
    source_placements, target_placements = tuple(source_placements), tuple(target_placements)
    _check_placements(source_placements, smesh, "source", allow_strided=True)
    _check_placements(target_placements, tmesh, "target", allow_strided=True)
    if any(isinstance(p, Partial) for p in target_placements):
        raise NotImplementedError("Partial is a source-only placement")
    shape = tuple(int(n) for n in global_shape)
    ndim = len(shape)
    for p in list(source_placements) + list(target_placements):
        if shards_dim(p) is not None and p.dim >= ndim:
            raise ValueError(f"{p} on a {ndim}-d tensor")
    reductions = [(i, p.reduce_op) for i, p in enumerate(source_placements) if isinstance(p, Partial)]
    sboxes, tboxes = _boxes(smesh, source_placements, shape), _boxes(tmesh, target_placements, shape)
    s_coords, t_coords = list(sboxes), list(tboxes)
    shard_dims = [i for i, p in enumerate(source_placements) if shards_dim(p) is not None]
    table: dict[tuple[int, Box], list[tuple[int, Box]]] = {}
    for j, tc in enumerate(t_coords):
        fam = s_coords[j % len(s_coords)]
        tshape, toff = tboxes[tc]
        if any(n == 0 for n in tshape):
            continue
        # producers of the family: free on the Shard mesh dims, pinned to the family coordinate elsewhere
        for sc in s_coords:
            if any(sc[i] != fam[i] for i in range(len(sc)) if i not in shard_dims):
                continue
            sshape, soff = sboxes[sc]
            lo = [max(a, b) for a, b in zip(soff, toff)]
            hi = [min(a + n, b + m) for a, n, b, m in zip(soff, sshape, toff, tshape)]
            if any(h <= l for l, h in zip(lo, hi)):
                continue
            sbox = tuple((l - o, h - o) for l, h, o in zip(lo, hi, soff))
            dbox = tuple((l - o, h - o) for l, h, o in zip(lo, hi, toff))
            table.setdefault((int(smesh[sc]), sbox), []).append((int(tmesh[tc]), dbox))
    routes = [ShapedRoute(r, box, tuple(sorted(dsts))) for (r, box), dsts in sorted(table.items())]
    return ShapedPlan(routes, shape, reductions)


def infer_global_shape(mesh: Any, placements: Sequence[Placement], local_shapes: dict[int, Sequence[int]]) -> tuple[int, ...]:
    """Global shape from every rank's local shape: per tensor dim, the local extents of the ranks that differ only
    along the mesh dims sharding that dim add up."""
    return tuple(_global_by_brute_force(mesh_tensor_of(mesh), tuple(placements), local_shapes))


def _global_by_brute_force(m: torch.Tensor, placements, local_shapes) -> list[int]:
    first = int(m.reshape(-1)[0])
    ndim = len(local_shapes[first])
    out = list(local_shapes[first])
    for d in range(ndim):
        dims = [i for i, p in enumerate(placements) if shards_dim(p) == d]
        if not dims:
            continue
        total = 0
        for combo in itertools.product(*[range(m.shape[i]) for i in dims]):
            index = [0] * m.dim()
            for i, c in zip(dims, combo):
                index[i] = c
            total += local_shapes[int(m[tuple(index)])][d]
        out[d] = total
    return out


def shaped_to_chunks(plan: ShapedPlan, rank: int, source_tensor: torch.Tensor | None = None,
                     target_tensor: torch.Tensor | None = None, transfer_dtype: torch.dtype | None = None, *,
                     source_mesh: Any = None, tensor_id: int = 0) -> list[Chunk]:
    """Chunks of one tensor for `rank` (same contract as `m2m_to_chunks`, explicit boxes instead of cells)."""
    reductions = plan.source_partial_reductions
    fams: dict[int, PartialFamily | None] = {}

    def fam_of(primary: int):
        if not reductions:
            return None
        if primary not in fams:
            if source_mesh is None:
                raise ValueError("Partial source: pass source_mesh=")
            fams[primary] = partial_family(mesh_tensor_of(source_mesh), reductions, primary)
        return fams[primary]

    sl = lambda box: tuple(slice(a, b) for a, b in box)
    chunks: list[Chunk] = []
    for route_id, route in enumerate(plan.routes):
        primary, fam = route.src_rank, fam_of(route.src_rank)
        wire = tuple(sorted({r for r, _ in route.dsts if r != primary}))
        local = next((box for r, box in route.dsts if r == primary), None)
        transport = Transport.LOCAL if not wire else (Transport.P2P if len(wire) == 1 else Transport.BROADCAST)
        cell = tuple(a for a, _ in route.src_box)
        if primary == rank:
            c = Chunk(transport=transport, is_source=True, is_target=local is not None, src_rank=primary, dst_ranks=wire,
                      chunk_shape=route.shape, src_idx=cell, src_tensor=source_tensor, src_index=sl(route.src_box),
                      transfer_dtype=transfer_dtype, family=fam, tensor_id=tensor_id, route_id=route_id)
            if local is not None:
                c.dst_tensor, c.dst_index, c.dst_idx = target_tensor, sl(local), tuple(a for a, _ in local)
            chunks.append(c)
        elif fam is not None and rank in fam.ranks and source_tensor is not None:
            chunks.append(Chunk(transport=Transport.NONE, is_source=True, is_target=False, src_rank=primary, dst_ranks=wire,
                                chunk_shape=route.shape, src_idx=cell, src_tensor=source_tensor, src_index=sl(route.src_box),
                                transfer_dtype=transfer_dtype, family=fam, contributes_to=primary, tensor_id=tensor_id,
                                route_id=route_id))
        if primary != rank:
            for r, box in route.dsts:
                if r == rank:
                    chunks.append(Chunk(transport=Transport.P2P if len(wire) == 1 else Transport.BROADCAST, is_source=False,
                                        is_target=True, src_rank=primary, dst_ranks=wire, chunk_shape=route.shape, src_idx=cell,
                                        dst_idx=tuple(a for a, _ in box), dst_tensor=target_tensor, dst_index=sl(box),
                                        transfer_dtype=transfer_dtype, family=fam, tensor_id=tensor_id, route_id=route_id))
    return chunks
