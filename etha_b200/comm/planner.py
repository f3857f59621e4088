"""Pair-level planner: (source mesh, placements) x (target mesh, placements) -> `M2MMap`.

The reference derives the map by *tracing*: it pushes a tensor of encoded cell ids through
`distribute_tensor`/`full_tensor` and a round of sends (src/etha/comm/get_m2m_map.py:117-265).
This planner computes the same map in closed form, with no collective, no process group and no
DTensor call, so it also works for a rank that sits on both meshes and it costs microseconds.

Model.  Per tensor dimension `d` a side cuts the tensor into `shards[d]` equal pieces (the product
of the sizes of the mesh dims that carry `Shard(d)`; mesh dims listed first are the outer cut).
Both sides are refined to the common grid `grid[d] = lcm(source shards, target shards)`; one cell of
that grid is the unit of transfer.  A rank's local shard then holds `grid[d] / shards[d]` cells
along `d` (`*_num_slicers`).  Target rank number `j` (row-major position on the target mesh) takes
every cell it needs from the replica family of source rank number `j mod S` — the same spreading
rule as the reference's trace (src/etha/comm/get_m2m_map.py:194-206).
"""

from __future__ import annotations

import itertools
import math
from typing import Any, Sequence

import torch
from torch.distributed.tensor.placement_types import Partial, Placement, Replicate, Shard

from .ir import Endpoint, M2MMap, Route, route_kind

__all__ = ["plan_m2m", "get_m2m_map", "mesh_tensor_of", "shard_counts", "tensor_ndim_of"]


def mesh_tensor_of(mesh: Any) -> torch.Tensor:
    """Accept a `DeviceMesh`, a tensor or nested lists of global ranks."""
    inner = getattr(mesh, "mesh", None)
    if inner is not None:
        return torch.as_tensor(inner).cpu().to(torch.int64)
    t = torch.as_tensor(mesh).to(torch.int64)
    return t.reshape(1) if t.dim() == 0 else t


try:  # a private DTensor placement; since torch 2.11 it is no longer a subclass of Shard
    from torch.distributed.tensor.placement_types import _StridedShard
except ImportError:  # pragma: no cover
    _StridedShard = ()


def is_strided_shard(p: Placement) -> bool:
    return bool(_StridedShard) and isinstance(p, _StridedShard)


def shards_dim(p: Placement) -> int | None:
    """Tensor dim a placement cuts (`Shard` or `_StridedShard`), else None."""
    return p.dim if isinstance(p, Shard) or is_strided_shard(p) else None


def _check_placements(placements: Sequence[Placement], mesh: torch.Tensor, side: str, allow_strided: bool = False) -> None:
    if len(placements) != mesh.dim():
        raise ValueError(f"{side}: {len(placements)} placements for a {mesh.dim()}-d mesh")
    for i, p in enumerate(placements):
        if is_strided_shard(p):
            if not allow_strided:
                raise NotImplementedError(
                    f"{side}: {p!r} has no shape-independent plan; use the explicit-box planner "
                    "(etha_b200.comm.shaped.plan_for_shape, or a PairLayout in a P2PBatch, which selects it itself)")
            # `_StridedShard(d, split_factor=f)` on mesh dim i says: dim d was cut FIRST by later mesh dims of total
            # size f (e.g. tensor parallel), and only then by mesh dim i (e.g. FSDP).  The local shard is one
            # contiguous box exactly when the later mesh dims that shard d multiply to f; other combinations give a
            # strided union of pieces, which a box plan cannot express.
            later = 1
            for size, q in zip(mesh.shape[i + 1:], placements[i + 1:]):
                if shards_dim(q) == p.dim:
                    later *= int(size)
            if later != p.split_factor:
                raise NotImplementedError(
                    f"{side}: {p!r} on mesh dim {i} needs later mesh dims sharding dim {p.dim} of total size "
                    f"{p.split_factor}, found {later}: the local shard would not be a contiguous box")
            continue
        if not isinstance(p, (Shard, Replicate, Partial)):
            raise NotImplementedError(f"{side}: placement {p!r} is not supported (Shard, Replicate, Partial, _StridedShard only)")


def tensor_ndim_of(*placement_lists: Sequence[Placement]) -> int:
    """Number of leading tensor dims the plan has to know about: highest Shard dim + 1 (at least 1)."""
    dims = [p.dim for pl in placement_lists for p in pl if isinstance(p, Shard)]
    if any(d < 0 for d in dims):
        raise ValueError("negative Shard dims must be normalised before planning")
    return max(dims, default=0) + 1


def shard_counts(mesh_shape: Sequence[int], placements: Sequence[Placement], ndim: int) -> list[int]:
    counts = [1] * ndim
    for size, p in zip(mesh_shape, placements):
        if isinstance(p, Shard):
            counts[p.dim] *= int(size)
    return counts


def _shard_index(coord: Sequence[int], mesh_shape: Sequence[int], placements: Sequence[Placement], ndim: int) -> list[int]:
    """Which of the `shards[d]` pieces the rank at mesh coordinate `coord` owns, per tensor dim."""
    idx = [0] * ndim
    for c, size, p in zip(coord, mesh_shape, placements):
        if isinstance(p, Shard):
            idx[p.dim] = idx[p.dim] * int(size) + int(c)
    return idx


def _coord_for_shard_index(
    piece: Sequence[int], base_coord: Sequence[int], mesh_shape: Sequence[int], placements: Sequence[Placement]
) -> list[int]:
    """Inverse of `_shard_index`: mesh coordinate owning `piece`, non-Shard coordinates taken from `base_coord`."""
    coord = list(base_coord)
    rest = list(piece)
    for m in reversed(range(len(mesh_shape))):
        p = placements[m]
        if isinstance(p, Shard):
            size = int(mesh_shape[m])
            coord[m] = rest[p.dim] % size
            rest[p.dim] //= size
    return coord


def plan_m2m(
    source_mesh: Any,
    source_placements: Sequence[Placement],
    target_mesh: Any,
    target_placements: Sequence[Placement],
) -> M2MMap:
    """Closed-form mesh-to-mesh plan.  Pure function of its arguments; every rank gets the same map."""
    smesh = mesh_tensor_of(source_mesh)
    tmesh = mesh_tensor_of(target_mesh)
    source_placements = tuple(source_placements)
    target_placements = tuple(target_placements)
    _check_placements(source_placements, smesh, "source")
    _check_placements(target_placements, tmesh, "target")
    if any(isinstance(p, Partial) for p in target_placements):
        raise NotImplementedError(
            f"Partial in target placements {target_placements} is not supported: how a tensor splits into "
            "pending contributions on an independent process group is not defined. Partial is a source-only placement."
        )

    reductions = [(i, p.reduce_op) for i, p in enumerate(source_placements) if isinstance(p, Partial)]
    ndim = tensor_ndim_of(source_placements, target_placements)
    sshape, tshape = tuple(smesh.shape), tuple(tmesh.shape)
    s_counts = shard_counts(sshape, source_placements, ndim)
    t_counts = shard_counts(tshape, target_placements, ndim)
    grid = [math.lcm(a, b) for a, b in zip(s_counts, t_counts)]
    s_slicers = [g // a for g, a in zip(grid, s_counts)]
    t_slicers = [g // b for g, b in zip(grid, t_counts)]

    s_flat = smesh.reshape(-1).tolist()
    t_flat = tmesh.reshape(-1).tolist()
    s_coords = list(itertools.product(*[range(n) for n in sshape]))
    t_coords = list(itertools.product(*[range(n) for n in tshape]))
    n_src = len(s_flat)

    # (src_rank, src_cell) -> [(dst_rank, dst_cell)], consumers appended in target-mesh order
    table: dict[tuple[int, tuple[int, ...]], list[Endpoint]] = {}
    cells_of_target = list(itertools.product(*[range(n) for n in t_slicers]))
    for j, (t_rank, t_coord) in enumerate(zip(t_flat, t_coords)):
        family_coord = s_coords[j % n_src]
        t_piece = _shard_index(t_coord, tshape, target_placements, ndim)
        for t_cell in cells_of_target:
            g = [t_piece[d] * t_slicers[d] + t_cell[d] for d in range(ndim)]
            s_piece = [g[d] // s_slicers[d] for d in range(ndim)]
            s_cell = tuple(g[d] % s_slicers[d] for d in range(ndim))
            s_coord = _coord_for_shard_index(s_piece, family_coord, sshape, source_placements)
            s_rank = int(smesh[tuple(s_coord)])
            table.setdefault((s_rank, s_cell), []).append(Endpoint(rank=int(t_rank), cell=tuple(t_cell)))

    # consumers of one cell are listed in ascending rank order, as a gather over a rank-ordered group yields
    for key in table:
        table[key].sort(key=lambda e: e.rank)

    # Reduce-only entries: every member of a Partial family owns a (possibly empty) route for every
    # cell that any member of the family ships (reference: src/etha/comm/get_m2m_map.py:63-114).
    if reductions:
        partial_dims = [d for d, _ in reductions]
        rank_coord = {int(r): c for r, c in zip(s_flat, s_coords)}
        family_of: dict[int, tuple[int, ...]] = {}
        for r, c in rank_coord.items():
            index: list = list(c)
            for d in partial_dims:
                index[d] = slice(None)
            family_of[r] = tuple(int(x) for x in smesh[tuple(index)].reshape(-1).tolist())
        for (s_rank, s_cell) in list(table):
            for member in family_of[s_rank]:
                table.setdefault((member, s_cell), [])

    routes = [
        Route(src=Endpoint(rank=r, cell=c), dsts=tuple(dsts), kind=route_kind(len(dsts)))
        for (r, c), dsts in sorted(table.items(), key=lambda kv: kv[0])
    ]
    return M2MMap(
        routes=routes,
        source_num_slicers=s_slicers,
        target_num_slicers=t_slicers,
        source_partial_reductions=reductions,
    )


def get_m2m_map(
    source_mesh: Any,
    source_placements: Sequence[Placement],
    target_mesh: Any,
    target_placements: Sequence[Placement],
    group: Any = None,
    device: str = "cpu",
) -> M2MMap:
    """Signature-compatible entry point (reference: src/etha/comm/get_m2m_map.py:117-124).

    `group` and `device` exist for call compatibility only: the plan is computed locally, so no rank
    has to take part in a collective and callers need no lock-step discipline around this call.
    """
    del group, device
    return plan_m2m(source_mesh, source_placements, target_mesh, target_placements)
