"""Batch-level specializer: an `M2MMap` plus this rank's local tensors -> `Chunk` descriptors.

Counterpart of the reference's `m2m_to_chunks` (src/etha/comm/get_chunks.py:22-128) with three
deliberate differences:

* a route whose consumers include the producing rank yields ONE chunk that both ships to the other
  consumers and writes the local destination (the reference emits a wire chunk addressed to itself
  plus a local chunk that reads the target tensor);
* a `Partial` source is described by a `PartialFamily` (who contributes, in which order) instead of
  process groups, so no executor has to create sub-groups;
* dimensions that do not divide evenly raise instead of silently dropping the remainder.
"""

from __future__ import annotations

from typing import Any, Sequence

import torch

from .ir import Chunk, M2MMap, PartialFamily, Transport, partial_family

__all__ = ["m2m_to_chunks", "cell_slices", "padded_slicers", "chunk_shape_of", "plan_fits_shapes"]


def padded_slicers(num_slicers: Sequence[int], ndim: int) -> list[int]:
    """Slicer counts extended with 1s (or cut) to the tensor's rank (reference: get_chunks.py:41,46)."""
    out = (list(num_slicers) + [1] * ndim)[:ndim]
    if any(n != 1 for n in list(num_slicers)[ndim:]):
        raise ValueError(f"plan cuts dims {list(num_slicers)} but the tensor has only {ndim} dims")
    return out


def chunk_shape_of(shape: Sequence[int], slicers: Sequence[int]) -> tuple[int, ...]:
    for d, (n, k) in enumerate(zip(shape, slicers)):
        if n % k:
            raise ValueError(
                f"dim {d} of local shape {tuple(shape)} is not divisible into {k} cells; "
                "uneven shards need the shape-aware planner (plan_for_shapes)"
            )
    return tuple(n // k for n, k in zip(shape, slicers))


def plan_fits_shapes(m2m: M2MMap, source_shapes: dict, target_shapes: dict) -> bool:
    """True if the lcm plan applies: every rank's local shape divides into its cells and all cells have one shape.

    Every rank must take this decision from the shapes of ALL ranks of both sides, otherwise a producer whose own
    shard happens to divide evenly and a consumer whose shard does not would pick different plans."""
    cell = None
    for shapes, slicers in ((source_shapes, m2m.source_num_slicers), (target_shapes, m2m.target_num_slicers)):
        for shape in shapes.values():
            try:
                c = chunk_shape_of(shape, padded_slicers(slicers, len(shape)))
            except ValueError:
                return False
            if cell is not None and tuple(c) != tuple(cell):
                return False
            cell = c
    return True


def cell_slices(cell: Sequence[int], cshape: Sequence[int], ndim: int) -> tuple[slice, ...]:
    cell = (tuple(cell) + (0,) * ndim)[:ndim]
    return tuple(slice(c * n, (c + 1) * n) for c, n in zip(cell, cshape))


def _family_from_groups(groups: Any, reductions: Sequence[tuple[int, str]]) -> PartialFamily | None:
    """Family from reference-style `[(group_or_ranks, op)]`; enough information only for one Partial dim."""
    if not groups:
        return None
    if len(groups) != 1 or len(reductions) != 1:
        raise ValueError("several Partial mesh dims need source_mesh= to enumerate the contributing ranks")
    g, op = groups[0]
    if isinstance(g, (list, tuple)):
        ranks = tuple(int(r) for r in g)
    else:
        import torch.distributed as dist

        ranks = tuple(dist.get_process_group_ranks(g))
    return PartialFamily(ranks=ranks, sizes=(len(ranks),), ops=(op,))


def m2m_to_chunks(
    m2m: M2MMap,
    rank: int,
    source_tensor: torch.Tensor | None = None,
    target_tensor: torch.Tensor | None = None,
    transfer_dtype: torch.dtype | None = None,
    source_partial_groups: Any = None,
    *,
    source_mesh: Any = None,
    tensor_id: int = 0,
) -> list[Chunk]:
    """Chunks of one tensor for `rank`, in canonical route order.

    `source_tensor` is this rank's local shard when it is a producer, `target_tensor` its local shard
    when it is a consumer; a rank on both meshes passes both.  With a `Partial` source pass
    `source_mesh` (tensor or DeviceMesh of global ranks); `source_partial_groups` is accepted for
    call compatibility and is sufficient only for a single Partial mesh dim.
    """
    routes = m2m.routes
    if not routes:
        return []
    reductions = list(m2m.source_partial_reductions or [])

    s_slicers = s_cshape = t_slicers = t_cshape = None
    if source_tensor is not None:
        s_slicers = padded_slicers(m2m.source_num_slicers, source_tensor.dim())
        s_cshape = chunk_shape_of(source_tensor.shape, s_slicers)
    if target_tensor is not None:
        t_slicers = padded_slicers(m2m.target_num_slicers, target_tensor.dim())
        t_cshape = chunk_shape_of(target_tensor.shape, t_slicers)

    families: dict[int, PartialFamily | None] = {}

    def family_of(primary: int) -> PartialFamily | None:
        if not reductions:
            return None
        if primary not in families:
            if source_mesh is not None:
                from .planner import mesh_tensor_of

                families[primary] = partial_family(mesh_tensor_of(source_mesh), reductions, primary)
            else:
                fam = _family_from_groups(source_partial_groups, reductions)
                if fam is None:
                    raise ValueError("Partial source: pass source_mesh= (or source_partial_groups for one Partial dim)")
                if primary not in fam.ranks:
                    raise ValueError(f"route primary {primary} is outside the given Partial group {fam.ranks}")
                families[primary] = fam
        return families[primary]

    chunks: list[Chunk] = []
    for route_id, route in enumerate(routes):
        if not route.dsts:
            continue  # reduce-only entries are implied by the primary's family
        primary = route.src.rank
        src_cell = route.src.cell
        fam = family_of(primary)
        wire_dsts = tuple(sorted({d.rank for d in route.dsts if d.rank != primary}))
        local_dst = next((d for d in route.dsts if d.rank == primary), None)

        if primary == rank:
            if source_tensor is None:
                raise ValueError(f"rank {rank} produces route {route_id} but no source_tensor was given")
            ndim = source_tensor.dim()
            c = Chunk(
                transport=Transport.LOCAL if not wire_dsts else (Transport.P2P if len(wire_dsts) == 1 else Transport.BROADCAST),
                is_source=True,
                is_target=local_dst is not None,
                src_rank=primary,
                dst_ranks=wire_dsts,
                chunk_shape=s_cshape,
                src_idx=tuple(src_cell),
                src_tensor=source_tensor,
                src_index=cell_slices(src_cell, s_cshape, ndim),
                transfer_dtype=transfer_dtype,
                family=fam,
                tensor_id=tensor_id,
                route_id=route_id,
            )
            if local_dst is not None:
                if target_tensor is None:
                    raise ValueError(f"rank {rank} consumes its own route {route_id} but no target_tensor was given")
                c.dst_idx = tuple(local_dst.cell)
                c.dst_tensor = target_tensor
                c.dst_index = cell_slices(local_dst.cell, t_cshape, target_tensor.dim())
                if t_cshape != s_cshape:
                    raise ValueError(f"cell shapes differ between sides: {s_cshape} vs {t_cshape}")
            chunks.append(c)
        elif fam is not None and rank in fam.ranks and source_tensor is not None:
            # this rank only contributes its pending value of the cell to the primary
            ndim = source_tensor.dim()
            chunks.append(
                Chunk(
                    transport=Transport.NONE,
                    is_source=True,
                    is_target=False,
                    src_rank=primary,
                    dst_ranks=wire_dsts,
                    chunk_shape=s_cshape,
                    src_idx=tuple(src_cell),
                    src_tensor=source_tensor,
                    src_index=cell_slices(src_cell, s_cshape, ndim),
                    transfer_dtype=transfer_dtype,
                    family=fam,
                    contributes_to=primary,
                    tensor_id=tensor_id,
                    route_id=route_id,
                )
            )

        if primary != rank:
            for d in route.dsts:
                if d.rank != rank:
                    continue
                if target_tensor is None:
                    raise ValueError(f"rank {rank} consumes route {route_id} but no target_tensor was given")
                chunks.append(
                    Chunk(
                        transport=Transport.P2P if len(wire_dsts) == 1 else Transport.BROADCAST,
                        is_source=False,
                        is_target=True,
                        src_rank=primary,
                        dst_ranks=wire_dsts,
                        chunk_shape=t_cshape,
                        src_idx=tuple(src_cell),
                        dst_idx=tuple(d.cell),
                        dst_tensor=target_tensor,
                        dst_index=cell_slices(d.cell, t_cshape, target_tensor.dim()),
                        transfer_dtype=transfer_dtype,
                        family=fam,
                        tensor_id=tensor_id,
                        route_id=route_id,
                    )
                )
    return chunks
