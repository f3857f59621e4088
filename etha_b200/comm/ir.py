"""Plan structures shared by the planner, the specializer and every executor.

Two layers live here:

* the *pair-level* plan (`Endpoint`, `Route`, `M2MMap`) — shape independent, serialisable with
  msgspec as JSON or msgpack, field for field the plan format of the reference
  (src/etha/comm/ir.py:16-48, src/etha/comm/transfer.py:11-17), so plans can be exchanged
  with it;
* the *batch-level* descriptors (`Chunk`, `Bucket`) used by the bucket executors (gloo on CPU,
  NCCL as the baseline on GPUs).  The peer-to-peer executor does not use buckets: it lowers
  chunks to a device-resident copy table (see `etha_b200.comm.table`).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Sequence

import msgspec
import torch


class Transport(Enum):
    """How the bytes of one route reach their consumers."""

    P2P = "p2p"  # one consumer rank
    BROADCAST = "broadcast"  # several consumer ranks get the same cell
    LOCAL = "local"  # producer and consumer are the same rank: a device-local copy
    NONE = "none"  # reduce-only participant of a Partial source; ships nothing itself


class Endpoint(msgspec.Struct, frozen=True):
    """A rank together with the multi-index of one cell of that rank's local shard."""

    rank: int
    cell: tuple[int, ...]


class Route(msgspec.Struct, frozen=True):
    """Delivery of one source cell: where it lives and every place it has to land."""

    src: Endpoint
    dsts: tuple[Endpoint, ...]
    kind: Transport


class M2MMap(msgspec.Struct):
    """Mesh-to-mesh plan for one (source layout, target layout) pair.

    `routes` is sorted by `(src.rank, src.cell)`.  `source_num_slicers[d]` / `target_num_slicers[d]`
    say into how many equal pieces each side cuts dimension `d` of its *local* shard.
    `source_partial_reductions` lists `(mesh_dim, reduce_op)` for every `Partial` source mesh dim.
    """

    routes: list[Route] | None = None
    source_num_slicers: list[int] | None = None
    target_num_slicers: list[int] | None = None
    source_partial_reductions: list[tuple[int, str]] = []

    def to_json(self) -> bytes:
        return msgspec.json.encode(self)

    def to_msgpack(self) -> bytes:
        return msgspec.msgpack.encode(self)

    @classmethod
    def from_json(cls, data: bytes | str) -> "M2MMap":
        return msgspec.json.decode(data, type=cls)

    @classmethod
    def from_msgpack(cls, data: bytes) -> "M2MMap":
        return msgspec.msgpack.decode(data, type=cls)


REDUCE_OPS = ("sum", "avg", "max", "min", "product")


def route_kind(num_dsts: int) -> Transport:
    if num_dsts == 0:
        return Transport.NONE
    return Transport.P2P if num_dsts == 1 else Transport.BROADCAST


# --------------------------------------------------------------------------------------
# Partial families
# --------------------------------------------------------------------------------------


@dataclass(frozen=True)
class PartialFamily:
    """The ranks whose local values must be combined to materialise one rank's Partial shard.

    `ranks` is laid out with the *first* listed Partial mesh dim varying fastest, so that the
    sequential "reduce over mesh dim a, then over mesh dim b" of DTensor's Partial -> Replicate
    becomes: reduce groups of `sizes[0]` consecutive entries with `ops[0]`, then groups of
    `sizes[1]` of those results with `ops[1]`, and so on.
    """

    ranks: tuple[int, ...]
    sizes: tuple[int, ...]
    ops: tuple[str, ...]


def partial_family(mesh: torch.Tensor, reductions: Sequence[tuple[int, str]], rank: int) -> PartialFamily | None:
    """Family of `rank` on `mesh` for the Partial mesh dims in `reductions` (None if no Partial)."""
    if not reductions:
        return None
    mesh = torch.as_tensor(mesh)
    pos = (mesh == rank).nonzero()
    if pos.numel() == 0:
        raise ValueError(f"rank {rank} is not on the mesh")
    coord = pos[0].tolist()
    dims = [d for d, _ in reductions]
    index: list = list(coord)
    for d in dims:
        index[d] = slice(None)
    sub = mesh[tuple(index)]  # dims ordered as in the mesh, restricted to the partial dims
    # reorder so that the first listed partial dim is the fastest varying one
    order = sorted(range(len(dims)), key=lambda i: dims[i])  # position of each listed dim inside `sub`
    pos_in_sub = {dims[i]: k for k, i in enumerate(order)}
    perm = [pos_in_sub[d] for d in reversed(dims)]
    ranks = tuple(int(r) for r in sub.permute(perm).reshape(-1).tolist())
    return PartialFamily(ranks=ranks, sizes=tuple(int(mesh.shape[d]) for d in dims), ops=tuple(op for _, op in reductions))


def reduce_family_values(values: Sequence[torch.Tensor], family: PartialFamily, out_dtype: torch.dtype) -> torch.Tensor:
    """Reference arithmetic of the Partial collapse, shared by the CPU executor and the kernel tests.

    Floating inputs are accumulated in fp32 (fp64 stays fp64) in ascending family order, one level
    per Partial mesh dim, and rounded once to `out_dtype` — callers pass the source dtype, the dtype a
    Partial -> Replicate redistribution yields, and convert to the wire / target dtype afterwards.
    Integer inputs accumulate in int64.
    """
    src_dtype = values[0].dtype
    if src_dtype == torch.float64:
        acc_dtype = torch.float64
    elif src_dtype.is_floating_point:
        acc_dtype = torch.float32
    else:
        acc_dtype = torch.int64
    level = [v.to(acc_dtype) for v in values]
    for size, op in zip(family.sizes, family.ops):
        nxt = []
        for g in range(0, len(level), size):
            acc = level[g].clone()
            for v in level[g + 1 : g + size]:
                if op in ("sum", "avg"):
                    acc += v
                elif op == "max":
                    acc = torch.maximum(acc, v)
                elif op == "min":
                    acc = torch.minimum(acc, v)
                elif op == "product":
                    acc *= v
                else:
                    raise ValueError(f"unknown reduce op {op!r}")
            if op == "avg":
                acc = acc / size if acc_dtype.is_floating_point else acc // size
            nxt.append(acc)
        level = nxt
    assert len(level) == 1
    return level[0].to(out_dtype)


# --------------------------------------------------------------------------------------
# Batch-level descriptors
# --------------------------------------------------------------------------------------


@dataclass(slots=True, kw_only=True)
class Chunk:
    """One cell of one registered tensor, seen from one rank.

    A chunk may produce (`is_source`: this rank reads `src_index` of `src_tensor`), consume
    (`is_target`: this rank writes `dst_index` of `dst_tensor`) or both (`Transport.LOCAL`).
    `contributes_to` is set on the members of a Partial family that are not the route's primary:
    they hand their cell to the primary and ship nothing to the consumers.
    Counterpart of the reference's Chunk (src/etha/comm/ir.py:60-169), with the source and the
    target tensor kept apart so that a rank holding both roles never reads the wrong storage.
    """

    transport: Transport
    is_source: bool
    is_target: bool
    src_rank: int
    dst_ranks: tuple[int, ...]
    chunk_shape: tuple[int, ...]
    src_idx: tuple[int, ...]
    dst_idx: tuple[int, ...] | None = None
    src_tensor: torch.Tensor | None = None
    dst_tensor: torch.Tensor | None = None
    src_index: tuple[slice, ...] = ()
    dst_index: tuple[slice, ...] = ()
    transfer_dtype: torch.dtype | None = None
    family: PartialFamily | None = None  # set on the primary (and on contributors) of a Partial route
    contributes_to: int | None = None  # primary rank this reduce-only chunk feeds
    tensor_id: int = 0
    route_id: int = 0

    def __post_init__(self) -> None:
        if self.transfer_dtype is None:
            t = self.src_tensor if self.src_tensor is not None else self.dst_tensor
            self.transfer_dtype = t.dtype if t is not None else None

    @property
    def tensor(self) -> torch.Tensor | None:
        """The tensor this rank touches for the chunk (source side first)."""
        return self.src_tensor if self.src_tensor is not None else self.dst_tensor

    @property
    def numel(self) -> int:
        return math.prod(self.chunk_shape)

    @property
    def nbytes(self) -> int:
        """Bytes on the wire (transfer dtype)."""
        return self.numel * self.transfer_dtype.itemsize

    @property
    def bucket_key(self) -> tuple:
        """Chunks with equal keys may share one wire message."""
        return (self.src_rank, self.dst_ranks, self.contributes_to, self.transport, self.family is not None)

    def src_view(self) -> torch.Tensor:
        return self.src_tensor[self.src_index]

    def dst_view(self) -> torch.Tensor:
        return self.dst_tensor[self.dst_index]

    def __repr__(self) -> str:
        role = ("S" if self.is_source else "") + ("T" if self.is_target else "") or "-"
        return (
            f"Chunk({self.transport.value}/{role} t{self.tensor_id} {self.src_rank}{list(self.src_idx)}"
            f"->{list(self.dst_ranks)} shape={list(self.chunk_shape)})"
        )


@dataclass(slots=True, kw_only=True)
class Bucket:
    """Chunks that travel as one message between the same producer and consumers.

    Same role as the reference's Bucket (src/etha/comm/ir.py:172-310); the execution methods live in
    the executors, the bucket itself only carries layout (`offsets`, `total_bytes`).
    """

    chunks: list[Chunk]
    device: torch.device | None = None
    offsets: list[int] = field(init=False)
    total_bytes: int = field(init=False)

    def __post_init__(self) -> None:
        cursor = 0
        self.offsets = []
        for c in self.chunks:
            # keep every chunk 16-byte aligned inside the staging buffer so views of any dtype are legal
            cursor = (cursor + 15) & ~15
            self.offsets.append(cursor)
            cursor += c.nbytes
        self.total_bytes = cursor

    @property
    def head(self) -> Chunk:
        return self.chunks[0]

    @property
    def transport(self) -> Transport:
        return self.head.transport

    @property
    def is_source(self) -> bool:
        return self.head.is_source

    @property
    def is_target(self) -> bool:
        return self.head.is_target

    @property
    def src_rank(self) -> int:
        return self.head.src_rank

    @property
    def dst_ranks(self) -> tuple[int, ...]:
        return self.head.dst_ranks

    @property
    def key(self) -> tuple:
        return self.head.bucket_key

    def __repr__(self) -> str:
        return f"Bucket({self.transport.value} n={len(self.chunks)} {self.src_rank}->{list(self.dst_ranks)} {self.total_bytes}B)"
