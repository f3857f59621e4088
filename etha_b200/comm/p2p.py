"""Peer-to-peer executor: the plan is lowered to a device copy table and run by the sm_100a kernels.

Every producing rank reads its own shard and stores each cell straight into the consumers' strided
destination slices through peer pointers (no staging bucket, no pack/unpack, no NCCL call); a Replicate
target is served by one read and a store per replica (or one NVLS multicast store); a Partial source is
collapsed by the route's primary, which loads the other family members' pending values over NVLink,
accumulates in fp32 and stores the rounded result directly in the target layout.  Completion is
published by the last CTA of each producer to a flag on every consumer; consumers wait with a bounded
acquire-spin kernel, so no host barrier follows the transfer.

Replaces the reference's `bucket_comm` over NCCL (src/etha/comm/comm_methods.py:53-119, src/etha/comm/
ir.py:229-310, src/etha/comm/transfer.py:20-41).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch

from .. import ops
from ..ops.table import CopyTable, DEFAULT_TILE_BYTES
from ..parallel.peer import PeerMemory, TensorDesc
from ..utils.profiling import nvtx_range
from .chunks import cell_slices, chunk_shape_of, padded_slicers
from .ir import M2MMap, partial_family
from .planner import mesh_tensor_of, plan_m2m

__all__ = ["PairLayout", "P2PBatch", "TransferTimeout"]


class TransferTimeout(RuntimeError):
    """A consumer gave up waiting for a producer's completion flag."""


@dataclass
class PairLayout:
    """Source and target layouts of one pair; meshes hold global ranks."""

    source_mesh: Any
    source_placements: Sequence
    target_mesh: Any
    target_placements: Sequence
    global_shape: Sequence[int] | None = None  # set it (or leave it to be inferred) for unevenly sharded tensors
    _plan: M2MMap | None = None
    # no layout was declared: the k-th source rank sends its whole tensor to the k-th target rank (1-D rank lists)
    plain: bool = False

    def plan(self) -> M2MMap:
        if self._plan is None:
            self._plan = plan_m2m(self.source_mesh, self.source_placements, self.target_mesh, self.target_placements)
        return self._plan

    @property
    def source_ranks(self) -> list[int]:
        return mesh_tensor_of(self.source_mesh).reshape(-1).tolist()

    @property
    def target_ranks(self) -> list[int]:
        return mesh_tensor_of(self.target_mesh).reshape(-1).tolist()


def _single_process_exchange(obj):
    return [obj]


class P2PBatch:
    """All tensors of one registration, executed with one table launch per producing rank.

    `exchange(obj) -> list[obj]` is the only collective: it returns every participating rank's object in
    the order of `ranks` (e.g. `all_gather_object` on a gloo group).  In a single process that plays all
    ranks, pass several `P2PBatch` objects the same dictionary through `link_local`.
    """

    def __init__(
        self,
        rank: int,
        ranks: Sequence[int],
        device: torch.device | int | str,
        exchange: Callable[[Any], list[Any]] | None = None,
        peer: PeerMemory | None = None,
        tile_bytes: int = DEFAULT_TILE_BYTES,
        use_ipc: bool | None = None,
        nvls=None,
        dma_min_bytes: int | None = None,
        dma_mode: str = "graph",
        dma_fraction: float = 1.0,
    ):
        self.rank = rank
        self.ranks = list(ranks)
        self.device = torch.device(device) if not isinstance(device, torch.device) else device
        self.exchange = exchange or _single_process_exchange
        self.peer = peer or PeerMemory(self.device)
        self.use_ipc = (len(self.ranks) > 1) if use_ipc is None else use_ipc
        self.tile_bytes = tile_bytes
        # optional `NvlsTeam`: routes whose consumers are exactly the team, at one common arena offset, are written
        # with one multicast store instead of one store per replica
        self.nvls = nvls
        # copies of at least `dma_min_bytes` whose destination is on another GPU are run by the DMA engines (a CUDA
        # graph of memcpy nodes built once, launched per transfer); None keeps every copy in the kernels
        self.dma_min_bytes, self.dma_mode, self.dma_fraction = dma_min_bytes, dma_mode, dma_fraction
        self.multicast_ops = 0
        self.stripe_partial = True  # split the collapse of a Partial cell over the family members
        self._entries: list[tuple[PairLayout, torch.Tensor | None, torch.Tensor | None]] = []
        self.table: CopyTable | None = None
        self.epoch = 0
        self._built = False

    def add(self, layout: PairLayout, source: torch.Tensor | None = None, target: torch.Tensor | None = None) -> None:
        """Register the next tensor of the batch (same order on every rank)."""
        if self._built:
            raise RuntimeError("batch already built")
        self._entries.append((layout, source, target))

    # ---- build (collective) ---------------------------------------------------------------
    def _describe(self, t: torch.Tensor | None) -> TensorDesc | None:
        if t is None:
            return None
        return self.peer.describe(t) if self.use_ipc else self.peer.describe_local_only(t)

    def build(self) -> "P2PBatch":
        self._flags = torch.zeros(max(len(self.ranks), 1), dtype=torch.int32, device=self.device)
        self._status = torch.zeros(2, dtype=torch.int32, device=self.device)
        mine = {
            "rank": self.rank,
            "src": [self._describe(s) for _, s, _ in self._entries],
            "dst": [self._describe(t) for _, _, t in self._entries],
            "flags": self._describe(self._flags),
            "gpu": self._gpu_id(),
        }
        with nvtx_range("etha.p2p.exchange_descriptors"):
            everyone = self.exchange(mine)
        with nvtx_range("etha.p2p.build_table"):
            self._finish_build({e["rank"]: e for e in everyone})
        return self

    def _gpu_id(self) -> str:
        return str(torch.cuda.get_device_properties(self.device).uuid)

    def build_from(self, layouts: Sequence[PairLayout], by_rank: dict[int, dict], flags: torch.Tensor) -> "P2PBatch":
        """Build from descriptors gathered by the caller (the agent exchanges them through its KV store).

        `by_rank[r]` = `{"src": [TensorDesc | None, ...], "dst": [...], "flags": TensorDesc}` with one entry per
        tensor of the batch, in batch order; `flags` is this rank's own flag array (int32, one slot per rank of
        `ranks`), the tensor `by_rank[rank]["flags"]` describes.
        """
        self._entries = [(layout, None, None) for layout in layouts]
        self._flags = flags
        self._status = torch.zeros(2, dtype=torch.int32, device=self.device)
        with nvtx_range("etha.p2p.build_table"):
            self._finish_build(by_rank)
        return self

    def _finish_build(self, by_rank: dict[int, dict]) -> None:
        # this batch is one user of every peer allocation its descriptors live in (released by `close`)
        regions = {}
        for entry in by_rank.values():
            for d in list(entry.get("src") or []) + list(entry.get("dst") or []) + [entry.get("flags")]:
                if d is not None:
                    regions[(d.region.pid, d.region.handle, d.region.base)] = d.region
        retain = getattr(self.peer, "retain", None)
        self._retained = retain(regions.values()) if retain else []
        table = CopyTable(self.device, tile_bytes=self.tile_bytes, dma_min_bytes=getattr(self, "dma_min_bytes", None),
                          dma_mode=getattr(self, "dma_mode", "graph"), dma_fraction=getattr(self, "dma_fraction", 1.0))
        my_gpu = by_rank[self.rank].get("gpu") if self.rank in by_rank else None
        consumers_i_write: set[int] = set()
        producers_i_wait: set[int] = set()
        self._all_local = True  # every destination lies in this process's memory on this device
        for i, (layout, src, dst) in enumerate(self._entries):
            items = self._work_items(layout, i, by_rank)
            mine = []
            for executor, members, s_index, cshape, dst_list, fam in items:
                if executor == self.rank:
                    mine.append((members, s_index, cshape, dst_list, fam))
                # whoever writes into this rank's memory (itself included), or reads it as a Partial family member,
                # must be waited for
                if any(d_rank == self.rank for d_rank, _ in dst_list) or (executor != self.rank and self.rank in members):
                    producers_i_wait.add(executor)
            # Producers walk their table in order, so if every producer served consumer 0 first, then consumer 1, ...
            # all of them would pour into the same GPU at the same time and share its ingress.  Rotate: producer
            # number p starts with consumer p, then p+1, ... (a permutation schedule over the NVSwitch).
            s_ranks, t_ranks = layout.source_ranks, layout.target_ranks
            if self.rank in s_ranks and len(t_ranks) > 1 and not layout.plain:
                p, nt = s_ranks.index(self.rank), len(t_ranks)
                mine.sort(key=lambda t: min((t_ranks.index(r) - p) % nt for r, _ in t[3]))
            for members, s_index, cshape, dst_list, fam in mine:
                srcs = [self.peer.slice_ref(by_rank[q]["src"][i], s_index) for q in members]
                for q in members:
                    if q != self.rank:
                        consumers_i_write.add(q)  # tell the contributor when its shard has been read
                dsts = []
                all_remote = my_gpu is not None and len(members) == 1
                for d_rank, d_index in dst_list:
                    ddesc = by_rank[d_rank]["dst"][i]
                    dsts.append(self.peer.slice_ref(ddesc, d_index))
                    if ddesc.region.pid != self.peer.pid or ddesc.region.device_index != self.device.index:
                        self._all_local = False
                    if by_rank[d_rank].get("gpu") in (None, my_gpu):
                        all_remote = False  # this GPU's own memory: the kernels copy HBM to HBM faster than the DMA engines
                    consumers_i_write.add(d_rank)
                if not self._add_multicast(table, cshape, srcs, [r for r, _ in dst_list], by_rank, i, dsts, fam):
                    table.add(cshape, srcs, dsts, fam.sizes if fam else (), fam.ops if fam else (), dma_ok=all_remote)
        table.finalize()
        self.table = table
        # flags: slot k of a consumer's flag array belongs to producer ranks[k]
        my_slot = self.ranks.index(self.rank)
        addrs = []
        for c in sorted(consumers_i_write):
            fref = self.peer.slice_ref(by_rank[c]["flags"])
            addrs.append(fref.ptr + 4 * my_slot)
        self._signals = torch.tensor(addrs, dtype=torch.int64, device=self.device) if addrs else None
        self._consumers = sorted(consumers_i_write)
        self._producers = sorted(producers_i_wait)
        self._wait_slots = (
            torch.tensor([self.ranks.index(p) for p in self._producers], dtype=torch.int32, device=self.device)
            if self._producers else None
        )
        self._built = True

    def _work_items(self, layout: "PairLayout", i: int, by_rank: dict[int, dict]):
        """Every copy of tensor `i`, for all ranks: `(executing rank, source ranks, source slices, box shape,
        [(consumer, slices)], family)`.

        A plain route is executed by its producer.  Routes of a Partial source that collapse the same cell are merged
        into one fan-out, which is then cut into one stripe per family member along the first dimension that is long enough: member k collapses stripe k (reading the other members'
        stripes over NVLink, its own locally, always in family order, so the result does not depend on who computes
        it) and stores it into the consumers.  Every member then moves 1/F of the cell instead of the primary moving
        all of it while the others idle."""
        smesh = mesh_tensor_of(layout.source_mesh)
        reductions, transfers = self._transfers_of(layout, i, by_rank)
        items = []
        if not reductions:
            for primary, s_index, cshape, dst_list in transfers:
                items.append((primary, (primary,), s_index, tuple(cshape), dst_list, None))
            return items
        # Routes of a Partial source that collapse the same cell of the same family differ only in their consumer
        # (the planner gives every replica of a Replicate target its own primary).  They are merged: the cell is
        # collapsed once and the result stored into every consumer, so the contributors' shards cross NVLink once
        # instead of once per replica.
        merged: dict[tuple, list] = {}
        for primary, s_index, cshape, dst_list in transfers:
            fam = partial_family(smesh, reductions, primary)
            key = (fam.ranks, tuple((sl.start, sl.stop) for sl in s_index), tuple(cshape))
            if key in merged:
                merged[key][3].extend(dst_list)
            else:
                merged[key] = [primary, s_index, tuple(cshape), list(dst_list), fam]
        for primary, s_index, cshape, dst_list, fam in merged.values():
            sdesc = by_rank[primary]["src"][i]
            for q in fam.ranks:
                qdesc = by_rank[q]["src"][i]
                if qdesc is None or tuple(qdesc.shape) != tuple(sdesc.shape):
                    raise ValueError(f"Partial contributor {q} of tensor {i} has no matching shard")
            n_members = len(fam.ranks)
            dim = next((d for d, n in enumerate(cshape) if n >= n_members), None) if self.stripe_partial else None
            if dim is None or n_members == 1:
                items.append((primary, fam.ranks, s_index, cshape, dst_list, fam))
                continue
            extent = cshape[dim]
            for k, member in enumerate(fam.ranks):
                lo, hi = k * extent // n_members, (k + 1) * extent // n_members

                def cut(index, lo=lo, hi=hi):
                    index = list(index) + [slice(None)] * (len(cshape) - len(index))
                    start = index[dim].start or 0
                    index[dim] = slice(start + lo, start + hi)
                    return tuple(index)

                shape_k = tuple(hi - lo if d == dim else n for d, n in enumerate(cshape))
                items.append((member, fam.ranks, cut(s_index), shape_k, [(r, cut(ix)) for r, ix in dst_list], fam))
        return items

    def _transfers_of(self, layout: "PairLayout", i: int, by_rank: dict[int, dict]):
        """Normalised transfer list of tensor `i`: `(primary, source slices, box shape, [(consumer, slices), ...])`.

        Evenly divisible shards use the shape-independent lcm plan; anything else (or a layout that names its
        global shape) uses the explicit-box plan of `etha_b200.comm.shaped`."""
        s_ranks, t_ranks = layout.source_ranks, layout.target_ranks
        s_shapes = {r: tuple(by_rank[r]["src"][i].shape) for r in s_ranks if by_rank[r]["src"][i] is not None}
        t_shapes = {r: tuple(by_rank[r]["dst"][i].shape) for r in t_ranks if by_rank[r]["dst"][i] is not None}
        if len(s_shapes) != len(s_ranks) or len(t_shapes) != len(t_ranks):
            missing = [r for r in s_ranks if r not in s_shapes] + [r for r in t_ranks if r not in t_shapes]
            raise ValueError(f"tensor {i}: ranks {missing} registered no tensor for their side")
        if layout.plain:
            if len(s_ranks) != len(t_ranks):
                raise ValueError(f"tensor {i}: whole-tensor transfer needs equally many ranks on both sides")
            out = []
            for s, t in zip(s_ranks, t_ranks):
                if s_shapes[s] != t_shapes[t]:
                    raise ValueError(f"tensor {i}: rank {s} holds {s_shapes[s]} but its peer {t} expects {t_shapes[t]}")
                full = tuple(slice(0, n) for n in s_shapes[s])
                out.append((s, full, s_shapes[s], [(t, full)]))
            return [], out
        from .planner import is_strided_shard

        strided = any(is_strided_shard(p) for p in tuple(layout.source_placements) + tuple(layout.target_placements))
        m2m = None if strided else layout.plan()  # a strided shard has explicit boxes only
        out = []
        even = layout.global_shape is None and not strided
        if even:
            try:
                for route in m2m.routes:
                    if not route.dsts:
                        continue
                    sshape = s_shapes[route.src.rank]
                    s_cshape = chunk_shape_of(sshape, padded_slicers(m2m.source_num_slicers, len(sshape)))
                    dst_list = []
                    for d in route.dsts:
                        tshape = t_shapes[d.rank]
                        t_cshape = chunk_shape_of(tshape, padded_slicers(m2m.target_num_slicers, len(tshape)))
                        if tuple(t_cshape) != tuple(s_cshape):
                            raise ValueError(f"tensor {i}: cell shapes differ, source {s_cshape} vs target {t_cshape}")
                        dst_list.append((d.rank, cell_slices(d.cell, t_cshape, len(tshape))))
                    out.append((route.src.rank, cell_slices(route.src.cell, s_cshape, len(sshape)), tuple(s_cshape), dst_list))
                return list(m2m.source_partial_reductions or []), out
            except ValueError:
                out = []  # uneven shards: fall through to the explicit-box plan
        from .shaped import infer_global_shape, plan_for_shape

        gshape = layout.global_shape or infer_global_shape(layout.source_mesh, layout.source_placements, s_shapes)
        plan = plan_for_shape(layout.source_mesh, layout.source_placements, layout.target_mesh, layout.target_placements, gshape)
        sl = lambda box: tuple(slice(a, b) for a, b in box)
        for r in plan.routes:
            out.append((r.src_rank, sl(r.src_box), r.shape, [(d, sl(box)) for d, box in r.dsts]))
        return plan.source_partial_reductions, out

    def _add_multicast(self, table, shape, srcs, dst_ranks, by_rank, i, dsts, fam=None) -> bool:
        """Try to serve a fan-out route through the NVLS team; False means "use one store per replica"."""
        team = self.nvls
        if team is None or len(dsts) < getattr(self, "multicast_min_replicas", 2):
            return False
        if set(dst_ranks) != set(getattr(team, "replicas", None) or team.ranks):
            return False
        descs = [by_rank[r]["dst"][i] for r in dst_ranks]
        if any(dd.region.handle != b"vmm" for dd in descs):
            return False
        # same offset inside every member's arena, same strides and dtype: one multicast address serves all
        offs = set()
        for ref, dd in zip(dsts, descs):
            base = self.peer.map_region(dd.region)
            offs.add((ref.ptr - base, ref.strides, ref.dtype))
        if len(offs) != 1:
            return False
        off, strides, dtype = next(iter(offs))
        from ..ops.table import SliceRef

        mc = SliceRef(team.mc_va + off, strides, dtype, team.mc_va, team.mc_va + team.arena.size)
        try:
            table.add(shape, srcs, [mc], fam.sizes if fam else (), fam.ops if fam else (), multimem=True)
        except ValueError:
            return False  # not a 16-byte aligned bit copy: the packer refuses, fall back
        self.multicast_ops += 1
        return True

    # ---- execution -----------------------------------------------------------------------
    @property
    def is_producer(self) -> bool:
        return self.table is not None and (not self.table.empty or bool(self._consumers))

    @property
    def is_consumer(self) -> bool:
        return bool(self._producers)

    def begin(self) -> int:
        """Advance to the next transfer epoch (every rank calls it once per transfer)."""
        self.epoch += 1
        return self.epoch

    def send(self, stream: torch.cuda.Stream | None = None, ctas_per_sm: int = 2, bulk: bool = False,
             dma: bool | None = None) -> None:
        """Enqueue this rank's copies and the completion signal. Call `begin()` first.  `dma=False` keeps every copy
        in the kernels for this transfer even when the batch was built with a DMA plan."""
        if self.table is None:
            raise RuntimeError("build() first")
        if self._signals is None and self.table.empty:
            return
        # `bulk`: run the 16-byte bit copies through the TMA ring kernel (local loads, plain bulk stores to local or
        # peer memory) instead of the LD/ST kernel
        with nvtx_range("etha.p2p.launch_copies"):
            self.table.launch(stream, self._signals, self.epoch, ctas_per_sm=ctas_per_sm, bulk=bulk, dma=dma)

    def recv(self, stream: torch.cuda.Stream | None = None, timeout_s: float = 10.0) -> None:
        """Enqueue the bounded wait for every producer that writes into this rank."""
        if self._wait_slots is None:
            return
        with nvtx_range("etha.p2p.launch_wait"):
            ops.wait_flags(self._flags, self._wait_slots, self.epoch, self._status, timeout_s, stream)

    def check(self) -> None:
        """After a stream synchronize: raise if the wait timed out or a kernel reported a bad op."""
        if self._wait_slots is not None:
            st = self._status.tolist()
            if st[0] == ops.STATUS_TIMEOUT:
                who = self._producers[st[1]] if 0 <= st[1] < len(self._producers) else st[1]
                raise TransferTimeout(f"rank {self.rank}: no completion flag from producer rank {who} (epoch {self.epoch})")
        if self.table is not None and not self.table.empty and self.table.error_word() != 0:
            raise RuntimeError(f"rank {self.rank}: copy kernel reported error {self.table.error_word()}")

    def transfer(self, stream: torch.cuda.Stream | None = None, timeout_s: float = 10.0, **kw) -> None:
        """begin + send + recv for ranks that may hold either or both roles."""
        self.begin()
        self.send(stream, **kw)
        self.recv(stream, timeout_s)

    @property
    def payload_bytes(self) -> int:
        return self.table.payload_bytes if self.table is not None else 0

    def close(self) -> None:
        """Give up this batch's use of the peers' allocations (mappings no other batch uses are closed) and drop the
        copy table.  Call it only when none of the batch's kernels is in flight."""
        keys, self._retained = getattr(self, "_retained", []), []
        if keys:
            self.peer.release(keys)
        self.table = None
        self._signals = self._wait_slots = None
        self._built = False


def link_local(batches: Sequence[P2PBatch]) -> None:
    """Build several logical ranks that live in ONE process (tests, 1-GPU runs): no IPC, no collective."""
    gathered = []
    for b in batches:
        b.use_ipc = False
        b._flags = torch.zeros(max(len(b.ranks), 1), dtype=torch.int32, device=b.device)
        b._status = torch.zeros(2, dtype=torch.int32, device=b.device)
        gathered.append({
            "rank": b.rank,
            "gpu": b._gpu_id(),
            "src": [b._describe(s) for _, s, _ in b._entries],
            "dst": [b._describe(t) for _, _, t in b._entries],
            "flags": b._describe(b._flags),
        })
    by_rank = {e["rank"]: e for e in gathered}
    for b in batches:
        b._finish_build(by_rank)
