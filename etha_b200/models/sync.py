"""Whole-model weight sync between a trainer layout and an inference layout on one NVLink domain.

`WeightSync` materialises this rank's shards of every parameter of a `ModelSpec` (random-init, seeded
per tensor so that any rank can regenerate any slice for verification), registers them as one
`P2PBatch` and exposes `sync()`.  It stands in for the reference's trainer / vLLM worker pair
(examples/vllm_weight_sync/trainer.py:173-249, examples/vllm_weight_sync/vllm_server.py:198-325) with a
fake consumer that only holds vLLM's tensor-parallel layout.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch
from torch.distributed.tensor._utils import _compute_local_shape_and_global_offset
from torch.distributed.tensor.placement_types import Partial, Replicate

from ..comm.p2p import P2PBatch, PairLayout
from ..comm.planner import mesh_tensor_of
from .catalog import LayoutRule, ModelSpec, TensorSpec

__all__ = ["WeightSync", "local_shape_and_offset", "full_tensor_for"]


def local_shape_and_offset(shape, mesh: torch.Tensor, placements, rank: int):
    coord = (mesh == rank).nonzero()[0].tolist()
    eff = tuple(Replicate() if isinstance(p, Partial) else p for p in placements)
    return _compute_local_shape_and_global_offset(tuple(shape), tuple(mesh.shape), coord, eff)


def full_tensor_for(spec: TensorSpec, index: int, seed: int, dtype: torch.dtype, device) -> torch.Tensor:
    """The logical (global) value of parameter `index`: randn * 0.02 from a per-tensor seed."""
    g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + index)
    return (torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Arena:
    """One allocation holding many tensors, so that a rank exports a single IPC handle per side."""

    def __init__(self, sizes_bytes: Sequence[int], device):
        offs, cur = [], 0
        for n in sizes_bytes:
            offs.append(cur)
            cur += _align(n)
        self.offsets = offs
        self.buffer = torch.empty(max(cur, 256), dtype=torch.uint8, device=device)

    def view(self, k: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * dtype.itemsize
        return self.buffer.narrow(0, self.offsets[k], nbytes).view(dtype).view(tuple(shape))


@dataclass
class _Entry:
    spec: TensorSpec
    layout: PairLayout
    source: torch.Tensor | None
    target: torch.Tensor | None


class WeightSync:
    def __init__(
        self,
        model: ModelSpec,
        rank: int,
        ranks: Sequence[int],
        device,
        source_mesh: Any,
        target_mesh: Any,
        source_rule: LayoutRule,
        target_rule: LayoutRule,
        exchange: Callable[[Any], list[Any]] | None = None,
        source_dtype: torch.dtype = torch.bfloat16,
        target_dtype: torch.dtype = torch.bfloat16,
        seed: int = 2,
        fill: bool = True,
        partial_scale: bool = True,
        extra: Sequence[tuple[torch.Tensor | None, torch.Tensor | None]] = (),
        tile_bytes: int | None = None,
        nvls: bool = False,
        nvls_tag: str = "ws",
        dma_min_bytes: int | None = None,
        dma_mode: str = "graph",
        dma_fraction: float = 1.0,
    ):
        self.model, self.rank, self.device, self.seed = model, rank, torch.device(device), seed
        self.smesh, self.tmesh = mesh_tensor_of(source_mesh), mesh_tensor_of(target_mesh)
        self.source_dtype, self.target_dtype = source_dtype, target_dtype
        self.is_source = rank in self.smesh.reshape(-1).tolist()
        self.is_target = rank in self.tmesh.reshape(-1).tolist()
        self.source_rule, self.target_rule = source_rule, target_rule

        layouts: dict[tuple, PairLayout] = {}
        s_shapes, t_shapes = [], []
        self.entries: list[_Entry] = []
        for t in model.tensors:
            sp, tp = tuple(source_rule(t)), tuple(target_rule(t))
            key = (sp, tp)
            if key not in layouts:
                layouts[key] = PairLayout(self.smesh, sp, self.tmesh, tp)
            s_shapes.append(local_shape_and_offset(t.shape, self.smesh, sp, rank)[0] if self.is_source else None)
            t_shapes.append(local_shape_and_offset(t.shape, self.tmesh, tp, rank)[0] if self.is_target else None)
            self.entries.append(_Entry(t, layouts[key], None, None))

        def nbytes(shape, dt):
            n = dt.itemsize
            for s in shape:
                n *= s
            return n

        if self.is_source:
            self.src_arena = _Arena([nbytes(s, source_dtype) for s in s_shapes], self.device)
            for k, e in enumerate(self.entries):
                e.source = self.src_arena.view(k, s_shapes[k], source_dtype)
        if self.is_target:
            self.dst_arena = _Arena([nbytes(s, target_dtype) for s in t_shapes], self.device)
            self.dst_arena.buffer.zero_()
            for k, e in enumerate(self.entries):
                e.target = self.dst_arena.view(k, t_shapes[k], target_dtype)
        # NVLS: parameters that every consumer holds in full live in a VMM arena bound to one multicast object, so
        # a producer writes all replicas with one store; every rank of the job is a team member (producers bind an
        # equally sized scratch arena, see etha_b200.parallel.arena)
        self.team = None
        peer = None
        if nvls:
            from ..parallel.arena import NvlsTeam, VmmArena
            from ..parallel.peer import PeerMemory

            rep = [k for k, e in enumerate(self.entries) if all(isinstance(p, Replicate) for p in e.layout.target_placements)]
            offs, cur = {}, 0
            for k in rep:
                offs[k] = cur
                cur += _align(nbytes(self.entries[k].spec.shape, target_dtype))
            if cur:
                peer = PeerMemory(self.device)
                self.rep_arena = VmmArena(cur, self.device, n_team=len(ranks))
                self.team = NvlsTeam(rank, list(ranks), self.rep_arena, nvls_tag, exchange, peer=peer)
                self.team.replicas = self.tmesh.reshape(-1).tolist()
                if self.is_target:
                    for k in rep:
                        t = self.rep_arena.tensor(offs[k], self.entries[k].spec.shape, target_dtype)
                        t.zero_()
                        self.entries[k].target = t
        self.scale = 1.0  # every source currently holds `scale` x its seeded value (see `rescale_sources`)
        if fill and self.is_source:
            self.fill_sources(partial_scale)

        kw = {} if tile_bytes is None else {"tile_bytes": tile_bytes}
        self.batch = P2PBatch(rank, ranks, self.device, exchange=exchange, peer=peer, nvls=self.team,
                              dma_min_bytes=dma_min_bytes, dma_mode=dma_mode, dma_fraction=dma_fraction, **kw)
        for e in self.entries:
            self.batch.add(e.layout, e.source, e.target)
        for layout, s, t in extra:
            self.batch.add(layout, s, t)
        self.payload_bytes = 0
        for t in model.tensors:
            tp = tuple(target_rule(t))
            copies = 1
            for size, p in zip(self.tmesh.shape, tp):
                if isinstance(p, Replicate):
                    copies *= size
            self.payload_bytes += nbytes(t.shape, target_dtype) * copies

    # ---- data -------------------------------------------------------------------------------
    def _partial_divisor(self, placements) -> int:
        n = 1
        for size, p in zip(self.smesh.shape, placements):
            if isinstance(p, Partial) and p.reduce_op == "sum":
                n *= size
        return n

    def fill_sources(self, partial_scale: bool = True) -> None:
        """Every source rank writes its shard of the seeded logical tensor; with a `Partial("sum")`
        mesh dim each contributor holds value / group size, so that the collapse restores the value
        exactly for power-of-two groups."""
        for k, e in enumerate(self.entries):
            full = full_tensor_for(e.spec, k, self.seed, torch.float32, self.device)
            div = self._partial_divisor(e.layout.source_placements) if partial_scale else 1
            if div > 1:
                full = full / div
            shape, off = local_shape_and_offset(e.spec.shape, self.smesh, e.layout.source_placements, self.rank)
            index = tuple(slice(o, o + n) for o, n in zip(off, shape))
            e.source.copy_(full[index].to(self.source_dtype))
            del full

    def rescale_sources(self, factor: float = 0.5) -> None:
        """Multiply every source shard by a power of two, in place on the device (exact in fp32/bf16/fp16 away from
        the subnormals), and remember it: `verify()` then expects the rescaled values.  A benchmark calls this after
        its warm-up, so that only transfers of the timed region can make the final `verify()` pass."""
        m, _ = __import__("math").frexp(factor)
        if m != 0.5:
            raise ValueError("factor must be a power of two")
        self.scale *= factor
        if self.is_source:
            for e in self.entries:
                e.source.mul_(factor)

    def verify(self) -> int:
        """Bit-exact check of every target shard against the regenerated logical tensors. Returns mismatching tensors."""
        bad = 0
        if not self.is_target:
            return 0
        for k, e in enumerate(self.entries):
            full = full_tensor_for(e.spec, k, self.seed, torch.float32, self.device) * self.scale
            div = self._partial_divisor(e.layout.source_placements)
            if div > 1:
                part = (full / div).to(self.source_dtype).to(torch.float32)
                full = part * div  # exact for power-of-two groups: sum of equal parts
            else:
                full = full.to(self.source_dtype)
            want = full.to(self.target_dtype)
            shape, off = local_shape_and_offset(e.spec.shape, self.tmesh, e.layout.target_placements, self.rank)
            index = tuple(slice(o, o + n) for o, n in zip(off, shape))
            if not torch.equal(e.target, want[index]):
                bad += 1
            del full, want
        return bad

    # ---- execution ------------------------------------------------------------------------
    def build(self) -> "WeightSync":
        self.batch.build()
        return self

    def sync(self, stream: torch.cuda.Stream | None = None, timeout_s: float = 10.0, **kw) -> None:
        """One full-model transfer: enqueue copies (producer role) and the bounded wait (consumer role)."""
        self.batch.transfer(stream, timeout_s, **kw)

    def check(self) -> None:
        self.batch.check()

    def close(self) -> None:
        """Release the multicast team and its arena (call on every rank before exit when `nvls=True`)."""
        if self.team is not None:
            torch.cuda.synchronize(self.device)
            self.team.close()
            self.rep_arena.close()
            self.team = None
