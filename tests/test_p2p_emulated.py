"""The peer-to-peer executor's lowering (plan -> per-rank copy tables -> flags) checked without a GPU.

Every logical rank gets a fake address range backed by a numpy buffer; each rank's `P2PBatch` is built from the
same descriptors it would receive over the control plane, and its packed ops are then interpreted on the host
exactly like the kernels walk them (see test_table_emulation).  The consumers' shards must come out equal to
DTensor's sharding of the logical tensor, every consumer byte written by exactly the producers the consumer
waits for.  Covers bit-copy routes: resharding, fan-out, overlapping meshes, uneven shards, producer rotation."""

import math

import numpy as np
import pytest
import torch
from torch.distributed.tensor.placement_types import Replicate, Shard, _StridedShard

from etha_b200.comm.baselines import local_slice_of
from etha_b200.comm.p2p import P2PBatch, PairLayout
from etha_b200.ops.table import CopyTable, SliceRef
from etha_b200.parallel.peer import RegionDesc, TensorDesc

from test_table_emulation import _emulate
from test_table_pack import OpView

R = Replicate()
REGION = 1 << 30


class World:
    """Fake NVLink domain: rank r owns addresses [(r+1)<<40, +REGION) backed by `mem[r]`."""

    def __init__(self, ranks):
        self.mem = {r: np.zeros(1 << 22, dtype=np.uint8) for r in ranks}
        self.cursor = {r: 256 for r in ranks}

    def base(self, r):
        return (r + 1) << 40

    def alloc(self, r, shape, dtype):
        n = int(np.prod(shape)) * dtype.itemsize
        off = self.cursor[r]
        self.cursor[r] = (off + n + 255) // 256 * 256
        t = torch.from_numpy(self.mem[r][off : off + max(n, 1)])[:n].view(dtype).view(tuple(shape))
        strides = tuple(t.stride())
        desc = TensorDesc(RegionDesc(1000 + r, r, self.base(r), REGION, b"fake"), off, tuple(shape), strides,
                          str(dtype).replace("torch.", ""))
        return t, desc

    def buffer_of(self, ptr):
        r = (ptr >> 40) - 1
        return r, self.mem[r], self.base(r)


class FakePeer:
    def __init__(self, pid):
        self.pid = pid

    def map_region(self, region):
        return region.base

    def slice_ref(self, desc, index=()):
        dt = desc.torch_dtype
        off = desc.offset
        for sl, st in zip(index, desc.strides):
            off += (sl.start or 0) * st * dt.itemsize
        return SliceRef(desc.region.base + off, desc.strides, dt, desc.region.base, desc.region.base + desc.region.size)


CASES = [
    ((4,), (Shard(0),), (4,), (Shard(1),), (64, 64)),
    ((4,), (Shard(0),), (4,), (R,), (32, 16)),
    ((4,), (R,), (4,), (Shard(0),), (32, 16)),
    ((1, 2, 2), (R, Shard(0), Shard(0)), (4,), (Shard(0),), (8, 16, 32)),
    ((2, 2), (Shard(0), Shard(1)), (2, 2), (Shard(1), Shard(0)), (64, 64)),
    ((2, 2), (R, Shard(0)), (2, 2), (R, Shard(0)), (8, 16)),
    ((3,), (Shard(0),), (2,), (Shard(1),), (12, 10)),
    ((2,), (Shard(0),), (2,), (Shard(1),), (1000, 333)),
    ((2,), (Shard(0),), (2,), (Shard(1),), (7, 4096)),
    ((2, 2), (Shard(0), Shard(1)), (3,), (Shard(0),), (10, 7)),
    ((4,), (Shard(0),), (2, 2), (_StridedShard(0, split_factor=2), Shard(0)), (32, 16)),
]


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_tables_of_all_ranks_deliver_every_shard(case, overlap, monkeypatch):
    _check_copy_case(case, overlap, monkeypatch)


def _check_copy_case(case, overlap, monkeypatch):
    ss, sp, ts, tp, shape = case
    ns, nt = math.prod(ss), math.prod(ts)
    smesh = torch.arange(ns).view(ss)
    t0 = 0 if overlap else ns
    tmesh = torch.arange(t0, t0 + nt).view(ts)
    ranks = sorted(set(smesh.reshape(-1).tolist()) | set(tmesh.reshape(-1).tolist()))
    world = World(ranks)
    g = torch.Generator().manual_seed(4)
    full = torch.randn(shape, generator=g).to(torch.bfloat16)
    by_rank = {r: {"rank": r, "src": [None], "dst": [None]} for r in ranks}
    targets = {}
    for r in ranks:
        if r in smesh.reshape(-1).tolist():
            t, desc = world.alloc(r, local_slice_of(full, smesh, sp, r).shape, torch.bfloat16)
            t.copy_(local_slice_of(full, smesh, sp, r))
            by_rank[r]["src"] = [desc]
        if r in tmesh.reshape(-1).tolist():
            t, desc = world.alloc(r, local_slice_of(full, tmesh, tp, r).shape, torch.bfloat16)
            by_rank[r]["dst"] = [desc]
            targets[r] = t
        _, by_rank[r]["flags"] = world.alloc(r, (len(ranks),), torch.int32)

    monkeypatch.setattr(CopyTable, "finalize", lambda self, sm_count=None: self)
    layout = PairLayout(smesh, sp, tmesh, tp)
    batches = {}
    for r in ranks:
        b = P2PBatch.__new__(P2PBatch)
        b.rank, b.ranks, b.device, b.peer = r, ranks, torch.device("cpu"), FakePeer(1000 + r)
        b.nvls, b.tile_bytes, b.multicast_ops, b.stripe_partial = None, 4096, 0, True
        b._entries = [(layout, None, None)]
        b._finish_build(by_rank)
        batches[r] = b

    writers = {r: set() for r in ranks}
    for r, b in batches.items():
        for cls, tiles, raw, *_ in b.table._packed:
            op = OpView.from_buffer_copy(raw)
            assert op.mode == 0 and op.nsrc == 1
            src_rank, src_buf, src_base = world.buffer_of(op.src[0])
            assert src_rank == r, "producers read their own memory only"
            for j in range(op.ndst):
                dst_rank, dst_buf, dst_base = world.buffer_of(op.dst[j])
                writers[dst_rank].add(r)
                single = OpView.from_buffer_copy(raw)
                single.ndst = 1
                single.dst[0] = op.dst[j]
                _emulate(single, src_buf, dst_buf, src_base, dst_base)
    for r, t in targets.items():
        assert torch.equal(t, local_slice_of(full, tmesh, tp, r)), f"rank {r}"
        assert set(batches[r]._producers) == writers[r], "a consumer waits exactly for the producers that write into it"
    for r, b in batches.items():
        assert set(b._consumers) == {c for c in ranks if r in writers[c]}
        # flag addresses: slot of this producer in every consumer's flag array
        if b._signals is not None:
            want = sorted(by_rank[c]["flags"].region.base + by_rank[c]["flags"].offset + 4 * ranks.index(r) for c in b._consumers)
            assert sorted(b._signals.tolist()) == want


# ---- typed ops: conversion and Partial collapse ---------------------------------------------------------------
from torch.distributed.tensor.placement_types import Partial  # noqa: E402

from etha_b200.comm.ir import PartialFamily, reduce_family_values  # noqa: E402
from test_reshard_cpu import _make_source_local  # noqa: E402

_CODE_DTYPE = {1: torch.float32, 2: torch.bfloat16, 3: torch.float16}
_RED_NAMES = {0: "sum", 1: "avg", 2: "max", 3: "min", 4: "product"}


def _emulate_typed(op: OpView, world: World):
    """Conversion / reduction ops, one unit of `unit_elems` elements at a time, same order of operations as the kernels."""
    sdt, ddt = _CODE_DTYPE[op.src_dtype], _CODE_DTYPE[op.dst_dtype]
    n = op.unit_elems
    fam = None
    if op.mode == 2:
        sizes = (op.red_size[0],) + ((op.red_size[1],) if op.red_size[1] > 1 else ())
        ops = (_RED_NAMES[op.red_op[0]],) + ((_RED_NAMES[op.red_op[1]],) if op.red_size[1] > 1 else ())
        fam = PartialFamily(ranks=tuple(range(op.nsrc)), sizes=sizes, ops=ops)
    from test_table_emulation import _fast_div

    for unit in range(op.total_units):
        q = _fast_div(unit, op.div_mul[4], op.div_shr[4])
        col = unit - q * op.inner_units
        so, do = col * op.unit_bytes_src, col * op.unit_bytes_dst
        for d in reversed(range(op.ndim)):
            q2 = 0 if d == 0 else _fast_div(q, op.div_mul[d], op.div_shr[d])
            i = q - q2 * op.extent[d]
            so += i * op.src_stride[d]
            do += i * op.dst_stride[d]
            q = q2
        vals = []
        for k in range(op.nsrc):
            _, buf, base = world.buffer_of(op.src[k])
            a = op.src[k] - base + so
            vals.append(torch.frombuffer(bytearray(buf[a : a + n * sdt.itemsize].tobytes()), dtype=sdt).clone())
        out = reduce_family_values(vals, fam, sdt) if fam is not None else vals[0]
        out_bytes = np.frombuffer(out.to(ddt).contiguous().view(torch.uint8).numpy().tobytes(), dtype=np.uint8)
        for j in range(op.ndst):
            _, dbuf, dbase = world.buffer_of(op.dst[j])
            b = op.dst[j] - dbase + do
            dbuf[b : b + n * ddt.itemsize] = out_bytes


TYPED_CASES = [
    ((4,), (Partial(),), (4,), (R,), (8, 16), torch.float32, torch.float32),
    ((4,), (Partial("avg"),), (4,), (Shard(0),), (8, 16), torch.float32, torch.float32),
    ((2, 2), (Shard(0), Partial()), (4,), (Shard(0),), (8, 16), torch.bfloat16, torch.bfloat16),
    ((2, 2), (Partial(), Partial("max")), (2, 2), (R, Shard(1)), (8, 16), torch.float32, torch.bfloat16),
    ((2, 3), (Partial(), Partial()), (2,), (R,), (8, 16), torch.float32, torch.float32),
    ((2, 2), (Shard(0), Shard(1)), (4,), (Shard(0),), (16, 16), torch.float32, torch.bfloat16),
    ((2,), (Partial(),), (2,), (Shard(0),), (5, 3), torch.float32, torch.float32),
]


@pytest.mark.parametrize("case", TYPED_CASES, ids=[str(i) for i in range(len(TYPED_CASES))])
def test_typed_tables_convert_and_collapse(case, monkeypatch):
    _check_typed_case(case, monkeypatch)


def _check_typed_case(case, monkeypatch):
    ss, sp, ts, tp, shape, sdt, tdt = case
    ns, nt = math.prod(ss), math.prod(ts)
    smesh, tmesh = torch.arange(ns).view(ss), torch.arange(ns, ns + nt).view(ts)
    ranks = list(range(ns + nt))
    eff = tuple(R if isinstance(p, Partial) else p for p in sp)
    world = World(ranks)
    logical, contribs = _make_source_local(0, smesh, sp, shape, sdt, False)
    by_rank = {r: {"rank": r, "src": [None], "dst": [None]} for r in ranks}
    targets = {}
    for r in ranks:
        if r < ns:
            local = contribs[r] if contribs is not None else local_slice_of(logical, smesh, eff, r)
            t, desc = world.alloc(r, local.shape, sdt)
            t.copy_(local)
            by_rank[r]["src"] = [desc]
        else:
            t, desc = world.alloc(r, local_slice_of(logical, tmesh, tp, r).shape, tdt)
            by_rank[r]["dst"] = [desc]
            targets[r] = t
        _, by_rank[r]["flags"] = world.alloc(r, (len(ranks),), torch.int32)
    monkeypatch.setattr(CopyTable, "finalize", lambda self, sm_count=None: self)
    layout = PairLayout(smesh, sp, tmesh, tp)
    batches = {}
    for r in ranks:
        b = P2PBatch.__new__(P2PBatch)
        b.rank, b.ranks, b.device, b.peer = r, ranks, torch.device("cpu"), FakePeer(1000 + r)
        b.nvls, b.tile_bytes, b.multicast_ops, b.stripe_partial = None, 4096, 0, True
        b._entries = [(layout, None, None)]
        b._finish_build(by_rank)
        batches[r] = b
        for cls, tiles, raw, *_ in b.table._packed:
            op = OpView.from_buffer_copy(raw)
            if op.mode == 0:
                for j in range(op.ndst):
                    single = OpView.from_buffer_copy(raw)
                    single.ndst, single.dst[0] = 1, op.dst[j]
                    _, sbuf, sbase = world.buffer_of(op.src[0])
                    _, dbuf, dbase = world.buffer_of(op.dst[j])
                    _emulate(single, sbuf, dbuf, sbase, dbase)
            else:
                assert cls == 1
                _emulate_typed(op, world)
    for r, t in targets.items():
        assert torch.equal(t, local_slice_of(logical, tmesh, tp, r).to(tdt)), f"rank {r}"
    if any(isinstance(p, Partial) for p in sp):
        # contributors wait for the primaries that read their shard; primaries signal them
        red = [(i, p.reduce_op) for i, p in enumerate(sp) if isinstance(p, Partial)]
        from etha_b200.comm.ir import partial_family

        # the collapse is striped: every member of a family executes part of it (replica groups that no consumer
        # reads from, possible when the source also has Replicate dims, stay idle as a whole)
        if not any(isinstance(p, type(R)) for p in sp):
            assert all(batches[r].table._packed for r in range(ns))
        for r in range(ns):
            fam_ranks = partial_family(smesh, red, r).ranks
            assert len({bool(batches[q].table._packed) for q in fam_ranks}) == 1, "a family works as a whole or not at all"
        for r in range(ns):
            readers = {p for p in range(ns) if p != r and batches[p].table._packed and r in partial_family(smesh, red, p).ranks}
            assert readers <= set(batches[r]._producers)
            assert all(r in batches[p]._consumers for p in readers)


def test_plain_layout_sends_whole_tensors_rank_to_rank(monkeypatch):
    """No layout declared: the k-th producer's tensor goes whole into the k-th consumer's tensor, one op each."""
    ranks = [0, 1, 2, 3]
    world = World(ranks)
    by_rank = {r: {"rank": r, "src": [None], "dst": [None]} for r in ranks}
    sources, targets = {}, {}
    for r in ranks:
        if r < 2:
            t, desc = world.alloc(r, (24, 10), torch.float32)
            t.copy_(torch.randn(24, 10, generator=torch.Generator().manual_seed(r)))
            by_rank[r]["src"], sources[r] = [desc], t
        else:
            t, desc = world.alloc(r, (24, 10), torch.float32)
            by_rank[r]["dst"], targets[r] = [desc], t
        _, by_rank[r]["flags"] = world.alloc(r, (len(ranks),), torch.int32)
    monkeypatch.setattr(CopyTable, "finalize", lambda self, sm_count=None: self)
    layout = PairLayout(torch.tensor([0, 1]), None, torch.tensor([2, 3]), None, plain=True)
    for r in ranks:
        b = P2PBatch.__new__(P2PBatch)
        b.rank, b.ranks, b.device, b.peer = r, ranks, torch.device("cpu"), FakePeer(1000 + r)
        b.nvls, b.tile_bytes, b.multicast_ops, b.stripe_partial = None, 4096, 0, True
        b._entries = [(layout, None, None)]
        b._finish_build(by_rank)
        assert len(b.table._packed) == (1 if r < 2 else 0)
        assert b._producers == ([r - 2] if r >= 2 else []) and b._consumers == ([r + 2] if r < 2 else [])
        for cls, tiles, raw, *_ in b.table._packed:
            op = OpView.from_buffer_copy(raw)
            _, sbuf, sbase = world.buffer_of(op.src[0])
            _, dbuf, dbase = world.buffer_of(op.dst[0])
            _emulate(op, sbuf, dbuf, sbase, dbase)
    assert torch.equal(targets[2], sources[0]) and torch.equal(targets[3], sources[1])


def test_random_partial_layouts_collapse_to_the_logical_tensor():
    """Random source meshes with up to two Partial dims, random targets: whatever the merging of per-replica routes
    and the striping over the family do, every consumer shard must equal the logical (collapsed) tensor."""
    import random

    rng = random.Random(1234)
    source_meshes = [(2,), (4,), (2, 2), (2, 3), (3, 2)]
    target_meshes = [(2,), (3,), (4,), (2, 2)]
    ops = ["sum", "avg", "max", "min"]
    seen = 0
    for _ in range(60):
        ss, ts = rng.choice(source_meshes), rng.choice(target_meshes)
        sp = tuple(rng.choice([Shard(0), Shard(1), R, Partial(rng.choice(ops)), Partial(rng.choice(ops))]) for _ in ss)
        tp = tuple(rng.choice([Shard(0), Shard(1), R]) for _ in ts)
        if not any(isinstance(p, Partial) for p in sp):
            continue
        sdt, tdt = rng.choice([(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
        shape = (rng.choice([12, 24]), rng.choice([12, 36]))  # divisible by 2, 3, 4 and 6

        class Patch:  # the part of pytest's monkeypatch the helper uses
            def setattr(self, obj, name, value):
                self.saved = (obj, name, getattr(obj, name))
                setattr(obj, name, value)

        mp = Patch()
        try:
            _check_typed_case((ss, sp, ts, tp, shape, sdt, tdt), mp)
        finally:
            obj, name, old = mp.saved
            setattr(obj, name, old)
        seen += 1
    assert seen >= 30


def test_random_copy_layouts_deliver_every_shard():
    """Random meshes, placements and (often unevenly divisible) shapes, disjoint and overlapping rank sets."""
    import random

    rng = random.Random(99)
    meshes = [(1,), (2,), (3,), (4,), (2, 2), (2, 3), (1, 2, 2)]
    for _ in range(40):
        ss, ts = rng.choice(meshes), rng.choice(meshes)
        sp = tuple(rng.choice([Shard(0), Shard(1), R]) for _ in ss)
        tp = tuple(rng.choice([Shard(0), Shard(1), R]) for _ in ts)
        shape = (rng.choice([7, 12, 16, 30]), rng.choice([5, 12, 64]))
        overlap = rng.random() < 0.4

        class Patch:
            def setattr(self, obj, name, value):
                self.saved = (obj, name, getattr(obj, name))
                setattr(obj, name, value)

        mp = Patch()
        try:
            _check_copy_case((ss, sp, ts, tp, shape), overlap, mp)
        except Exception as e:
            raise AssertionError(f"{(ss, sp, ts, tp, shape, overlap)}: {type(e).__name__}: {e}") from e
        finally:
            obj, name, old = mp.saved
            setattr(obj, name, old)
