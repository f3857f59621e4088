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
from torch.distributed.tensor.placement_types import Replicate, Shard

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
]


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_tables_of_all_ranks_deliver_every_shard(case, overlap, monkeypatch):
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
        b.nvls, b.tile_bytes, b.multicast_ops = None, 4096, 0
        b._entries = [(layout, None, None)]
        b._finish_build(by_rank)
        batches[r] = b

    writers = {r: set() for r in ranks}
    for r, b in batches.items():
        for cls, tiles, raw in b.table._packed:
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
