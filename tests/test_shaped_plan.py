"""Uneven shards: explicit-box plans checked against DTensor's chunking, and executed on gloo."""

import math

import pytest
import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard, _StridedShard

from etha_b200.comm import bucket_comm, chunk_to_bucket_ops, m2m_to_chunks, plan_m2m
from etha_b200.comm.baselines import local_slice_of
from etha_b200.comm.shaped import infer_global_shape, needs_shaped_plan, plan_for_shape, shaped_to_chunks

from dist_utils import run_distributed

R = Replicate()

CASES = [
    ((2,), (Shard(0),), (2,), (Shard(1),), (1000, 333)),
    ((2,), (Shard(0),), (2,), (Shard(1),), (7, 4096)),
    ((2,), (Shard(0),), (2,), (Shard(0),), (4097,)),
    ((2, 2), (Shard(0), Shard(1)), (3,), (Shard(0),), (10, 7)),
    ((3,), (Shard(0),), (2, 2), (R, Shard(0)), (5, 6)),
    ((2, 2), (Shard(0), Shard(0)), (4,), (Shard(1),), (9, 9)),
    ((2,), (Partial(),), (2,), (Shard(0),), (5, 3)),
    # FSDP over TP: the strided shard on mesh dim 0 follows the plain shard on mesh dim 1
    ((4,), (Shard(0),), (2, 2), (_StridedShard(0, split_factor=2), Shard(0)), (16, 6)),
    ((2, 2), (_StridedShard(1, split_factor=2), Shard(1)), (3,), (Shard(0),), (9, 8)),
    # layouts of the reference's CPU test: [R, R, S0, S1] -> [R, _StridedShard(1, 2), R, S1]
    ((1, 1, 2, 2), (R, R, Shard(0), Shard(1)), (2, 1, 1, 2), (R, _StridedShard(1, split_factor=2), R, Shard(1)), (64, 64)),
    ((1, 2, 2, 1), (R, R, Shard(0), Shard(1)), (1, 2, 1, 2), (R, _StridedShard(1, split_factor=2), R, Shard(1)), (64, 64)),
    ((4,), (Shard(0),), (4,), (Shard(1),), (64, 64)),  # even: must move exactly what the lcm plan moves
]
N_GLOO = 9  # the cases before the 8-rank ones and the even one run on gloo


@pytest.mark.parametrize("case", CASES)
def test_plan_covers_every_consumer_element_exactly_once(case):
    ss, sp, ts, tp, shape = case
    ns, nt = math.prod(ss), math.prod(ts)
    smesh, tmesh = torch.arange(ns).view(ss), torch.arange(ns, ns + nt).view(ts)
    plan = plan_for_shape(smesh, sp, tmesh, tp, shape)
    eff = tuple(R if isinstance(p, Partial) else p for p in sp)
    full = torch.arange(math.prod(shape), dtype=torch.float64).view(shape)
    got = {r: torch.full_like(local_slice_of(full, tmesh, tp, r), -1.0) for r in tmesh.reshape(-1).tolist()}
    hits = {r: torch.zeros_like(got[r]) for r in got}
    for route in plan.routes:
        src = local_slice_of(full, smesh, eff, route.src_rank)[tuple(slice(a, b) for a, b in route.src_box)]
        for r, box in route.dsts:
            idx = tuple(slice(a, b) for a, b in box)
            got[r][idx] = src
            hits[r][idx] += 1
    for r in got:
        assert torch.equal(got[r], local_slice_of(full, tmesh, tp, r))
        assert bool((hits[r] == 1).all())
    assert needs_shaped_plan(smesh, sp, shape) or needs_shaped_plan(tmesh, tp, shape) or case is CASES[-1]
    if case is CASES[-1]:
        assert not needs_shaped_plan(smesh, sp, shape) and not needs_shaped_plan(tmesh, tp, shape)
    local_shapes = {r: tuple(local_slice_of(full, smesh, eff, r).shape) for r in smesh.reshape(-1).tolist()}
    assert infer_global_shape(smesh, sp, local_shapes) == tuple(shape)


def test_even_shape_moves_same_bytes_as_lcm_plan():
    smesh, tmesh = torch.arange(4), torch.arange(4, 8)
    plan = plan_for_shape(smesh, (Shard(0),), tmesh, (Shard(1),), (64, 64))
    m2m = plan_m2m(smesh, (Shard(0),), tmesh, (Shard(1),))
    assert len(plan.routes) == len([r for r in m2m.routes if r.dsts]) == 16
    assert all(r.shape == (16, 16) for r in plan.routes)


def _worker(rank, world):
    for (ss, sp, ts, tp, shape) in CASES[:N_GLOO]:
        ns, nt = math.prod(ss), math.prod(ts)
        if ns + nt > world:
            continue
        smesh, tmesh = torch.arange(ns).view(ss), torch.arange(ns, ns + nt).view(ts)
        eff = tuple(R if isinstance(p, Partial) else p for p in sp)
        g = torch.Generator().manual_seed(3)
        full = torch.randn(shape, generator=g)
        has_partial = any(isinstance(p, Partial) for p in sp)
        src = tgt = None
        if rank < ns:
            src = local_slice_of(full, smesh, eff, rank).clone()
            if has_partial:
                src = src / 2  # two contributors, sum restores the value exactly
        elif rank < ns + nt:
            tgt = torch.full_like(local_slice_of(full, tmesh, tp, rank), float("nan")).clone()
        plan = plan_for_shape(smesh, sp, tmesh, tp, shape)
        chunks = shaped_to_chunks(plan, rank, src, tgt, source_mesh=smesh)
        for bucket_size in (1, 1 << 16):
            if tgt is not None:
                tgt.fill_(float("nan"))
            bucket_comm(chunk_to_bucket_ops(chunks, bucket_size))
            if tgt is not None:
                assert torch.equal(tgt, local_slice_of(full, tmesh, tp, rank)), (ss, sp, ts, tp, shape)
        dist.barrier()
    # the divisible-only path refuses uneven shapes loudly
    if rank == 0:
        m2m = plan_m2m(torch.arange(2), (Shard(0),), torch.arange(2, 4), (Shard(1),))
        with pytest.raises(ValueError, match="not divisible"):
            m2m_to_chunks(m2m, 0, source_tensor=torch.zeros(500, 333))


def test_uneven_redistribution_on_gloo():
    run_distributed(_worker, 7)


def test_strided_shard_that_is_not_a_box_is_refused():
    smesh, tmesh = torch.arange(4), torch.arange(4, 8).view(2, 2)
    with pytest.raises(NotImplementedError, match="contiguous box"):
        plan_for_shape(smesh, (Shard(0),), tmesh, (_StridedShard(0, split_factor=2), R), (16, 4))
    with pytest.raises(NotImplementedError, match="explicit-box planner"):
        plan_m2m(smesh, (Shard(0),), tmesh, (_StridedShard(0, split_factor=2), Shard(0)))
