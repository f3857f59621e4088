"""Redistribution on CPU/gloo through plan -> chunks -> buckets -> bucket_comm, checked bit for bit.

The matrix follows the reference's reshard tests (tests/test_communication_replicate_shard.py:329-431,
tests/test_communication_cpu.py, tests/test_communication_symmetric_mesh.py): MoE 3-D -> EP 1-D,
identical layouts, all-Replicate sources, slice views, Partial sum/avg/max, 2-D Shard+Partial, double
Partial, the asymmetric (2,3) case, both coalescing modes, plus overlapping meshes.
"""

import math

import pytest
import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from etha_b200.comm import bucket_comm, chunk_to_bucket_ops, m2m_to_chunks, plan_m2m
from etha_b200.comm.baselines import local_slice_of
from etha_b200.comm.ir import partial_family, reduce_family_values

from dist_utils import run_distributed

R, P = Replicate(), Partial()


def S(d):
    return Shard(d)


# (source mesh shape, source placements, target mesh shape, target placements, global shape, slice_view)
CASES_8 = [
    ((1, 2, 2), (R, S(0), S(0)), (4,), (S(0),), (8, 16, 32), False),
    ((2, 2), (R, S(0)), (2, 2), (R, S(0)), (8, 16), False),
    ((1, 4), (R, R), (2, 2), (R, S(0)), (8, 16), False),
    ((1, 2, 2), (R, S(0), S(0)), (4,), (S(0),), (8, 16, 32), True),
    ((2, 2), (S(0), S(0)), (4,), (S(0),), (8, 16, 32), True),
    ((4,), (P,), (4,), (R,), (8, 16), False),
    ((4,), (Partial("avg"),), (4,), (S(0),), (8, 16), False),
    ((2, 2), (S(0), P), (4,), (S(0),), (8, 16), False),
    ((2, 2), (P, P), (4,), (R,), (8, 16), False),
    ((2, 3), (P, P), (2,), (R,), (8, 16), False),
    ((4,), (S(0),), (4,), (S(1),), (64, 64), False),
    ((4,), (S(1),), (4,), (S(0),), (64, 64), False),
    ((2, 2), (S(0), S(1)), (2, 2), (S(1), S(0)), (64, 64), False),
    ((2, 2), (Partial("max"), S(1)), (4,), (S(0),), (8, 16), False),
    ((2, 2), (Partial("sum"), Partial("max")), (2, 2), (R, S(1)), (8, 16), False),
    ((3,), (S(0),), (2,), (S(1),), (12, 10), False),
]


def _make_source_local(rank, smesh, splc, shape, dtype, slice_view):
    """Local shard (or pending Partial contribution) of `rank`, plus the logical full tensor."""
    has_partial = any(isinstance(p, Partial) for p in splc)
    eff = tuple(R if isinstance(p, Partial) else p for p in splc)
    g = torch.Generator().manual_seed(0)
    full = torch.randn(shape, generator=g).to(dtype)
    if not has_partial:
        return full, None
    # every rank of a family holds an independent random value of the family's shard; ranks that differ only along a
    # Replicate mesh dim hold the same value (that is what Replicate means), so the seed ignores those coordinates
    contribs = {}
    for r in smesh.reshape(-1).tolist():
        coord = (smesh == r).nonzero()[0].tolist()
        key = 0
        for c, size, p in zip(coord, smesh.shape, splc):
            key = key * int(size) + (0 if isinstance(p, Replicate) else int(c))
        gr = torch.Generator().manual_seed(1000 + key)
        contribs[r] = torch.randn(local_slice_of(full, smesh, eff, r).shape, generator=gr).to(dtype)
    reductions = [(i, p.reduce_op) for i, p in enumerate(splc) if isinstance(p, Partial)]
    logical = torch.zeros(shape, dtype=dtype)
    for r in smesh.reshape(-1).tolist():
        fam = partial_family(smesh, reductions, r)
        val = reduce_family_values([contribs[q] for q in fam.ranks], fam, dtype)
        local_slice_of(logical, smesh, eff, r).copy_(val)
    return logical, contribs


def _run_case(rank, case, bucket_size, overlap, dtype=torch.float32, wire_dtype=None, tgt_dtype=None):
    sshape, splc, tshape, tplc, shape, slice_view = case
    ns, nt = math.prod(sshape), math.prod(tshape)
    smesh = torch.arange(ns).view(sshape)
    t0 = 0 if overlap else ns
    tmesh = torch.arange(t0, t0 + nt).view(tshape)
    eff = tuple(R if isinstance(p, Partial) else p for p in splc)
    tgt_dtype = tgt_dtype or dtype

    wide = list(shape)
    if slice_view:
        wide[1] *= 2
    logical, contribs = _make_source_local(rank, smesh, splc, tuple(wide), dtype, slice_view)
    g = torch.Generator().manual_seed(99)
    tgt_init_full = torch.randn(tuple(wide), generator=g).to(tgt_dtype)

    src_local = tgt_local = tgt_backing = None
    if rank in smesh.reshape(-1).tolist():
        base = contribs[rank].clone() if contribs is not None else local_slice_of(logical, smesh, eff, rank).clone()
        src_local = base[:, : shape[1]] if slice_view else base
        src_snapshot = src_local.clone()
    if rank in tmesh.reshape(-1).tolist():
        tgt_backing = local_slice_of(tgt_init_full, tmesh, tplc, rank).clone()
        tgt_local = tgt_backing[:, : shape[1]] if slice_view else tgt_backing

    m2m = plan_m2m(smesh, splc, tmesh, tplc)
    chunks = m2m_to_chunks(
        m2m, rank, source_tensor=src_local, target_tensor=tgt_local, transfer_dtype=wire_dtype, source_mesh=smesh
    )
    bucket_comm(chunk_to_bucket_ops(chunks, bucket_size))

    if src_local is not None:
        assert torch.equal(src_local, src_snapshot), "source was modified"
    if tgt_local is not None:
        want_full = logical[:, : shape[1]] if slice_view else logical
        want = local_slice_of(logical, tmesh, tplc, rank)
        want = want[:, : shape[1]] if slice_view else want
        if wire_dtype is not None:
            want = want.to(wire_dtype)
        want = want.to(tgt_dtype)
        assert torch.equal(tgt_local, want), f"rank {rank}: max diff {(tgt_local.float() - want.float()).abs().max()}"
        if slice_view:
            untouched = local_slice_of(tgt_init_full, tmesh, tplc, rank)[:, shape[1] :]
            assert torch.equal(tgt_backing[:, shape[1] :], untouched), "bytes outside the registered view were written"


def _worker(rank, world_size, cases, bucket_size, overlap):
    for case in cases:
        ns, nt = math.prod(case[0]), math.prod(case[2])
        need = max(ns, nt) if overlap else ns + nt
        if rank < need:
            pass
        # every rank walks every case: ranks outside both meshes simply have no chunks
        _run_case(rank, case, bucket_size, overlap)
        dist.barrier()


@pytest.mark.parametrize("bucket_size", [1, 256 * 1024])
def test_reshard_matrix_disjoint(bucket_size):
    run_distributed(_worker, 8, CASES_8, bucket_size, False)


@pytest.mark.parametrize("bucket_size", [1, 4096])
def test_reshard_matrix_overlapping_meshes(bucket_size):
    # producer and consumer meshes share ranks 0..: every rank may hold both roles
    run_distributed(_worker, 6, CASES_8, bucket_size, True)


def _mixed_dtype_worker(rank, world_size):
    # fp32 Partial source -> bf16 Replicate target: the reduction happens before the down-cast
    # (reference regression: tests/test_communication_replicate_shard.py:202-327)
    case = ((4,), (P,), (4,), (R,), (8, 16), False)
    for bucket_size in (1, 1 << 20):
        _run_case(rank, case, bucket_size, False, dtype=torch.float32, wire_dtype=torch.bfloat16, tgt_dtype=torch.bfloat16)
    # plain down-cast on the wire and bf16 -> fp32 up-cast at the consumer
    case = ((2, 2), (S(0), S(1)), (4,), (S(0),), (16, 16), False)
    _run_case(rank, case, 1, False, dtype=torch.float32, wire_dtype=torch.bfloat16, tgt_dtype=torch.bfloat16)
    _run_case(rank, case, 1 << 20, False, dtype=torch.bfloat16, wire_dtype=torch.bfloat16, tgt_dtype=torch.float32)
    # equal item sizes: the source dtype travels and the consumer converts values (never a byte reinterpretation)
    _run_case(rank, case, 1, False, dtype=torch.float16, wire_dtype=torch.float16, tgt_dtype=torch.bfloat16)


def test_mixed_dtypes():
    run_distributed(_mixed_dtype_worker, 8)


def _dtensor_worker(rank, world_size):
    """Config: producer mesh [2] Shard(0) -> consumer mesh [2] Shard(1), 8 fp32 tensors, then a Partial pair;
    the expected values come from DTensor itself (distribute_tensor / redistribute / full_tensor)."""
    from torch.distributed.device_mesh import DeviceMesh
    from torch.distributed.tensor import DTensor, distribute_tensor

    prod = DeviceMesh("cpu", torch.tensor([0, 1]))
    cons = DeviceMesh("cpu", torch.tensor([2, 3]))
    torch.manual_seed(0)
    shapes = [(1024, 512), (512, 1024), (4096,), (2048, 256), (256, 2048), (1000, 334), (8, 4096), (128, 128)]
    fulls = [torch.randn(s) for s in shapes]
    chunks = []
    targets = []
    for i, full in enumerate(fulls):
        tplc = (S(1),) if full.dim() > 1 else (S(0),)
        m2m = plan_m2m(prod, (S(0),), cons, tplc)
        src = tgt = None
        if rank < 2:
            src = distribute_tensor(full, prod, [S(0)]).to_local()
        else:
            tgt = torch.zeros_like(distribute_tensor(full, cons, list(tplc)).to_local())
            targets.append((tgt, full, tplc))
        chunks += m2m_to_chunks(m2m, rank, source_tensor=src, target_tensor=tgt, tensor_id=i)
    bucket_comm(chunk_to_bucket_ops(chunks, 64 * 1024))
    for tgt, full, tplc in targets:
        want = distribute_tensor(full, cons, list(tplc)).to_local()
        assert torch.equal(tgt, want)

    # Partial source (each rank holds randn/2) collapsed into a Replicate target
    torch.manual_seed(100 + rank)
    m2m = plan_m2m(prod, (P,), cons, (R,))
    src = tgt = None
    if rank < 2:
        src = torch.randn(256, 128) / 2
        want = DTensor.from_local(src, prod, [P]).redistribute(prod, [R]).to_local()
        dist.send(want, dst=rank + 2)
    else:
        tgt = torch.zeros(256, 128)
        want = torch.empty(256, 128)
        dist.recv(want, src=rank - 2)
    ch = m2m_to_chunks(m2m, rank, source_tensor=src, target_tensor=tgt, source_mesh=prod)
    bucket_comm(chunk_to_bucket_ops(ch, 1))
    if tgt is not None:
        assert torch.equal(tgt, want)


def test_against_dtensor_world4():
    run_distributed(_dtensor_worker, 4)
