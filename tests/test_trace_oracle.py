"""Tracing oracle: derive the mesh-to-mesh map by pushing cell ids through DTensor itself (from_local ->
full_tensor -> distribute_tensor on real gloo meshes), the way the reference's planner works
(src/etha/comm/get_m2m_map.py:174-250), and compare with the closed-form planner."""

import math

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor, distribute_tensor
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from etha_b200.comm import plan_m2m

from dist_utils import run_distributed

R = Replicate()
CASES = [
    ((2,), (Shard(0),), (2,), (Shard(1),)),
    ((1, 2, 2), (R, Shard(0), Shard(0)), (4,), (Shard(0),)),
    ((2, 2), (R, Shard(0)), (2, 2), (R, Shard(0))),
    ((2, 2), (Shard(0), Shard(1)), (2, 2), (Shard(1), Shard(0))),
    ((2, 2), (Partial(), Shard(0)), (4,), (Shard(0),)),
    ((4,), (R,), (2, 2), (R, Shard(0))),
    ((3,), (Shard(0),), (2,), (Shard(0),)),
]


def _trace(rank, smesh_t, splc, tmesh_t, tplc):
    eff = tuple(R if isinstance(p, Partial) else p for p in splc)
    plan = plan_m2m(smesh_t, splc, tmesh_t, tplc)  # only for the grid extents
    grid = [a * b for a, b in zip(plan.source_num_slicers, _counts(smesh_t, eff, len(plan.source_num_slicers)))]
    smesh, tmesh = DeviceMesh("cpu", smesh_t), DeviceMesh("cpu", tmesh_t)
    s_flat, t_flat = smesh_t.reshape(-1).tolist(), tmesh_t.reshape(-1).tolist()
    full = None
    if rank in s_flat:
        cells = plan.source_num_slicers
        local = torch.arange(math.prod(cells), dtype=torch.int64).view(cells) + rank * 10_000
        full = DTensor.from_local(local, smesh, list(eff), run_check=False).full_tensor()
        assert list(full.shape) == grid
    grids = [None] * dist.get_world_size()
    dist.all_gather_object(grids, full)
    found = {}
    if rank in t_flat:
        j = t_flat.index(rank)
        src_grid = grids[s_flat[j % len(s_flat)]]
        mine = distribute_tensor(src_grid, tmesh, list(tplc), src_data_rank=None).to_local()
        for t_cell in torch.cartesian_prod(*[torch.arange(n) for n in mine.shape]).view(-1, mine.dim()).tolist():
            v = int(mine[tuple(t_cell)])
            s_rank, lin = divmod(v, 10_000)
            s_cell = []
            for n in reversed(plan.source_num_slicers):
                s_cell.append(lin % n)
                lin //= n
            found.setdefault((s_rank, tuple(reversed(s_cell))), []).append((rank, tuple(t_cell)))
    merged = [None] * dist.get_world_size()
    dist.all_gather_object(merged, found)
    table = {}
    for part in merged:
        for k, v in (part or {}).items():
            table.setdefault(k, []).extend(v)
    return plan, {k: sorted(v) for k, v in table.items()}


def _counts(mesh, plc, ndim):
    c = [1] * ndim
    for n, p in zip(mesh.shape, plc):
        if isinstance(p, Shard):
            c[p.dim] *= n
    return c


def _worker(rank, world):
    for ss, sp, ts, tp in CASES:
        ns, nt = math.prod(ss), math.prod(ts)
        smesh_t = torch.arange(ns).view(ss)
        tmesh_t = torch.arange(ns, ns + nt).view(ts)
        plan, traced = _trace(rank, smesh_t, sp, tmesh_t, tp)
        planned = {(r.src.rank, r.src.cell): sorted((d.rank, d.cell) for d in r.dsts) for r in plan.routes if r.dsts}
        assert planned == traced, (ss, sp, ts, tp)
        dist.barrier()


def test_closed_form_plan_equals_dtensor_trace():
    run_distributed(_worker, 8)
