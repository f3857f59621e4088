"""The gather-broadcast comparison method agrees with the chunk and bucket paths (the reference asserts the same in
tests/test_communication_cpu.py:103-117), on gloo with world_size 4."""

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.tensor import DTensor
from torch.distributed.tensor.placement_types import Replicate, Shard

from etha_b200.comm import bucket_comm, chunk_to_bucket_ops, m2m_to_chunks, plan_m2m
from etha_b200.comm.baselines import gather_broadcast_comm, local_slice_of

from dist_utils import run_distributed

LAYOUTS = [((Shard(0),), (Shard(1),)), ((Shard(0),), (Replicate(),)), ((Replicate(),), (Shard(0),)), ((Shard(1),), (Shard(1),))]


def _worker(rank, world):
    k = world // 2
    smesh_t, tmesh_t = torch.arange(k), torch.arange(k, world)
    smesh = DeviceMesh("cpu", smesh_t)  # built on every rank: sub-mesh creation is collective
    for i, (sp, tp) in enumerate(LAYOUTS):
        full = torch.randn(64, 48, generator=torch.Generator().manual_seed(i))
        src = local_slice_of(full, smesh_t, sp, rank).clone() if rank < k else None
        results = {}
        for name, bucket_size in (("chunk", 1), ("bucket", 256 * 1024)):
            tgt = torch.zeros_like(local_slice_of(full, tmesh_t, tp, rank)) if rank >= k else None
            chunks = m2m_to_chunks(plan_m2m(smesh_t, sp, tmesh_t, tp), rank, source_tensor=src, target_tensor=tgt,
                                   source_mesh=smesh_t, tensor_id=i)
            bucket_comm(chunk_to_bucket_ops(chunks, bucket_size))
            results[name] = tgt
        local_dt = DTensor.from_local(src, smesh, sp) if rank < k else None
        results["gather_broadcast"] = gather_broadcast_comm(tmesh_t, tp, local_dt, full, k)
        if rank >= k:
            want = local_slice_of(full, tmesh_t, tp, rank)
            for name, got in results.items():
                assert got is not None and torch.equal(got, want), (name, sp, tp)
        else:
            assert results["gather_broadcast"] is None
        dist.barrier()


def test_three_methods_agree():
    run_distributed(_worker, 4)
