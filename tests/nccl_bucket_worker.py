"""NCCL path of the bucket executor on real GPUs (ordered channels, bounded window, completion polling).
Run by test_nccl_bucket_gpu.py under torchrun; world = 2k ranks, first half produces, second half consumes."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torch.distributed.tensor.placement_types import Partial, Replicate, Shard  # noqa: E402

from etha_b200.comm import bucket_comm, chunk_to_bucket_ops, m2m_to_chunks, plan_m2m  # noqa: E402
from etha_b200.comm.baselines import local_slice_of  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("cuda:nccl,cpu:gloo", rank=rank, world_size=world)
    k = world // 2
    smesh, tmesh = torch.arange(k), torch.arange(k, world)
    cases = [((Shard(0),), (Shard(0),), (256, 512), torch.bfloat16, torch.bfloat16),
             ((Shard(0),), (Replicate(),), (128, 256), torch.float32, torch.bfloat16),
             ((Replicate(),), (Shard(0),), (64, 1024), torch.float32, torch.float32)]
    if k >= 2:
        cases += [((Shard(0),), (Shard(1),), (256, 512), torch.bfloat16, torch.bfloat16),
                  ((Partial(),), (Replicate(),), (64, 64), torch.float32, torch.float32)]
    ok = True
    for bucket_size in (1, 1 << 20):
        chunks, checks = [], []
        for i, (sp, tp, shape, sdt, tdt) in enumerate(cases):
            g = torch.Generator().manual_seed(10 + i)
            full = torch.randn(shape, generator=g)
            eff = tuple(Replicate() if isinstance(p, Partial) else p for p in sp)
            partial = any(isinstance(p, Partial) for p in sp)
            src = tgt = None
            if rank < k:
                src = local_slice_of(full, smesh, eff, rank).to(sdt)
                if partial:
                    src = src / k
                src = src.to(dev)
            else:
                tgt = torch.zeros(local_slice_of(full, tmesh, tp, rank).shape, dtype=tdt, device=dev)
                want = local_slice_of(full, tmesh, tp, rank).to(sdt)
                if partial:
                    want = sum(want / k for _ in range(k))
                checks.append((tgt, want.to(tdt).to(dev) if sdt.itemsize >= tdt.itemsize else want.to(dev).to(tdt)))
            wire = sdt if sdt.itemsize <= tdt.itemsize else tdt
            chunks += m2m_to_chunks(plan_m2m(smesh, sp, tmesh, tp), rank, source_tensor=src, target_tensor=tgt,
                                    transfer_dtype=wire, source_mesh=smesh, tensor_id=i)
        for _ in range(2):
            bucket_comm(chunk_to_bucket_ops(chunks, bucket_size))
        for tgt, want in checks:
            ok = ok and torch.equal(tgt, want)
        dist.barrier()
    print(f"rank {rank} RESULT {'PASS' if ok else 'FAIL'}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
