"""Two ranks, two GPUs: VMM arenas shared by file descriptor, an NVLS multicast team, and a Replicate fan-out
written with multimem.st.  Run by test_nvls_gpu.py under torchrun."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torch.distributed.tensor.placement_types import Replicate  # noqa: E402

from etha_b200.comm.p2p import P2PBatch, PairLayout  # noqa: E402
from etha_b200.ops import device_info  # noqa: E402
from etha_b200.parallel.arena import NvlsTeam, VmmArena  # noqa: E402
from etha_b200.parallel.peer import PeerMemory  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    if not device_info()["multicast"]:
        print("SKIP: multicast not supported", flush=True)
        dist.destroy_process_group()
        return
    ranks = list(range(world))
    peer = PeerMemory(dev)
    arena = VmmArena(4 << 20, dev, n_team=world)
    team = None
    ok = True
    try:
        team = NvlsTeam(rank, ranks, arena, tag=os.environ.get("MASTER_PORT", "0"), all_gather=all_gather, peer=peer)
        layout = PairLayout(torch.tensor([0]), (Replicate(),), torch.arange(world), (Replicate(),))
        g = torch.Generator(device=dev).manual_seed(5)
        want = torch.randn(512, 1024, generator=g, device=dev).to(torch.bfloat16)  # same on every rank
        for use_nvls in (False, True):
            tgt = arena.tensor(256 << 10, (512, 1024), torch.bfloat16)
            tgt.zero_()
            guard = arena.tensor(0, (1024,), torch.int32)
            guard.fill_(7)
            torch.cuda.synchronize()
            batch = P2PBatch(rank, ranks, dev, exchange=all_gather, peer=peer, nvls=team if use_nvls else None)
            batch.add(layout, want if rank == 0 else None, tgt)
            batch.build()
            dist.barrier()
            for _ in range(2):
                batch.transfer(timeout_s=5.0)
                torch.cuda.synchronize()
                batch.check()
                dist.barrier()
            good = torch.equal(tgt, want) and bool((guard == 7).all())
            if rank == 0:
                good = good and batch.multicast_ops == (1 if use_nvls else 0)
            print(f"rank {rank} nvls={use_nvls} ok={good} multicast_ops={batch.multicast_ops}", flush=True)
            ok = ok and good
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        if team is not None:
            team.close()
        arena.close()
        dist.barrier()
        dist.destroy_process_group()
    print(f"rank {rank} RESULT {'PASS' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
