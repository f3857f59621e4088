"""`bus_roundtrip`: agents spawned from inside a running job, one client per logical rank, timed transfer rounds.
CPU/gloo data path; covers both the one-process-per-rank layout and the single process that plays both sides."""

import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Replicate, Shard

from etha_b200.models.bus_sync import BusItem, bus_roundtrip

from dist_utils import run_distributed


def _two_process_worker(rank, world):
    def share(obj):
        box = [obj]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    g = torch.Generator().manual_seed(1)
    full = torch.randn(64, 48, generator=g)
    stamp_src, stamp_dst = torch.zeros(4, dtype=torch.int64), torch.zeros(4, dtype=torch.int64)
    tgt = torch.zeros(64, 48)
    items = [BusItem(full.clone() if rank == 0 else None, tgt if rank == 1 else None, (Shard(0),), (Shard(1),)),
             BusItem(stamp_src if rank == 0 else None, stamp_dst if rank == 1 else None, (Replicate(),), (Replicate(),))]
    seen = []

    def on_step(k, phase):
        if phase == "before_send":
            stamp_src.fill_(k)
        else:
            seen.append(int(stamp_dst[0]))

    out = bus_roundtrip(rank, world, 0, items, [0], [1], steps=3, warmup=1, share=share, on_step=on_step, device_type="cpu",
                        timeout=90.0)
    assert out["ms_per_step"] > 0 and out["agents"] == 2
    if rank == 1:
        assert torch.equal(tgt, full) and seen == [-1, 0, 1, 2]


def test_one_process_per_rank():
    run_distributed(_two_process_worker, 2)


def test_single_process_plays_both_sides():
    full = torch.arange(32 * 16, dtype=torch.float32).view(32, 16)
    tgt = torch.zeros(32, 16)
    out = bus_roundtrip(0, 1, 0, [BusItem(full, tgt, (Shard(0),), (Shard(0),))], [0], [1], steps=2, warmup=1,
                        share=lambda obj: obj, device_type="cpu", timeout=90.0)
    assert out["agents"] == 2 and torch.equal(tgt, full)
