"""One worker of the NVLS-through-the-bus test: the trainer (agent rank 0) sends, every inference worker (agent
ranks 1..n) receives Replicate targets that live in its client's replicated arena.  Launched by test_y_bus_nvls_gpu.py
next to one agent process per GPU."""

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
from torch.distributed.tensor.placement_types import Replicate, Shard  # noqa: E402

from etha_b200.tensor_bus.client import TensorBusClient  # noqa: E402

SHAPES = [(512, 1024), (4096,), (64, 2048)]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--agent-rank", type=int, required=True)
    ap.add_argument("--consumers", type=int, required=True)
    ap.add_argument("--path-prefix", required=True)
    ap.add_argument("--arena", type=int, default=1, help="0: consumers use ordinary tensors (software fan-out)")
    args = ap.parse_args()
    r, n = args.agent_rank, args.consumers
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    client = TensorBusClient(r, f"{args.path_prefix}{r}_command.lmdb", f"{args.path_prefix}{r}_state.lmdb",
                             connection_timeout=120.0, replicated_arena_bytes=64 << 20)
    trainer = r == 0
    me, other = ("trainer", "inference") if trainer else ("inference", "trainer")
    smesh, tmesh = torch.tensor([0]), torch.arange(1, n + 1)
    client.init_pair("rep", me, other, 1 if trainer else n, smesh if trainer else tmesh, (Replicate(),), timeout=120.0)
    client.init_pair("tp", me, other, 1 if trainer else n, smesh if trainer else tmesh,
                     (Replicate(),) if trainer else (Shard(0),), timeout=120.0)
    g = torch.Generator().manual_seed(11)
    fulls = [torch.randn(s, generator=g).to(torch.bfloat16) for s in SHAPES]
    sharded_full = torch.randn(8 * n, 256, generator=g).to(torch.bfloat16)
    tensors, mine = [], []
    for f in fulls:
        if trainer:
            t = f.to(dev)
        elif args.arena:
            t = client.empty_replicated(f.shape, torch.bfloat16, dev)
            t.zero_()
        else:
            t = torch.zeros(f.shape, dtype=torch.bfloat16, device=dev)
        tensors.append((t, "rep"))
        mine.append(t)
    # one ordinary sharded tensor next to the replicated ones: it takes the plain peer-store path in the same batch
    sh = sharded_full.to(dev) if trainer else torch.zeros(8, 256, dtype=torch.bfloat16, device=dev)
    tensors.append((sh, "tp"))
    batch = client.register_tensors("nvls", tensors, timeout=180.0)
    bad = 0
    for step in range(3):
        if trainer:
            for t, f in zip(mine, fulls):
                t.copy_((f.float() * (step + 1)).to(torch.bfloat16))
            torch.cuda.synchronize()
            batch.transfer("send", blocking=True, timeout=120.0)
        else:
            while not batch.query_transfer_signal(timeout=60.0):
                time.sleep(0.002)
            batch.transfer("recv", blocking=True, timeout=120.0)
            for t, f in zip(mine, fulls):
                if not torch.equal(t.cpu(), (f.float() * (step + 1)).to(torch.bfloat16)):
                    bad += 1
            if not torch.equal(sh.cpu(), sharded_full[8 * (r - 1): 8 * r]):
                bad += 1
    raw = client.state.get("batch:nvls/state:multicast_ops")
    print(json.dumps({"agent_rank": r, "bad": bad, "multicast_ops": int(raw.decode()) if raw else None}), flush=True)
    batch.close()
    client.close()
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
