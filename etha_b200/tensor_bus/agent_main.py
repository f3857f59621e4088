"""Command-line entry of one agent: `python -m etha_b200.tensor_bus.agent_main` under torchrun (or with
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set by hand).

Counterpart of the reference's example agent script (examples/vllm_weight_sync/agent.py): removes stale
queue/state files and semaphores of a previous run, then serves commands until terminated.
"""

from __future__ import annotations

import argparse
import logging
import os
import signal

from ..ops.hostlib import unlink_semaphore
from .agent import TensorBusAgent
from .bootstrap import default_paths


def sweep_stale(command_path: str, state_path: str) -> None:
    for p in (command_path, state_path):
        try:
            os.unlink(p)
        except OSError:
            pass
    stem = os.path.splitext(os.path.basename(command_path))[0]
    for name in (f"/cq_{stem}", f"/cq_space_{stem}", f"/cq_ready_{stem}"):
        try:
            unlink_semaphore(name)
        except Exception:
            pass


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--store-host", default="127.0.0.1")
    ap.add_argument("--store-port", type=int, default=49001)
    ap.add_argument("--store-backend", default="tcp", choices=["tcp", "etcd"])
    ap.add_argument("--path-prefix", default="/tmp/agent_rank")
    ap.add_argument("--device", default=None, help="cpu to force the gloo data path")
    ap.add_argument("--log-level", default="WARNING")
    args = ap.parse_args()
    logging.basicConfig(level=args.log_level, format="%(asctime)s agent %(message)s")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if args.path_prefix == "/tmp/agent_rank":
        cq, st = default_paths(rank)
    else:
        cq, st = f"{args.path_prefix}{rank}_command.lmdb", f"{args.path_prefix}{rank}_state.lmdb"
    sweep_stale(cq, st)
    agent = TensorBusAgent(rank, world, args.store_host, args.store_port, cq, st, store_backend=args.store_backend,
                           device=args.device)
    signal.signal(signal.SIGTERM, lambda *_: agent.stop())
    signal.signal(signal.SIGINT, lambda *_: agent.stop())
    try:
        agent.run()
    finally:
        agent.close(destroy=True)


if __name__ == "__main__":
    main()
