"""Launches the closed loop of the weight-sync example on one machine:

    2n agents (one per GPU)  +  n trainer workers (GPUs 0..n-1)  +  n inference workers (GPUs n..2n-1)

    python examples/weight_sync/launch.py --side-size 4 --model llama3-8b --syncs 5      # 8 GPUs
    python examples/weight_sync/launch.py --side-size 2 --model tiny --device cpu        # no GPU: gloo data path
    python examples/weight_sync/launch.py --scenario moe --trainer-mesh 2x2 --inference-mesh 2x2 --device cpu

`--scenario moe` runs `moe_worker.py`: a 2-D HSDP trainer mesh plus a 3-D expert mesh, eight named pairs, fused
qkv / gate-up tensors registered as views, and rounds gated on control keys (see that file).

Same process layout as the reference's launcher (examples/vllm_weight_sync/launch.py:113-143): agents first, then the
two worker groups with `AGENT_RANK_OFFSET` 0 and n.  Exit status 0 iff every inference rank verified its shards.
"""

from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--side-size", type=int, default=1)
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--syncs", type=int, default=3)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--source-dtype", default="bfloat16")
    ap.add_argument("--share-gpu", action="store_true", help="run every agent and worker on GPU 0 (several ranks per GPU)")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--scenario", default="dense", choices=["dense", "moe"])
    ap.add_argument("--trainer-mesh", default="2x2", help="moe scenario: dp_replicate x dp_shard of the trainer side")
    ap.add_argument("--inference-mesh", default="2x2", help="moe scenario: dp x tp of the inference side")
    args = ap.parse_args()
    n = args.side_size
    world = 2 * n
    sides = [("trainer", 0, n), ("inference", n, n)]
    if args.scenario == "moe":
        nt = int(args.trainer_mesh.split("x")[0]) * int(args.trainer_mesh.split("x")[1])
        ni = int(args.inference_mesh.split("x")[0]) * int(args.inference_mesh.split("x")[1])
        world = nt + ni
        sides = [("trainer", 0, nt), ("inference", nt, ni)]
    prefix = os.path.join(tempfile.mkdtemp(prefix="etha_bus_"), "agent_rank")
    master_port, store_port = free_port(), free_port()
    base = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), MASTER_ADDR="127.0.0.1")
    procs: list[tuple[str, subprocess.Popen]] = []

    def spawn(tag, argv, env):
        procs.append((tag, subprocess.Popen([sys.executable, *argv], env=env)))

    for r in range(world):
        env = dict(base, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r if args.device == "cuda" and not args.share_gpu else 0),
                   MASTER_PORT=str(master_port))
        argv = ["-m", "etha_b200.tensor_bus.agent_main", "--store-port", str(store_port), "--path-prefix", prefix]
        if args.device == "cpu":
            argv += ["--device", "cpu"]
        spawn(f"agent{r}", argv, env)
    for role, offset, size in sides:
        for r in range(size):
            env = dict(base, RANK=str(r), WORLD_SIZE=str(size), LOCAL_RANK=str(r + offset if args.device == "cuda" and not args.share_gpu else 0),
                       AGENT_RANK_OFFSET=str(offset))
            if args.scenario == "moe":
                argv = [os.path.join(HERE, "moe_worker.py"), "--role", role, "--trainer-mesh", args.trainer_mesh,
                        "--inference-mesh", args.inference_mesh, "--rounds", str(args.syncs), "--path-prefix", prefix,
                        "--store-port", str(store_port), "--device", args.device]
            else:
                argv = [os.path.join(HERE, "worker.py"), "--role", role, "--model", args.model, "--side-size", str(n),
                        "--syncs", str(args.syncs), "--path-prefix", prefix, "--device", args.device,
                        "--source-dtype", args.source_dtype]
            spawn(f"{role}{r}", argv, env)
    deadline = time.time() + args.timeout
    workers = [(t, p) for t, p in procs if not t.startswith("agent")]
    status = 0
    try:
        for tag, p in workers:
            try:
                rc = p.wait(timeout=max(1.0, deadline - time.time()))
            except subprocess.TimeoutExpired:
                rc = 124
            if rc != 0:
                print(f"[launch] {tag} exited with {rc}", flush=True)
                status = 1
    finally:
        for tag, p in procs:
            if p.poll() is None:
                p.terminate()
        for tag, p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()
    print(f"[launch] {'all inference ranks verified their shards' if status == 0 else 'FAILED'}", flush=True)
    return status


if __name__ == "__main__":
    sys.exit(main())
