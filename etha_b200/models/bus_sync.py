"""Run a weight sync through the whole tensor bus from inside an existing job: spawn one agent per logical
rank, attach `TensorBusClient`s, declare pairs, register tensors and time `transfer("send"|"recv")` rounds.

This is the path a user of the bus takes (`TensorBusClient.init_pair` / `register_tensors` /
`BatchHandler.transfer`, reference: src/etha/tensor_bus/client.py:184-323), as opposed to driving the
executor directly.  Used by `bench.py` for its end-to-end-through-the-bus figure and by the tests.

Rank model: with `world > 1` process `r` owns logical agent rank `r`.  With `world == 1` the single process
plays both sides, so two agents (ranks 0 and 1) are started on the same device and the process holds one
client per side; completion then goes through the KV store (see the agent's shared-GPU rule).
"""

from __future__ import annotations

import os
import socket
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch

from ..tensor_bus.client import TensorBusClient

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _clean_env() -> dict:
    """Environment for a child agent: nothing of an enclosing torchrun job may leak into its own rendezvous."""
    env = {k: v for k, v in os.environ.items() if not k.startswith(("TORCHELASTIC_", "TORCH_NCCL_", "GROUP_", "ROLE_"))}
    for k in ("LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_WORLD_SIZE", "MASTER_PORT", "RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    env["MASTER_ADDR"] = "127.0.0.1"
    return env


@dataclass
class BusItem:
    source: torch.Tensor | None  # this process's shard on the producing side (None if it does not produce)
    target: torch.Tensor | None  # this process's shard on the consuming side
    source_placements: tuple
    target_placements: tuple


def bus_roundtrip(
    rank: int,
    world: int,
    local_device: int,
    items: Sequence[BusItem],
    source_agent_ranks: Sequence[int],
    target_agent_ranks: Sequence[int],
    steps: int,
    warmup: int,
    share: Callable[[Any], Any],
    on_step: Callable[[int, str], None] | None = None,
    device_type: str = "cuda",
    timeout: float = 120.0,
    timer: tuple[Callable[[], None], Callable[[], float]] | None = None,
    source_mesh_shape: Sequence[int] | None = None,
    target_mesh_shape: Sequence[int] | None = None,
) -> dict:
    """Time `steps` sync rounds through the bus.  Returns `{"ms_per_step": wall ms on this process, ...}`.

    `share(obj)` returns rank 0's object on every process (a broadcast; identity when world == 1): it distributes
    the ports and the scratch directory.  `on_step(k, phase)` is called with phase "before_send" on producers and
    "after_recv" on consumers so that the caller can upload / read back a per-step stamp inside the timed region.
    `timer = (start, stop)` replaces the wall clock around the timed rounds (`stop()` returns milliseconds), e.g. a
    pair of CUDA events on the caller's stream.  No collective is issued after the first `share`, so a rank that
    fails cannot strand the others: they run into their own timeouts.
    """
    n_agents = max(world, 2) if world == 1 else world
    my_agents = [0, 1] if world == 1 else [rank]
    cfg = share({"store_port": _free_port(), "agent_port": _free_port(),
                 "prefix": os.path.join(tempfile.mkdtemp(prefix="etha_bus_"), "agent_rank")} if rank == 0 else None)
    prefix = cfg["prefix"]
    paths = lambda r: (f"{prefix}{r}_command.lmdb", f"{prefix}{r}_state.lmdb")
    agents, clients, batches = [], {}, {}
    deadline = time.monotonic() + timeout
    left = lambda: max(1.0, deadline - time.monotonic())
    try:
        for a in my_agents:
            env = _clean_env()
            env.update(RANK=str(a), WORLD_SIZE=str(n_agents), LOCAL_RANK=str(local_device), MASTER_PORT=str(cfg["agent_port"]))
            argv = [sys.executable, "-m", "etha_b200.tensor_bus.agent_main", "--store-port", str(cfg["store_port"]),
                    "--path-prefix", prefix]
            if device_type == "cpu":
                argv += ["--device", "cpu"]
            log = open(f"{prefix}{a}.log", "wb")
            agents.append(subprocess.Popen(argv, env=env, stdout=log, stderr=subprocess.STDOUT))
        for a in my_agents:
            cq, st = paths(a)
            clients[a] = TensorBusClient(a, cq, st, connection_timeout=left())
        smesh, tmesh = torch.tensor(list(source_agent_ranks)), torch.tensor(list(target_agent_ranks))
        if source_mesh_shape is not None:
            smesh = smesh.view(tuple(source_mesh_shape))
        if target_mesh_shape is not None:
            tmesh = tmesh.view(tuple(target_mesh_shape))
        names: dict[tuple, str] = {}
        for it in items:
            names.setdefault((tuple(it.source_placements), tuple(it.target_placements)), f"pair{len(names)}")
        pending = []
        for a, c in clients.items():
            trainer = a in source_agent_ranks
            for (sp, tp), name in names.items():
                pending.append(c.init_pair(name, "trainer" if trainer else "inference", "inference" if trainer else "trainer",
                                           len(source_agent_ranks) if trainer else len(target_agent_ranks),
                                           smesh if trainer else tmesh, sp if trainer else tp, blocking=False))
        for p in pending:
            p.acquire(left())
        for a, c in clients.items():
            trainer = a in source_agent_ranks
            tensors = [((it.source if trainer else it.target), names[(tuple(it.source_placements), tuple(it.target_placements))])
                       for it in items]
            if any(t is None for t, _ in tensors):
                raise ValueError(f"agent rank {a}: a tensor of its side is missing")
            batches[a] = c.register_tensors("bench_weights", tensors, blocking=False)
        for b in batches.values():
            b.wait(left())

        def one_round(k: int) -> None:
            # post both directions first (a process holding both roles must not block on its send before its receive
            # is posted), then wait
            waits = []
            for a in my_agents:
                if a in source_agent_ranks:
                    if on_step:
                        on_step(k, "before_send")
                    waits.append(batches[a].transfer("send", blocking=False))
            for a in my_agents:
                if a in target_agent_ranks:
                    waits.append(batches[a].transfer("recv", blocking=False))
            for w in waits:
                w.acquire(left())
            if on_step and any(a in target_agent_ranks for a in my_agents):
                on_step(k, "after_recv")

        for k in range(warmup):
            one_round(-1 - k)
        t0 = time.perf_counter()
        if timer:
            timer[0]()
        for k in range(steps):
            one_round(k)
        ms = (timer[1]() if timer else (time.perf_counter() - t0) * 1e3) / steps
        dev_ms = None
        for a in my_agents:
            if a in source_agent_ranks:
                raw = clients[a].state.get("batch:bench_weights/state:last_send_device_ms")
                dev_ms = float(raw.decode()) if raw else None
        return {"ms_per_step": ms, "agent_send_device_ms_last": dev_ms, "agents": n_agents}
    finally:
        for b in batches.values():
            try:
                b.close(blocking=False)
            except Exception:
                pass
        for c in clients.values():
            try:
                c.close()
            except Exception:
                pass
        for p in agents:
            if p.poll() is None:
                p.terminate()
        for p in agents:
            try:
                p.wait(timeout=15)
            except subprocess.TimeoutExpired:
                p.kill()
