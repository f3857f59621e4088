"""NVLS multicast fan-out reached through the public bus API: inference workers allocate their Replicate targets with
`TensorBusClient.empty_replicated`, the agents bind those arenas into one multicast team, and the producer's copy table
writes every replica with `multimem.st` (`multicast_ops > 0`).  One agent and one worker process per GPU."""

import json
import os
import socket
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(consumers: int, arena: int):
    world = consumers + 1
    prefix = os.path.join(tempfile.mkdtemp(prefix="etha_nvls_"), "agent_rank")
    # every child logs to a file (kept when ETHA_TEST_LOG_DIR names a directory), so a run that is cut short still
    # leaves its output behind
    log_dir = os.environ.get("ETHA_TEST_LOG_DIR") or os.path.dirname(prefix)
    os.makedirs(log_dir, exist_ok=True)
    logs = []

    def log_file(tag):
        path = os.path.join(log_dir, f"nvls_bus_{'arena' if arena else 'plain'}_{tag}.log")
        logs.append(path)
        return open(path, "w")

    master, store = _free_port(), _free_port()
    base = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT")}
    base.update(PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), MASTER_ADDR="127.0.0.1",
                NCCL_NVLS_ENABLE="0", ETHA_NVLS_MIN_REPLICAS="1")
    agents, workers = [], []
    try:
        for r in range(world):
            env = dict(base, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_PORT=str(master))
            agents.append(subprocess.Popen([sys.executable, "-m", "etha_b200.tensor_bus.agent_main", "--store-port", str(store),
                                            "--path-prefix", prefix, "--log-level", "INFO"], env=env, stdout=log_file(f"agent{r}"),
                                           stderr=subprocess.STDOUT, text=True))
        for r in range(world):
            env = dict(base, LOCAL_RANK=str(r))
            workers.append(subprocess.Popen([sys.executable, os.path.join(HERE, "bus_nvls_worker.py"), "--agent-rank", str(r),
                                             "--consumers", str(consumers), "--path-prefix", prefix, "--arena", str(arena)],
                                            env=env, stdout=log_file(f"worker{r}"), stderr=subprocess.STDOUT, text=True))
        outs = []
        for r, w in enumerate(workers):
            try:
                w.wait(timeout=400)
            except subprocess.TimeoutExpired:
                w.kill()
                w.wait()
            outs.append((w.returncode, open(os.path.join(log_dir, f"nvls_bus_{'arena' if arena else 'plain'}_worker{r}.log")).read()))
    finally:
        for p in agents:
            if p.poll() is None:
                p.terminate()  # SIGTERM: the agent leaves its multicast teams and unmaps before it exits
        for p in agents:
            try:
                p.wait(timeout=60)
            except subprocess.TimeoutExpired:
                p.kill()
                p.wait()
        agent_logs = [open(path).read() for path in logs if "agent" in os.path.basename(path)]
    text = "\n".join(o for _, o in outs) + "\n--- agents ---\n" + "\n".join(a[-1500:] for a in agent_logs)
    assert all(rc == 0 for rc, _ in outs), text[-6000:]
    results = [json.loads(line) for _, o in outs for line in o.splitlines() if line.startswith("{")]
    assert len(results) == world and all(r["bad"] == 0 for r in results), text[-6000:]
    return {r["agent_rank"]: r for r in results}, text


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(900)
def test_replicated_arena_targets_are_written_by_multicast():
    import torch

    from etha_b200.ops import device_info

    torch.cuda.set_device(0)
    if not device_info()["multicast"]:
        pytest.skip("multicast not supported on this machine")
    consumers = 2 if torch.cuda.device_count() >= 3 else 1
    res, text = _run(consumers, arena=1)  # replicas are bit-exact whichever way they were written
    if res[0]["multicast_ops"] == 0 and "no multicast team" in text:
        pytest.xfail("the agents could not bind the workers' arenas to a multicast object here and fell back to peer stores")
    assert res[0]["multicast_ops"] == 3, text[-4000:]  # the three replicated tensors; the sharded one is a plain peer store


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(900)
def test_ordinary_replicate_targets_fall_back_to_peer_stores():
    import torch

    consumers = 2 if torch.cuda.device_count() >= 3 else 1
    res, text = _run(consumers, arena=0)
    assert res[0]["multicast_ops"] == 0, text[-4000:]
