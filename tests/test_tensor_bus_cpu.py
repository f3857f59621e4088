"""Whole tensor bus on CPU/gloo, world_size=4: agents (one thread per rank next to its worker), KV rendezvous
over TCPStore, command queue + semaphores, shared-memory tensor hand-over, both transfer directions, a Partial
pair, bf16 wire, the error channel and heartbeat handling."""

import os
import threading
import time
import uuid

import pytest
import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from etha_b200.comm.baselines import local_slice_of
from etha_b200.kvstore import TorchTCPStore
from etha_b200.tensor_bus.agent import TensorBusAgent
from etha_b200.tensor_bus.client import TensorBusClient, TensorBusError

from dist_utils import free_port, run_distributed

# includes the unevenly sharded shapes (1000 x 333 over 2 column shards, 7 rows over 2 row shards)
SHAPES = [(1024, 512), (512, 1024), (2048, 256), (256, 2048), (1000, 333), (7, 4096), (128, 128), (64, 64)]


def _start_agent(rank, world, port, tag, tmp):
    store = TorchTCPStore("127.0.0.1", port, world_size=world, is_master=(rank == 0), timeout=60.0,
                          wait_for_workers=True, namespace=tag)
    cq, st = f"{tmp}/{tag}_r{rank}_command.lmdb", f"{tmp}/{tag}_r{rank}_state.lmdb"
    agent = TensorBusAgent(rank, world, "127.0.0.1", port, cq, st, store_timeout=60.0, store_namespace=tag, store=store,
                           device="cpu")
    th = threading.Thread(target=agent.run, daemon=True)
    th.start()
    return agent, th, cq, st


def _worker(rank, world, port, tag, tmp):
    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        is_trainer = rank < 2
        me, other = ("trainer", "inference") if is_trainer else ("inference", "trainer")
        mesh = torch.tensor([0, 1]) if is_trainer else torch.tensor([2, 3])
        tmesh, imesh = torch.tensor([0, 1]), torch.tensor([2, 3])
        # pairs may be initialised in a different order on the two sides
        order = ["w", "p", "h"] if is_trainer else ["h", "p", "w"]
        plc = {"w": (Shard(0),) if is_trainer else (Shard(1),),
               "p": (Partial(),) if is_trainer else (Replicate(),),
               "h": (Shard(0),) if is_trainer else (Shard(0),)}
        pending = [client.init_pair(name, me, other, 2, mesh, plc[name], blocking=False) for name in order]
        for done in pending:
            done.acquire(30.0)
        assert all(client.state.matched(n) == "matched" for n in order)

        torch.manual_seed(0)
        fulls = [torch.randn(s) for s in SHAPES]
        torch.manual_seed(100)
        part_full = [torch.randn(256, 128) / 2 for _ in range(2)]  # the two trainer contributions
        tensors, mine = [], []
        for f in fulls:
            t = (local_slice_of(f, tmesh, (Shard(0),), rank) if is_trainer else
                 torch.zeros_like(local_slice_of(f, imesh, (Shard(1),), rank))).clone()
            tensors.append((t, "w"))
            mine.append(t)
        p_t = part_full[rank].clone() if is_trainer else torch.zeros(256, 128)
        tensors.append((p_t, "p"))
        half_full = torch.randn(64, 32, generator=torch.Generator().manual_seed(7))
        h_t = (local_slice_of(half_full, tmesh, (Shard(0),), rank).clone() if is_trainer
               else torch.zeros(32, 32, dtype=torch.bfloat16))  # fp32 -> bf16 on the wire and at rest
        tensors.append((h_t, "h"))
        batch = client.register_tensors("sync0", tensors, bucket_size=64 * 1024, timeout=30.0)
        assert batch.pair_names == ["w", "p", "h"]

        for it in range(2):
            if is_trainer:
                batch.transfer("send", blocking=True, timeout=30.0)
            else:
                deadline = time.time() + 20
                while not batch.query_transfer_signal(timeout=10.0):
                    assert time.time() < deadline
                    time.sleep(0.01)
                batch.transfer("recv", blocking=True, timeout=30.0)
                for f, t in zip(fulls, mine):
                    assert torch.equal(t, local_slice_of(f, imesh, (Shard(1),), rank))
                assert torch.equal(p_t, part_full[0] + part_full[1])
                assert torch.equal(h_t, local_slice_of(half_full, imesh, (Shard(0),), rank).to(torch.bfloat16))
                for t in mine:
                    t.zero_()
                p_t.zero_()
        if not is_trainer:  # every send has been consumed: nothing pending
            assert batch.query_transfer_signal(timeout=10.0) is False
        dist_done = client.state.get("batch:sync0/state:last_send_ms" if is_trainer else "batch:sync0/state:last_recv_ms")
        assert dist_done is not None

        # reverse direction on a batch without the Partial pair: inference -> trainer
        back = [(mine[0], "w")]
        if not is_trainer:
            mine[0].copy_(local_slice_of(fulls[1].t().contiguous(), imesh, (Shard(1),), rank))
        b2 = client.register_tensors("sync1", back, timeout=30.0)
        b2.transfer("recv" if is_trainer else "send", blocking=True, timeout=30.0)
        if is_trainer:
            assert torch.equal(mine[0], local_slice_of(fulls[1].t().contiguous(), tmesh, (Shard(0),), rank))

        # a Partial target direction is refused with a readable error, and the agent stays alive
        with pytest.raises(TensorBusError, match="Partial"):
            batch.transfer("recv" if is_trainer else "send", blocking=True, timeout=30.0)
        with pytest.raises(TensorBusError, match="unknown batch"):
            client.transfer("nope", "send", blocking=True, timeout=10.0)
        assert client.state.heartbeat_age() < 2.0
        b2.close()
        batch.close()
    finally:
        dist.barrier()
        agent.stop()
        th.join(timeout=5)
        client.close()
        agent.command_queue.close(destroy=True)
        agent.state.close()


def test_bus_end_to_end_cpu(tmp_path):
    run_distributed(_worker, 4, free_port(), "t" + uuid.uuid4().hex[:6], str(tmp_path))


def test_client_rejects_stale_or_missing_agent(tmp_path):
    from etha_b200.tensor_bus.state_store import StateStore

    with pytest.raises(ConnectionError, match="not found"):
        TensorBusClient(0, str(tmp_path / "cq.lmdb"), str(tmp_path / "absent_state.lmdb"), connection_timeout=0.3)
    path = str(tmp_path / "state.lmdb")
    s = StateStore(path)
    s.put("agent:heartbeat", str(time.time() - 60).encode())  # an agent that died a minute ago
    with pytest.raises(ConnectionError, match="not responding"):
        TensorBusClient(0, str(tmp_path / "cq.lmdb"), path, connection_timeout=0.5)
    s.close()


def test_command_without_agent_times_out(tmp_path):
    from etha_b200.tensor_bus.state_store import StateStore

    path = str(tmp_path / "state.lmdb")
    s = StateStore(path)
    s.beat()
    c = TensorBusClient(0, str(tmp_path / f"cq_{uuid.uuid4().hex[:6]}.lmdb"), path, connection_timeout=2.0)
    with pytest.raises(TimeoutError):
        c.transfer("b", "send", blocking=True, timeout=0.3)  # nobody ever posts the semaphore
    c.command_queue.close(destroy=True)
    s.close()


def _absent_peer_worker(rank, world, port, tag, tmp):
    """Only rank 0's worker ever declares the pair: the other side never shows up (an agent whose worker died
    before init_pair).  The waiting agent gives up after its store timeout, reports it, and keeps serving."""
    store = TorchTCPStore("127.0.0.1", port, world_size=world, is_master=(rank == 0), timeout=60.0,
                          wait_for_workers=True, namespace=tag)
    cq, st = f"{tmp}/{tag}_r{rank}_command.lmdb", f"{tmp}/{tag}_r{rank}_state.lmdb"
    agent = TensorBusAgent(rank, world, "127.0.0.1", port, cq, st, store_timeout=1.0, store_namespace=tag, store=store,
                           device="cpu")
    th = threading.Thread(target=agent.run, daemon=True)
    th.start()
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        if rank == 0:
            t0 = time.monotonic()
            pending = client.init_pair("lonely", "trainer", "inference", 1, torch.tensor([0]), (Shard(0),), blocking=False)
            worst = 0.0
            while time.monotonic() - t0 < 0.8:  # the handshake is still waiting: the heartbeat must stay fresh
                worst = max(worst, client.state.heartbeat_age())
                time.sleep(0.05)
            assert worst < 1.0
            with pytest.raises(TensorBusError, match="did not complete within"):
                pending.acquire(20.0)
            assert 0.9 < time.monotonic() - t0 < 10.0
            assert client.state.matched("lonely") is None
            # the agent is still alive and answers the next command
            with pytest.raises(TensorBusError, match="unknown batch"):
                client.transfer("nope", "recv", blocking=True, timeout=10.0)
            assert client.state.heartbeat_age() < 2.0
    finally:
        dist.barrier()
        agent.stop()
        th.join(timeout=5)
        client.close()
        agent.command_queue.close(destroy=True)
        agent.state.close()


def test_peer_that_never_registers_times_out_cleanly(tmp_path):
    run_distributed(_absent_peer_worker, 2, free_port(), "t" + uuid.uuid4().hex[:6], str(tmp_path))
