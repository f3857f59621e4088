"""Life cycle of registrations on the tensor bus (CPU/gloo, world_size=2): re-registering a batch id, many
register / transfer / cleanup cycles with a flat number of keys, meshes whose ranks are not ascending, expiry of
error messages, and the queue's item/semaphore pairing."""

import threading
import time

import pytest
import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Replicate, Shard

from etha_b200.comm.baselines import local_slice_of
from etha_b200.tensor_bus.client import TensorBusClient, TensorBusError

from dist_utils import free_port, run_distributed
from test_tensor_bus_cpu import _start_agent


def _teardown(agent, th, client):
    dist.barrier()
    agent.stop()
    th.join(timeout=5)
    client.close()
    agent.command_queue.close(destroy=True)
    agent.state.close()


def _reregister_worker(rank, world, port, tag, tmp):
    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        sender = rank == 0
        me, other = ("trainer", "inference") if sender else ("inference", "trainer")
        client.init_pair("w", me, other, 1, torch.tensor([rank]), (Replicate(),), timeout=30.0)
        # the same batch id three times, each time with other tensors (other shapes, other storage): a registration
        # must never see descriptors, barrier counts or epochs of the one before
        for round_no, shape in enumerate([(64, 32), (16, 8), (128, 4)]):
            g = torch.Generator().manual_seed(round_no)
            want = torch.randn(shape, generator=g)
            t = want.clone() if sender else torch.zeros(shape)
            batch = client.register_tensors("weight_sync", [(t, "w")], timeout=30.0)
            for step in range(2):
                if sender:
                    t.copy_(want * (step + 1))
                    batch.transfer("send", blocking=True, timeout=30.0)
                else:
                    batch.transfer("recv", blocking=True, timeout=30.0)
                    assert torch.equal(t, want * (step + 1)), f"registration {round_no}, transfer {step}"
                dist.barrier()
            if not sender:
                assert batch.query_transfer_signal(timeout=10.0) is False
            if round_no != 1:
                batch.close()  # round 1 is left open on purpose: registering again replaces it
            dist.barrier()
        assert agent.batches == {} or list(agent.batches) == ["weight_sync"]
    finally:
        _teardown(agent, th, client)


def test_same_batch_id_can_be_registered_again(tmp_path):
    run_distributed(_reregister_worker, 2, free_port(), "rereg", str(tmp_path))


CYCLES = 1000


def _cycle_worker(rank, world, port, tag, tmp):
    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        sender = rank == 0
        me, other = ("trainer", "inference") if sender else ("inference", "trainer")
        client.init_pair("w", me, other, 1, torch.tensor([rank]), (Replicate(),), timeout=30.0)
        t = torch.arange(64, dtype=torch.float32) if sender else torch.zeros(64)
        counts = []
        for cycle in range(CYCLES):
            batch = client.register_tensors("cyc", [(t, "w")], timeout=30.0)
            for _ in range(2):
                batch.transfer("send" if sender else "recv", blocking=True, timeout=30.0)
            batch.close()
            if cycle in (20, CYCLES - 1):
                dist.barrier()
                counts.append((agent.store.num_keys(), len(agent.state._kv), len(client._keepalive)))
                dist.barrier()
        if not sender:
            assert torch.equal(t, torch.arange(64, dtype=torch.float32))
        early, late = counts
        # one registration counter per rank is all that may remain; nothing grows with the number of cycles
        assert late[0] is None or late[0] <= early[0], f"store keys grew: {early[0]} -> {late[0]}"
        assert late[1] <= early[1], f"state-store slots grew: {early[1]} -> {late[1]}"
        assert late[2] == 0
        dist.barrier()
        import os

        assert not [f for f in os.listdir("/dev/shm") if "etha_nb_" in f], "rendezvous semaphores were left behind"
    finally:
        _teardown(agent, th, client)


@pytest.mark.timeout(600)
def test_register_transfer_cleanup_cycles_leave_nothing_behind(tmp_path):
    run_distributed(_cycle_worker, 2, free_port(), "cycles", str(tmp_path))


def _mesh_order_worker(rank, world, port, tag, tmp):
    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        # trainer ranks 0,1 hold Shard(0) over the mesh [1, 0]: rank 1 owns the FIRST row block; consumers 2,3 use
        # the mesh [3, 2] the same way.  An agent that refilled the meshes in ascending order would swap the halves.
        trainer = rank < 2
        me, other = ("trainer", "inference") if trainer else ("inference", "trainer")
        mesh = torch.tensor([1, 0]) if trainer else torch.tensor([3, 2])
        client.init_pair("w", me, other, 2, mesh, (Shard(0),) if trainer else (Shard(1),), timeout=30.0)
        full = torch.randn(8, 6, generator=torch.Generator().manual_seed(3))
        mine = local_slice_of(full, mesh, (Shard(0),) if trainer else (Shard(1),), rank).clone()
        t = mine if trainer else torch.zeros_like(mine)
        batch = client.register_tensors("order", [(t, "w")], timeout=30.0)
        batch.transfer("send" if trainer else "recv", blocking=True, timeout=30.0)
        if not trainer:
            assert torch.equal(t, mine)
        batch.close()
    finally:
        _teardown(agent, th, client)


def test_mesh_rank_order_is_honoured(tmp_path):
    run_distributed(_mesh_order_worker, 4, free_port(), "order", str(tmp_path))


def _error_ttl_worker(rank, world, port, tag, tmp):
    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    agent.error_ttl_s = 0.3
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        before = len(agent.state._kv)
        for _ in range(5):
            with pytest.raises(TensorBusError, match="unknown batch"):
                client.transfer("nope", "send", blocking=True, timeout=10.0)
        assert len(agent.state._kv) == before + 5  # the messages stay readable for a while ...
        time.sleep(0.5)
        client.init_pair("solo", "a", "a", 1, torch.tensor([0]), (Replicate(),), timeout=10.0)  # any command turns the loop
        deadline = time.time() + 5
        while len(agent.state._kv) > before + 1 and time.time() < deadline:
            time.sleep(0.05)
        assert len(agent.state._kv) <= before + 1  # ... and are then removed (the pair's match key is new)
    finally:
        _teardown(agent, th, client)


def test_error_messages_expire(tmp_path):
    run_distributed(_error_ttl_worker, 1, free_port(), "errttl", str(tmp_path))


def test_queue_item_and_semaphore_stay_paired(tmp_path):
    """A consumer polling without blocking while a producer sits between its push and its semaphore post must not
    take the item early: afterwards a blocking dequeue on the empty queue has to wait out its timeout."""
    from etha_b200.tensor_bus.command_queue import CommandQueue
    from etha_b200.tensor_bus.commands import CleanupBatch

    q = CommandQueue(str(tmp_path / "pairing.lmdb"), capacity=16)
    try:
        real_release = q._sem.release
        gate = threading.Event()
        pushed = threading.Event()

        def slow_release():
            pushed.set()
            gate.wait(5.0)
            real_release()

        q._sem.release = slow_release
        producer = threading.Thread(target=lambda: q.enqueue(CleanupBatch(batch_id="x")))
        producer.start()
        assert pushed.wait(5.0)
        assert q.size() == 1
        assert q.dequeue(block=False) is None  # pushed, not yet posted: not delivered
        gate.set()
        producer.join()
        q._sem.release = real_release
        got = q.dequeue(block=True, timeout=1.0)
        assert isinstance(got, CleanupBatch) and got.batch_id == "x"
        t0 = time.monotonic()
        assert q.dequeue(block=True, timeout=0.3) is None
        assert time.monotonic() - t0 >= 0.25, "a blocking dequeue on an empty queue returned before its timeout"
    finally:
        q.close(destroy=True)


def test_export_failure_names_the_unsupported_allocators(monkeypatch):
    """Worker memory that has no CUDA IPC handle (expandable segments, VMM pools) must fail with a message that says
    so; the native call is replaced by one that fails the way cudaIpcGetMemHandle does on such memory."""
    from etha_b200.parallel import peer as peer_mod

    class FakeLib:
        def etha_ipc_export(self, ptr, handle, base, size):
            return -1001

    class FakeTensor:
        is_cuda = True
        shape = (4, 4)
        dtype = torch.float32
        device = torch.device("cpu")

        def untyped_storage(self):
            return self

        def data_ptr(self):
            return 4096

    import contextlib

    pm = peer_mod.PeerMemory.__new__(peer_mod.PeerMemory)
    pm._lib, pm._arenas, pm._exported, pm._keepalive, pm.pid = FakeLib(), [], {}, {}, 1
    monkeypatch.setattr(peer_mod.torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(peer_mod.L, "last_error", lambda: "cudaIpcGetMemHandle: invalid argument")
    with pytest.raises(peer_mod.PeerExportError, match="expandable segments") as info:
        pm.describe(FakeTensor())
    assert "VmmArena" in str(info.value) and "invalid argument" in str(info.value)


def _strided_worker(rank, world, port, tag, tmp):
    """FSDP-over-TP target through the bus: 2 trainers hold Shard(0), 4 inference ranks hold
    (_StridedShard(0, split_factor=2), Shard(0)) on a 2x2 mesh — the placement the reference's CPU test uses."""
    from torch.distributed.tensor.placement_types import _StridedShard

    agent, th, cq, st = _start_agent(rank, world, port, tag, tmp)
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        trainer = rank < 2
        me, other = ("trainer", "inference") if trainer else ("inference", "trainer")
        mesh = torch.arange(2) if trainer else torch.arange(2, 6).view(2, 2)
        plc = (Shard(0),) if trainer else (_StridedShard(0, split_factor=2), Shard(0))
        client.init_pair("w", me, other, 2 if trainer else 4, mesh, plc, timeout=30.0)
        full = torch.randn(16, 6, generator=torch.Generator().manual_seed(5))
        mine = local_slice_of(full, mesh, plc, rank).clone()
        t = mine if trainer else torch.zeros_like(mine)
        batch = client.register_tensors("strided", [(t, "w")], timeout=30.0)
        batch.transfer("send" if trainer else "recv", blocking=True, timeout=30.0)
        if not trainer:
            assert torch.equal(t, mine)
        batch.close()
    finally:
        _teardown(agent, th, client)


def test_strided_shard_target_through_the_bus(tmp_path):
    run_distributed(_strided_worker, 6, free_port(), "strided", str(tmp_path))


def _abandoned_worker(rank, world, port, tag, tmp):
    """The receiving worker never asks for the transfer: the send times out with an error, every later transfer of
    that registration is refused, and registering the batch again works."""
    import threading

    from etha_b200.kvstore import TorchTCPStore
    from etha_b200.tensor_bus.agent import TensorBusAgent

    store = TorchTCPStore("127.0.0.1", port, world_size=world, is_master=(rank == 0), timeout=60.0,
                          wait_for_workers=True, namespace=tag)
    cq, st = f"{tmp}/{tag}_r{rank}_command.lmdb", f"{tmp}/{tag}_r{rank}_state.lmdb"
    agent = TensorBusAgent(rank, world, "127.0.0.1", port, cq, st, store_timeout=1.0, store_namespace=tag, store=store,
                           device="cpu")
    th = threading.Thread(target=agent.run, daemon=True)
    th.start()
    client = TensorBusClient(rank, cq, st, connection_timeout=10.0)
    try:
        sender = rank == 0
        me, other = ("trainer", "inference") if sender else ("inference", "trainer")
        client.init_pair("w", me, other, 1, torch.tensor([rank]), (Replicate(),), timeout=30.0)
        t = torch.ones(8) if sender else torch.zeros(8)
        batch = client.register_tensors("ab", [(t, "w")], timeout=30.0)
        if sender:
            with pytest.raises(TensorBusError, match="did not complete within"):
                batch.transfer("send", blocking=True, timeout=20.0)
            with pytest.raises(TensorBusError, match="register it again"):
                batch.transfer("send", blocking=True, timeout=20.0)
        dist.barrier()
        # both sides start over under the same batch id; the old handles lose their claim on it
        batch2 = client.register_tensors("ab", [(t, "w")], timeout=30.0)
        assert batch._closed
        del batch
        batch2.transfer("send" if sender else "recv", blocking=True, timeout=30.0)
        if not sender:
            assert torch.equal(t, torch.ones(8))
        batch2.close()
    finally:
        _teardown(agent, th, client)


def test_abandoned_transfer_poisons_the_registration_not_the_agent(tmp_path):
    run_distributed(_abandoned_worker, 2, free_port(), "abandon", str(tmp_path))
