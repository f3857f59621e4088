"""Command queue behaviours (list taken from the reference's tests/test_command_queue.py): FIFO, tagged
union round trip, batch dequeue, peek, clear, 1000 messages, persistence, destroy, capacity, wrap-around,
blocking enqueue released by a consumer thread, two handles sharing the semaphores."""

import json
import threading
import time
import uuid

import msgspec
import pytest

from etha_b200.tensor_bus import CleanupBatch, CommandQueue, InitPair, QueryStatus, QueueFullError, RegisterTensors, Transfer
from etha_b200.tensor_bus.commands import Message


@pytest.fixture
def qpath(tmp_path):
    return str(tmp_path / f"cq_{uuid.uuid4().hex[:8]}.lmdb")


@pytest.fixture
def queue(qpath):
    q = CommandQueue(qpath, capacity=64)
    yield q
    q.close()


def test_wire_format_is_tagged_by_class_name():
    raw = msgspec.json.encode(Transfer(batch_id="b", transfer_type="send", timestamp=1.0, semaphore_name="/s"))
    assert json.loads(raw) == {"type": "Transfer", "batch_id": "b", "transfer_type": "send", "timestamp": 1.0, "semaphore_name": "/s"}
    back = msgspec.msgpack.decode(msgspec.msgpack.encode(InitPair(pair_name="p", local_name="a", expected_world_size=2, remote_name="b",
                                  mesh_shape_payload=memoryview(b"\x01\x02"))), type=Message)
    assert isinstance(back, InitPair) and bytes(back.mesh_shape_payload) == b"\x01\x02" and back.placements_payload is None


def test_fifo_and_types(queue):
    msgs = [
        InitPair(pair_name="p", local_name="t", expected_world_size=4, remote_name="i"),
        RegisterTensors(batch_id="b", tensors=[("p", memoryview(b"abc")), ("p", memoryview(b"defg"))], bucket_size=1 << 20),
        Transfer(batch_id="b", transfer_type="recv"),
        QueryStatus(batch_id="b", state_name="transfer_signal"),
        CleanupBatch(batch_id="b"),
    ]
    for i, m in enumerate(msgs):
        assert queue.enqueue(m) == i
    assert queue.size() == 5 and not queue.is_empty()
    out = [queue.dequeue() for _ in range(5)]
    assert [type(m) for m in out] == [type(m) for m in msgs]
    assert [bytes(p) for _, p in out[1].tensors] == [b"abc", b"defg"] and out[1].bucket_size == 1 << 20
    assert queue.dequeue() is None and queue.is_empty()


def test_peek_batch_clear(queue):
    for i in range(10):
        queue.enqueue(CleanupBatch(batch_id=str(i)))
    assert queue.peek().batch_id == "0" and queue.size() == 10
    got = queue.dequeue_batch(max_count=4)
    assert [m.batch_id for m in got] == ["0", "1", "2", "3"] and queue.size() == 6
    queue.clear()
    assert queue.size() == 0 and queue.dequeue() is None and queue.peek() is None
    for i in range(64):  # full capacity is available again
        queue.enqueue(CleanupBatch(batch_id=str(i)), block=False)
    with pytest.raises(QueueFullError):
        queue.enqueue(CleanupBatch(batch_id="x"), block=False)


def test_thousand_messages_and_wrap_around(qpath):
    q = CommandQueue(qpath, capacity=16)
    n = 0
    for round_ in range(70):
        for _ in range(15):
            q.enqueue(Transfer(batch_id=str(n), transfer_type="send"))
            n += 1
        for k in range(15):
            assert q.dequeue().batch_id == str(n - 15 + k)
    assert n > 1000 and q.is_empty()
    q.close()


def test_persistence_across_reopen(qpath):
    q = CommandQueue(qpath, capacity=32)
    for i in range(5):
        q.enqueue(CleanupBatch(batch_id=str(i)))
    q.dequeue()
    q.close(destroy=False)
    q2 = CommandQueue(qpath, capacity=32)
    assert q2.size() == 4 and q2.dequeue().batch_id == "1"
    q2.close()
    q2.close()  # idempotent
    q3 = CommandQueue(qpath, capacity=32)  # destroyed: starts empty
    assert q3.size() == 0
    q3.close()


def test_capacity_and_timeout(qpath):
    q = CommandQueue(qpath, capacity=3)
    for i in range(3):
        q.enqueue(CleanupBatch(batch_id=str(i)), block=False)
    t0 = time.monotonic()
    with pytest.raises(QueueFullError):
        q.enqueue(CleanupBatch(batch_id="late"), block=True, timeout=0.2)
    assert 0.15 < time.monotonic() - t0 < 1.5
    q.close()


def test_blocking_enqueue_released_by_consumer(qpath):
    q = CommandQueue(qpath, capacity=2)
    q.enqueue(CleanupBatch(batch_id="0"))
    q.enqueue(CleanupBatch(batch_id="1"))
    threading.Timer(0.4, lambda: q.dequeue()).start()
    t0 = time.monotonic()
    q.enqueue(CleanupBatch(batch_id="2"), block=True, timeout=5.0)
    assert 0.3 < time.monotonic() - t0 < 2.0
    assert [q.dequeue().batch_id, q.dequeue().batch_id] == ["1", "2"]
    q.close()


def test_blocking_dequeue_and_two_handles_share_semaphores(qpath):
    producer = CommandQueue(qpath, capacity=8)
    consumer = CommandQueue(qpath, capacity=8)  # follower: opens what the leader created
    assert consumer.dequeue(block=True, timeout=0.05) is None
    threading.Timer(0.2, lambda: producer.enqueue(Transfer(batch_id="z", transfer_type="send"))).start()
    msg = consumer.dequeue(block=True, timeout=5.0)
    assert msg is not None and msg.batch_id == "z"
    consumer.close(destroy=False)
    producer.close()


def test_large_payload(queue):
    blob = bytes(200_000)
    queue.enqueue(RegisterTensors(batch_id="big", tensors=[("p", memoryview(blob))] * 3))
    m = queue.dequeue()
    assert len(m.tensors) == 3 and len(bytes(m.tensors[0][1])) == 200_000
