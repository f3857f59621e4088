"""Control flow of the agent's peer-to-peer transfer step with the device stubbed out: what is launched, which
completion path is taken (device-side wait, or the store when two agents share a GPU), and what is published."""

import torch

from etha_b200.tensor_bus.agent_handlers import AgentHandlers
from etha_b200.tensor_bus.batch_state import BatchState


class FakeEvent:
    def __init__(self, enable_timing=False):
        self.polls = 0

    def record(self, stream=None):
        pass

    def query(self):
        self.polls += 1
        return self.polls >= 3  # the copies "take" two polls

    def elapsed_time(self, other):
        return 1.25


class FakeStore:
    def __init__(self):
        self.sets, self.reached = [], {}

    def set(self, key, value, component=None):
        self.sets.append((key, value, component))

    def mark_reached(self, prefix, rank, n, component=None):
        self.reached[(prefix, rank)] = n

    def count_reached(self, prefix, ranks, n, component=None):
        return sum(1 for r in ranks if self.reached.get((prefix, r), 0) >= n)


class FakeState:
    def __init__(self):
        self.kv = {}

    def put(self, key, value):
        self.kv[key] = value


class FakeExec:
    def __init__(self, producers, consumers):
        self._producers, self._consumers = producers, consumers
        self.calls, self.epoch = [], 0

    def begin(self):
        self.epoch += 1
        self.calls.append(("begin", self.epoch))

    def send(self, stream):
        self.calls.append(("send",))

    def recv(self, stream, timeout_s):
        self.calls.append(("recv", timeout_s))

    def check(self):
        self.calls.append(("check",))


def _agent(monkeypatch, rank):
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: object())
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    a = AgentHandlers.__new__(AgentHandlers)
    a.rank, a.device, a.store, a.state, a.store_timeout = rank, torch.device("cpu"), FakeStore(), FakeState(), 30.0
    return a


def _drive(gen, limit=100):
    steps = 0
    for _ in gen:
        steps += 1
        assert steps < limit, "the transfer step never finished"
    return steps


def test_sender_launches_publishes_and_needs_no_wait(monkeypatch):
    a = _agent(monkeypatch, 0)
    batch = BatchState(batch_id="b", pair_names=["w"], local_leader=0, key="batch:b/gen:1")
    ex = FakeExec(producers=[], consumers=[1])
    steps = _drive(a._p2p_transfer(batch, ex, True, 4, "batch:b/state:transfer_signal"))
    assert steps == 2 and ex.calls == [("begin", 4), ("send",), ("check",)] and ex.epoch == 4
    assert ("batch:b/state:transfer_signal", "1", "global") in a.store.sets
    assert a.state.kv["batch:b/state:last_send_device_ms"] == b"1.250"
    assert not a.store.reached  # no other agent on this GPU: completion is the flags' business


def test_receiver_waits_on_the_device_unless_the_gpu_is_shared(monkeypatch):
    a = _agent(monkeypatch, 1)
    batch = BatchState(batch_id="b", pair_names=["w"], local_leader=1, key="batch:b/gen:1")
    ex = FakeExec(producers=[0], consumers=[])
    _drive(a._p2p_transfer(batch, ex, False, 1, None))
    assert ex.calls == [("begin", 1), ("recv", 30.0), ("check",)] and not a.store.sets

    # two agents on one GPU: never a device-side spin; the producer's store key ends the wait
    b = _agent(monkeypatch, 1)
    shared = BatchState(batch_id="b", pair_names=["w"], local_leader=1, key="batch:b/gen:1", shared_gpu=True,
                        any_shared_gpu=True)
    ex2 = FakeExec(producers=[0], consumers=[])
    gen = b._p2p_transfer(shared, ex2, False, 2, None)
    for _ in range(10):
        next(gen)  # still waiting: the producer has not published transfer 2
    b.store.mark_reached("batch:b/gen:1/done", 0, 2)
    _drive(gen)
    assert ("recv", 30.0) not in ex2.calls and ex2.calls[0] == ("begin", 2)

    # the producing side of a shared GPU publishes its completion
    c = _agent(monkeypatch, 0)
    ex3 = FakeExec(producers=[], consumers=[1])
    _drive(c._p2p_transfer(shared, ex3, True, 2, None))
    assert c.store.reached == {("batch:b/gen:1/done", 0): 2} and shared.wrote_done
