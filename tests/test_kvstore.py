"""KV store behaviours on both backends (TCPStore in-process; etcd through an in-process JSON gateway).
Mirrors the behaviour list of the reference's tests/test_kvstore.py."""

import threading
import time

import pytest

from etha_b200.kvstore import EtcdStore, TorchTCPStore, create_store
from etha_b200.kvstore.fake_etcd import FakeEtcdGateway

from conftest import free_port


@pytest.fixture(params=["tcp", "etcd"])
def store(request):
    if request.param == "tcp":
        s = TorchTCPStore("127.0.0.1", free_port(), world_size=1, is_master=True, timeout=10.0,
                          wait_for_workers=False, namespace="ns", component="tensorbus")
        yield s
        s.close()
    else:
        gw = FakeEtcdGateway().start()
        s = EtcdStore(gw.host, gw.port, timeout=5.0, namespace="ns")
        yield s
        s.close()
        gw.stop()


def test_set_get_exists_delete(store):
    assert store.get("a") is None and not store.exists("a")
    store.set("a", "1")
    assert store.get("a") == b"1" and store.exists("a")
    store.set("a", "2")
    assert store.get("a") == b"2"
    assert store.delete("a") is True
    assert not store.try_get("a")
    assert store.delete("never-there") is False


def test_bytes_roundtrip(store):
    blob = bytes(range(256)) * 9
    store.set_bytes("blob", blob)
    assert store.get_bytes("blob") == blob
    assert store.get_bytes("missing") is None


def test_component_and_namespace_isolation(store):
    store.set("k", "local")
    store.set("k", "global", component="global")
    assert store.get("k") == b"local" and store.get("k", component="global") == b"global"
    assert store._prefixed("k") == "ns/tensorbus/k" and store._strip_prefix("ns/tensorbus/pair:x/rank:1/y") == "pair:x/rank:1/y"
    if isinstance(store, EtcdStore):
        other = EtcdStore(store.host, store.port, namespace="other")
        assert other.get("k") is None
        other.close(cleanup=False)


def test_wait_for_key_existing_async_timeout(store):
    store.set("ready", "yes")
    assert store.wait_for_key("ready", timeout=1.0) == b"yes"
    threading.Timer(0.15, lambda: store.set("later", "v")).start()
    t0 = time.monotonic()
    assert store.wait_for_key("later", timeout=5.0) == b"v"
    assert 0.1 < time.monotonic() - t0 < 3.0
    with pytest.raises(TimeoutError):
        store.wait_for_key("never", timeout=0.1)


def test_wait_for_value(store):
    store.set("state", "0")
    threading.Timer(0.1, lambda: store.set("state", "1")).start()
    assert store.wait_for_value("state", "1", timeout=5.0) == b"1"
    with pytest.raises(TimeoutError):
        store.wait_for_value("state", "7", timeout=0.1)


def test_wait_for_keys_pattern_value_and_async(store):
    cands = [f"pair:p/rank:{r}/trainer" for r in range(8)]
    for r in (0, 1):
        store.set(cands[r], "1")
    store.set("pair:p/rank:5/trainer", "0")  # wrong value: must not count
    store.set("pair:q/rank:0/trainer", "1")  # other pair: must not match
    got = store.wait_for_keys("pair:p/rank:*/trainer", 2, timeout=1.0, candidate_keys=cands)
    assert got == [cands[0], cands[1]]

    def writer():
        time.sleep(0.1)
        store.set(cands[2], "1")
        store.set(cands[3], "1")

    threading.Thread(target=writer).start()
    got = store.wait_for_keys("pair:p/rank:*/trainer", 4, timeout=5.0, candidate_keys=cands)
    assert got == cands[:4]
    with pytest.raises(TimeoutError, match="got 4"):
        store.wait_for_keys("pair:p/rank:*/trainer", 6, timeout=0.1, candidate_keys=cands)
    assert store.poll_keys("pair:p/rank:*/trainer", "0", cands) == ["pair:p/rank:5/trainer"]


def test_tcp_needs_candidate_keys_etcd_does_not(store):
    store.set("x/1", "1")
    if isinstance(store, TorchTCPStore):
        with pytest.raises(ValueError, match="candidate_keys"):
            store.wait_for_keys("x/*", 1, timeout=0.1)
    else:
        assert store.wait_for_keys("x/*", 1, timeout=1.0) == ["x/1"]


def test_etcd_cleanup_removes_namespace():
    gw = FakeEtcdGateway().start()
    a = EtcdStore(gw.host, gw.port, namespace="n1")
    b = EtcdStore(gw.host, gw.port, namespace="n2")
    a.set("k", "1"), b.set("k", "1")
    a.close(cleanup=True)
    assert b.get("k") == b"1"
    c = EtcdStore(gw.host, gw.port, namespace="n1")
    assert c.get("k") is None
    gw.stop()


def test_etcd_unreachable_fails_fast():
    with pytest.raises(ConnectionError):
        EtcdStore("127.0.0.1", free_port(), timeout=0.5)


def test_create_store_factory(monkeypatch):
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    s = create_store("127.0.0.1", free_port(), backend="tcp", timeout=10.0, namespace="abc")
    assert isinstance(s, TorchTCPStore) and s.is_master and s.namespace == "abc"
    gw = FakeEtcdGateway().start()
    e = create_store(gw.host, gw.port, backend="etcd", namespace="abc")
    assert isinstance(e, EtcdStore)
    gw.stop()


def test_barrier_helpers(store):
    ranks = [0, 1, 2]
    assert store.barrier_count("b/go:1", ranks) == 0
    store.barrier_arrive("b/go:1", 0)
    store.barrier_arrive("b/go:1", 2)
    assert store.barrier_count("b/go:1", ranks) == 2
    store.barrier_arrive("b/go:1", 1)
    assert store.barrier_count("b/go:1", ranks) == 3
    assert store.barrier_count("b/go:2", ranks) == 0  # another barrier is independent
    # the same keys serve the next rounds: nothing new is left behind per round
    assert store.barrier_count("b/go:1", ranks, 2) == 0
    for r in ranks:
        store.barrier_arrive("b/go:1", r, 2)
    assert store.barrier_count("b/go:1", ranks, 2) == 3 and store.barrier_count("b/go:1", ranks, 1) == 3
    assert store.barrier_count("b/go:1", ranks, 3) == 0
    for r in ranks:
        store.barrier_forget("b/go:1", r)
    assert store.barrier_count("b/go:1", ranks) == 0
    # counters
    assert store.counter_add("b/gen") == 1 and store.counter_add("b/gen") == 2 and store.counter_add("b/gen", 0) == 2


def test_etcd_client_accepts_proto3_json_shapes():
    """The gateway writes int64 fields as strings and leaves out fields with default values: no `kvs` for an empty
    range, no `value` for an empty value, no `deleted` when nothing matched."""
    gw = FakeEtcdGateway().start()
    try:
        s = EtcdStore(gw.host, gw.port, namespace="p3")
        assert s.get("missing") is None and s.exists("missing") is False
        assert s.delete("missing") is False
        s.set("empty", "")
        assert s.get("empty") == b"" and s.exists("empty") is True
        assert s.try_get("empty") is None
        s.set_bytes("bin", b"\x00\x01")
        s.set("pair:x/rank:0/a", "1")
        s.set("pair:x/rank:1/a", "1")
        assert s.poll_keys("pair:x/rank:*/a") == ["pair:x/rank:0/a", "pair:x/rank:1/a"]
        assert s.poll_keys("pair:y/rank:*/a") == []
        assert s.delete("bin") is True and s.get_bytes("bin") is None
        assert s.counter_add("n") == 1 and s.counter_add("n", 2) == 3
        s.close(cleanup=True)
        assert EtcdStore(gw.host, gw.port, namespace="p3").get("empty") is None
    finally:
        gw.stop()


def test_etcd_waits_sleep_on_a_watch_stream():
    """Blocking waits open a watch, check once, and then issue no request until an event arrives."""
    import threading
    import time

    gw = FakeEtcdGateway().start()
    try:
        s = EtcdStore(gw.host, gw.port, namespace="w")
        writer = EtcdStore(gw.host, gw.port, namespace="w")
        calls = {"range": 0}
        real = s._call

        def counting(op, body):
            calls[op] = calls.get(op, 0) + 1
            return real(op, body)

        s._call = counting
        threading.Timer(0.4, lambda: writer.set("late", "v")).start()
        t0 = time.monotonic()
        assert s.wait_for_key("late", timeout=5.0) == b"v"
        assert 0.3 < time.monotonic() - t0 < 3.0
        assert calls["range"] <= 3, f"{calls['range']} range requests: the wait polled instead of watching"
        # several keys under a prefix, arriving one by one
        calls["range"] = 0
        for i, delay in enumerate((0.1, 0.2, 0.3)):
            threading.Timer(delay, lambda i=i: writer.set(f"pair:p/rank:{i}/t", "1")).start()
        got = s.wait_for_keys("pair:p/rank:*/t", 3, timeout=5.0)
        assert got == [f"pair:p/rank:{i}/t" for i in range(3)] and calls["range"] <= 6
        threading.Timer(0.2, lambda: writer.set("state", "ready")).start()
        writer.set("state", "starting")
        assert s.wait_for_value("state", "ready", timeout=5.0) == b"ready"
        with pytest.raises(TimeoutError):
            s.wait_for_key("never", timeout=0.3)
        with pytest.raises(TimeoutError):
            s.wait_for_keys("pair:q/rank:*/t", 1, timeout=0.3)
    finally:
        gw.stop()


def test_tcp_get_never_blocks_on_a_key_deleted_under_it():
    """Another process may delete a key between this store's existence check and its read (a batch cleanup racing
    with a status query): the read must come back empty at once, not wait for the store timeout."""
    import time

    s = TorchTCPStore("127.0.0.1", free_port(), world_size=1, is_master=True, timeout=30.0, wait_for_workers=False, namespace="race")
    s.set("k", "v")
    assert s.get("k") == b"v"
    real = s._store

    class CheckSaysYes:
        def __getattr__(self, name):
            return getattr(real, name)

        def check(self, keys):
            return True  # as if the key had existed a moment ago

    s._store = CheckSaysYes()
    t0 = time.monotonic()
    assert s.get("gone") is None and s.try_get("gone") is None and s.get_bytes("gone") is None
    assert time.monotonic() - t0 < 2.0
    assert s.get("k") == b"v"
