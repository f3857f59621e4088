"""Native queue and KV store against simple Python models under random operation sequences."""

import os
from collections import deque

from hypothesis import given, settings
from hypothesis import strategies as st

from etha_b200.ops.hostlib import ShmKV, ShmQueue

_ops = st.lists(
    st.one_of(
        st.tuples(st.just("push"), st.binary(min_size=0, max_size=300)),
        st.tuples(st.just("pop"), st.just(b"")),
        st.tuples(st.just("peek"), st.just(b"")),
        st.tuples(st.just("reopen"), st.just(b"")),
        st.tuples(st.just("clear"), st.just(b"")),
    ),
    max_size=120,
)


@settings(max_examples=60, deadline=None)
@given(_ops)
def test_queue_behaves_like_a_bounded_deque(tmp_path_factory, ops):
    path = str(tmp_path_factory.mktemp("q") / "q.bin")
    cap, data_bytes = 5, 1024
    q = ShmQueue(path, cap, data_bytes)
    model: deque[bytes] = deque()
    try:
        for op, payload in ops:
            if op == "push":
                pos = q.push(payload)
                if pos >= 0:
                    model.append(payload)
                else:
                    # refused: either the slot count or the byte ring is exhausted, never silently dropped
                    assert len(model) == cap or pos in (ShmQueue.FULL_BYTES, ShmQueue.TOO_BIG)
            elif op == "pop":
                got = q.pop()
                assert got == (model.popleft() if model else None)
            elif op == "peek":
                assert q.peek() == (model[0] if model else None)
            elif op == "reopen":
                q.close()
                q = ShmQueue(path, cap, data_bytes)
            else:
                q.clear()
                model.clear()
            assert q.size() == len(model)
    finally:
        q.close()
        os.unlink(path)


@settings(max_examples=40, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["put", "del", "get"]), st.integers(0, 40), st.binary(max_size=64)), max_size=200))
def test_kv_behaves_like_a_dict(tmp_path_factory, ops):
    path = str(tmp_path_factory.mktemp("kv") / "kv.bin")
    kv = ShmKV(path, nslots=64)
    reader = ShmKV(path, create=False, readonly=True)
    model: dict[bytes, bytes] = {}
    try:
        for op, k, v in ops:
            key = f"key:{k}".encode()
            if op == "put":
                kv.put(key, v)
                model[key] = v
            elif op == "del":
                assert kv.delete(key) == (model.pop(key, None) is not None)
            assert reader.get(key) == model.get(key)
            assert len(kv) == len(model)
    finally:
        kv.close()
        reader.close()
        os.unlink(path)
