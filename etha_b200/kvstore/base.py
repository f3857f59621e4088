"""Key/value rendezvous interface shared by the agents (reference: src/etha/kvstore/base.py:6-213).

Keys live under `{namespace}/{component}/{key}`; a call may override the component.  Ten operations:
`set`, `get`, `exists`, `delete`, `wait_for_key`, `wait_for_keys`, `set_bytes`, `get_bytes`,
`wait_for_value`, `close`.  Two non-blocking helpers (`poll_keys`, `try_get`) are added for the agent's
handshake state machine, which never blocks its command loop.
"""

from __future__ import annotations

import fnmatch
import time
from abc import ABC, abstractmethod


class KVStore(ABC):
    namespace: str
    component: str

    def __init__(self, namespace: str, component: str):
        self.namespace = namespace
        self.component = component

    # ---- key helpers ------------------------------------------------------------------------
    def _prefixed(self, key: str, component: str | None = None) -> str:
        return f"{self.namespace}/{component or self.component}/{key}"

    def _strip_prefix(self, key: str) -> str:
        parts = key.split("/", 2)
        return parts[2] if len(parts) > 2 else key

    # ---- required operations -----------------------------------------------------------------
    @abstractmethod
    def set(self, key: str, value: str, *, component: str | None = None) -> None: ...

    @abstractmethod
    def get(self, key: str, *, component: str | None = None) -> bytes | None: ...

    @abstractmethod
    def exists(self, key: str, *, component: str | None = None) -> bool: ...

    @abstractmethod
    def delete(self, key: str, *, component: str | None = None) -> bool: ...

    @abstractmethod
    def set_bytes(self, key: str, data: bytes, *, component: str | None = None) -> None: ...

    @abstractmethod
    def get_bytes(self, key: str, *, component: str | None = None) -> bytes | None: ...

    @abstractmethod
    def close(self, cleanup: bool = True) -> None: ...

    # ---- waits: generic polling implementations, backends may override with watches ------------
    poll_interval = 0.001

    def wait_for_key(self, key: str, timeout: float = 3600.0, *, component: str | None = None) -> bytes:
        deadline = time.monotonic() + timeout
        while True:
            v = self.get(key, component=component)
            if v:
                return v
            if time.monotonic() >= deadline:
                raise TimeoutError(f"Timeout waiting for key: {key}")
            time.sleep(self.poll_interval)

    def wait_for_value(self, key: str, expected: str, timeout: float = 3600.0, *, component: str | None = None) -> bytes:
        want = expected.encode()
        deadline = time.monotonic() + timeout
        while True:
            v = self.get(key, component=component)
            if v == want:
                return v
            if time.monotonic() >= deadline:
                raise TimeoutError(f"Timeout waiting for key '{key}' to have value '{expected}'")
            time.sleep(self.poll_interval)

    def poll_keys(
        self, key_pattern: str, value: str = "1", candidate_keys: list[str] | None = None, *, component: str | None = None
    ) -> list[str]:
        """Keys matching `key_pattern` whose value is `value`, right now (no waiting)."""
        if candidate_keys is None:
            raise ValueError(f"{type(self).__name__}.wait_for_keys requires candidate_keys: the backend cannot list a prefix")
        want = value.encode()
        out = []
        for k in candidate_keys:
            if fnmatch.fnmatch(k, key_pattern) and self.get(k, component=component) == want:
                out.append(k)
        return sorted(out)

    def wait_for_keys(
        self,
        key_pattern: str,
        expected_count: int,
        value: str = "1",
        timeout: float = 3600.0,
        candidate_keys: list[str] | None = None,
        *,
        component: str | None = None,
    ) -> list[str]:
        deadline = time.monotonic() + timeout
        found: list[str] = []
        while True:
            found = self.poll_keys(key_pattern, value, candidate_keys, component=component)
            if len(found) >= expected_count:
                return found[:expected_count]
            if time.monotonic() >= deadline:
                raise TimeoutError(f"Timeout waiting for {expected_count} keys matching '{key_pattern}', got {len(found)}")
            time.sleep(self.poll_interval)

    # ---- counters and the reusable rendezvous of a known set of ranks ---------------------------------
    def counter_add(self, key: str, amount: int = 1, *, component: str | None = None) -> int:
        """Add to an integer key and return the new value.  This default is only safe when one writer owns the
        key; backends with an atomic add override it."""
        raw = self.try_get(key, component=component)
        value = (int(raw.decode()) if raw else 0) + amount
        if amount:
            self.set(key, str(value), component=component)
        return value

    def mark_reached(self, key_prefix: str, rank: int, n: int, *, component: str | None = None) -> None:
        """Record that `rank` has reached step `n` of the progress named `key_prefix` (one key per rank, overwritten)."""
        self.set(f"{key_prefix}/rank:{rank}", str(n), component=component)

    def count_reached(self, key_prefix: str, ranks: list[int], n: int, *, component: str | None = None) -> int:
        """How many of `ranks` have reached step `n` (one poll, no waiting); any subset of the ranks may be asked."""
        count = 0
        for r in ranks:
            raw = self.try_get(f"{key_prefix}/rank:{r}", component=component)
            if raw and int(raw.decode()) >= n:
                count += 1
        return count

    def barrier_arrive(self, key_prefix: str, rank: int, round_no: int = 1, n_ranks: int | None = None, *,
                       component: str | None = None) -> None:
        """Announce `rank` at round `round_no` (1, 2, ...) of the barrier named `key_prefix`.  The same keys are
        reused by every round, so a barrier that runs once per transfer leaves a fixed number of keys behind.
        Every round must be asked about with the same full list of participants (`n_ranks` of them, for backends
        that want to recognise the last arrival)."""
        self.mark_reached(key_prefix, rank, round_no, component=component)

    def barrier_wait(self, key_prefix: str, ranks: list[int], round_no: int = 1, timeout_s: float = 0.0, *,
                     component: str | None = None) -> bool:
        """True once every rank of `ranks` has arrived at round `round_no`.  `timeout_s` is how long a backend may
        sleep on a server-side notification; the generic form polls once and returns.  (TCPStore's own `wait` is not
        used for this: a wait that times out costs milliseconds and leaves its answer pending on the connection.)"""
        return self.barrier_count(key_prefix, ranks, round_no, component=component) >= len(ranks)

    def barrier_count(self, key_prefix: str, ranks: list[int], round_no: int = 1, *, component: str | None = None) -> int:
        """How many of `ranks` have reached round `round_no` (one poll, no waiting)."""
        return self.count_reached(key_prefix, ranks, round_no, component=component)

    def barrier_forget(self, key_prefix: str, rank: int, *, component: str | None = None) -> None:
        """Drop what `rank` left at a barrier that will not be used again."""
        self.delete(f"{key_prefix}/rank:{rank}", component=component)

    def try_get(self, key: str, *, component: str | None = None) -> bytes | None:
        """`get` that treats an empty value (a deleted key on backends without delete) as missing."""
        v = self.get(key, component=component)
        return v if v else None
