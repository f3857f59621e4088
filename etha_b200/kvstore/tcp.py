"""KVStore over `torch.distributed.TCPStore` (reference: src/etha/kvstore/tcp.py:19-236).

TCPStore can neither list a prefix nor delete reliably across versions, so `wait_for_keys` needs the
caller's `candidate_keys`, deletion stores an empty value, and binary values are base64 text.
"""

from __future__ import annotations

import base64
import logging
from datetime import timedelta

import torch.distributed as dist

from .base import KVStore

logger = logging.getLogger(__name__)

POLL_INTERVAL = 0.001


class TorchTCPStore(KVStore):
    poll_interval = POLL_INTERVAL

    def __init__(
        self,
        host: str,
        port: int,
        world_size: int,
        is_master: bool,
        timeout: float = 3600.0,
        wait_for_workers: bool = True,
        namespace: str = "default",
        component: str = "tensorbus",
    ):
        super().__init__(namespace, component)
        self.host, self.port, self.world_size, self.is_master = host, port, world_size, is_master
        self._store = dist.TCPStore(
            host_name=host,
            port=port,
            world_size=world_size,
            is_master=is_master,
            timeout=timedelta(seconds=timeout),
            wait_for_workers=wait_for_workers,
        )
        self._known_keys: set[str] = set()
        logger.info("TorchTCPStore %s:%s master=%s world=%s ns=%s", host, port, is_master, world_size, namespace)

    @classmethod
    def wrap(cls, store: "dist.Store", namespace: str = "default", component: str = "tensorbus") -> "TorchTCPStore":
        """Reuse an existing c10d store (e.g. the one torchrun created) instead of opening a port."""
        self = cls.__new__(cls)
        KVStore.__init__(self, namespace, component)
        self.host = self.port = None
        self.world_size, self.is_master = -1, False
        self._store = store
        self._known_keys = set()
        return self

    def set(self, key: str, value: str, *, component: str | None = None) -> None:
        self._store.set(self._prefixed(key, component), value)
        self._known_keys.add(key)

    def get(self, key: str, *, component: str | None = None) -> bytes | None:
        k = self._prefixed(key, component)
        if not self._store.check([k]):
            return None
        # `TCPStore.get` would block for the whole store timeout if another process deleted the key between the check
        # and the read; a compare-and-set that changes nothing returns the current value and never waits (if the key
        # did vanish, it comes back empty, which every reader here treats as missing)
        v = self._store.compare_set(k, "", "")
        return v if v else None

    def exists(self, key: str, *, component: str | None = None) -> bool:
        return bool(self._store.check([self._prefixed(key, component)]))

    def delete(self, key: str, *, component: str | None = None) -> bool:
        k = self._prefixed(key, component)
        if not self._store.check([k]):
            return False
        try:
            self._store.delete_key(k)
        except Exception:  # a c10d store without delete: an empty value stands for "missing"
            self._store.set(k, "")
        self._known_keys.discard(key)
        return True

    def num_keys(self) -> int | None:
        """Keys held by the server (all namespaces), where the store can tell."""
        try:
            return int(self._store.num_keys())
        except Exception:
            return None

    def set_bytes(self, key: str, data: bytes, *, component: str | None = None) -> None:
        self._store.set(self._prefixed(key, component), base64.b64encode(data).decode("ascii"))
        self._known_keys.add(key)

    def get_bytes(self, key: str, *, component: str | None = None) -> bytes | None:
        v = self.get(key, component=component)
        return None if v is None else base64.b64decode(v)

    def wait_for_keys(self, key_pattern, expected_count, value="1", timeout=3600.0, candidate_keys=None, *, component=None):
        if candidate_keys is None:
            raise ValueError(
                "TorchTCPStore.wait_for_keys requires candidate_keys parameter. TCPStore doesn't support prefix listing."
            )
        return super().wait_for_keys(key_pattern, expected_count, value, timeout, candidate_keys, component=component)

    # TCPStore has an atomic counter: a barrier costs one round trip per poll instead of two per participant, and
    # one counter serves every round (round k is complete when it reaches k x participants)
    def counter_add(self, key: str, amount: int = 1, *, component: str | None = None) -> int:
        return int(self._store.add(self._prefixed(key, component), amount))

    def barrier_arrive(self, key_prefix: str, rank: int, round_no: int = 1, n_ranks: int | None = None, *,
                       component: str | None = None) -> None:  # noqa: ARG002
        self._store.add(self._prefixed(f"{key_prefix}/count", component), 1)

    def barrier_count(self, key_prefix: str, ranks: list[int], round_no: int = 1, *, component: str | None = None) -> int:
        done = int(self._store.add(self._prefixed(f"{key_prefix}/count", component), 0)) - (round_no - 1) * len(ranks)
        return max(0, min(done, len(ranks)))

    def barrier_forget(self, key_prefix: str, rank: int, *, component: str | None = None) -> None:  # noqa: ARG002
        try:
            self._store.delete_key(self._prefixed(f"{key_prefix}/count", component))
        except Exception:  # a c10d store without delete: one counter per barrier name is left behind
            pass

    def close(self, cleanup: bool = True) -> None:  # noqa: ARG002
        self._store = None
