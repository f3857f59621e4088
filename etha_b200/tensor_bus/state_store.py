"""Agent state visible to its workers: heartbeat, pair match, transfer signal, command errors.

Takes the place of the reference's State LMDB (named db `pair_state`, src/etha/tensor_bus/agent.py:131-144;
keys `agent:heartbeat`, `pair:{pair}/state:match`, `batch:{id}/state:transfer_signal`, values msgpack or
ASCII as there).  The agent is the only writer; workers open the file read-only and take no lock.
One key family is new: `error:{semaphore_name}` holds the message of a command that failed, so that a
worker woken by the semaphore can tell failure from success.
"""

from __future__ import annotations

import time

import msgspec

from ..ops.hostlib import ShmKV

HEARTBEAT_KEY = b"agent:heartbeat"


class StateStore:
    def __init__(self, path: str, readonly: bool = False):
        self.path = str(path)
        self._kv = ShmKV(self.path, create=not readonly, readonly=readonly)

    # raw
    def put(self, key: str | bytes, value: bytes) -> None:
        self._kv.put(key.encode() if isinstance(key, str) else key, value)

    def get(self, key: str | bytes) -> bytes | None:
        return self._kv.get(key.encode() if isinstance(key, str) else key)

    def delete(self, key: str | bytes) -> bool:
        return self._kv.delete(key.encode() if isinstance(key, str) else key)

    # typed helpers
    def beat(self) -> None:
        self._kv.put(HEARTBEAT_KEY, str(time.time()).encode())

    def heartbeat_age(self) -> float | None:
        raw = self._kv.get(HEARTBEAT_KEY)
        return None if not raw else time.time() - float(raw.decode())

    def set_matched(self, pair: str) -> None:
        self.put(f"pair:{pair}/state:match", msgspec.msgpack.encode("matched"))

    def matched(self, pair: str) -> str | None:
        raw = self.get(f"pair:{pair}/state:match")
        return None if raw is None else msgspec.msgpack.decode(raw, type=str)

    def set_signal(self, batch_id: str, name: str, value: bool) -> None:
        self.put(f"batch:{batch_id}/state:{name}", msgspec.msgpack.encode(bool(value)))

    def signal(self, batch_id: str, name: str) -> bool:
        raw = self.get(f"batch:{batch_id}/state:{name}")
        return False if raw is None else msgspec.msgpack.decode(raw, type=bool)

    def set_error(self, semaphore_name: str, message: str) -> None:
        self.put(f"error:{semaphore_name}", message.encode()[:2000])

    def pop_error(self, semaphore_name: str) -> str | None:
        raw = self.get(f"error:{semaphore_name}")
        return None if raw is None else raw.decode(errors="replace")

    def close(self) -> None:
        self._kv.close()
