"""KVStore over etcd v3 through its HTTP/JSON gateway (`/v3/kv/put|range|deleterange`).

The reference uses the `etcd3` gRPC client with watches (src/etha/kvstore/etcd.py:17-232).  That package
is not available here, so this backend speaks the gateway every etcd >= 3.4 serves on the client port,
with only the standard library.  Waits poll a prefix `range` (one request returns every candidate), so
`wait_for_keys` needs no `candidate_keys`; values are stored raw (bytes), as in the reference.
"""

from __future__ import annotations

import base64
import fnmatch
import json
import logging
import time
import urllib.error
import urllib.request

from .base import KVStore

logger = logging.getLogger(__name__)


def _b64(b: bytes) -> str:
    return base64.b64encode(b).decode("ascii")


def _prefix_end(prefix: bytes) -> bytes:
    """Smallest key greater than every key with this prefix (etcd range_end convention)."""
    b = bytearray(prefix)
    while b:
        if b[-1] < 0xFF:
            b[-1] += 1
            return bytes(b)
        b.pop()
    return b"\0"


class EtcdStore(KVStore):
    poll_interval = 0.005

    def __init__(
        self,
        host: str = "localhost",
        port: int = 2379,
        timeout: float | None = None,
        cleanup: bool = False,
        namespace: str = "default",
        component: str = "tensorbus",
    ):
        super().__init__(namespace, component)
        self.host, self.port = host, port
        self._url = f"http://{host}:{port}/v3/kv/"
        self._timeout = min(timeout, 30.0) if timeout else 30.0
        self._closed = False
        self._call("range", {"key": _b64(b"\0"), "limit": 1})  # fail fast if nothing answers
        if cleanup:
            self._delete_prefix(f"{namespace}/")

    def _call(self, op: str, body: dict) -> dict:
        req = urllib.request.Request(
            self._url + op, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"}, method="POST"
        )
        try:
            with urllib.request.urlopen(req, timeout=self._timeout) as resp:
                return json.loads(resp.read() or b"{}")
        except urllib.error.URLError as e:
            raise ConnectionError(f"etcd gateway {self._url}{op}: {e}") from e

    def _range_prefix(self, prefix: str) -> list[tuple[str, bytes]]:
        p = prefix.encode()
        out = self._call("range", {"key": _b64(p), "range_end": _b64(_prefix_end(p))})
        return [(base64.b64decode(kv["key"]).decode(), base64.b64decode(kv.get("value", ""))) for kv in out.get("kvs", [])]

    def _delete_prefix(self, prefix: str) -> int:
        p = prefix.encode()
        out = self._call("deleterange", {"key": _b64(p), "range_end": _b64(_prefix_end(p))})
        return int(out.get("deleted", 0))

    def set(self, key: str, value: str, *, component: str | None = None) -> None:
        self.set_bytes(key, value.encode(), component=component)

    def set_bytes(self, key: str, data: bytes, *, component: str | None = None) -> None:
        self._call("put", {"key": _b64(self._prefixed(key, component).encode()), "value": _b64(data)})

    def get(self, key: str, *, component: str | None = None) -> bytes | None:
        out = self._call("range", {"key": _b64(self._prefixed(key, component).encode())})
        kvs = out.get("kvs", [])
        return base64.b64decode(kvs[0].get("value", "")) if kvs else None

    def get_bytes(self, key: str, *, component: str | None = None) -> bytes | None:
        return self.get(key, component=component)

    def exists(self, key: str, *, component: str | None = None) -> bool:
        return self.get(key, component=component) is not None

    def delete(self, key: str, *, component: str | None = None) -> bool:
        out = self._call("deleterange", {"key": _b64(self._prefixed(key, component).encode())})
        return int(out.get("deleted", 0)) > 0

    def wait_for_key(self, key: str, timeout: float = 3600.0, *, component: str | None = None) -> bytes:
        deadline = time.monotonic() + timeout
        while True:
            v = self.get(key, component=component)
            if v is not None:
                return v
            if time.monotonic() >= deadline:
                raise TimeoutError(f"Timeout waiting for key: {key}")
            time.sleep(self.poll_interval)

    def poll_keys(self, key_pattern, value="1", candidate_keys=None, *, component=None):  # noqa: ARG002
        pattern = self._prefixed(key_pattern, component)
        prefix = pattern[: pattern.find("*")] if "*" in pattern else pattern
        want = value.encode()
        return sorted(self._strip_prefix(k) for k, v in self._range_prefix(prefix) if v == want and fnmatch.fnmatch(k, pattern))

    def close(self, cleanup: bool = True) -> None:
        if self._closed:
            return
        if cleanup:
            n = self._delete_prefix(f"{self.namespace}/")
            logger.info("EtcdStore: deleted %d keys under %s/", n, self.namespace)
        self._closed = True
