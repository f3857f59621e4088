"""KVStore over etcd v3 through its HTTP/JSON gateway (`/v3/kv/put|range|deleterange`).

The reference uses the `etcd3` gRPC client with watches (src/etha/kvstore/etcd.py:17-232).  That package
is not available here, so this backend speaks the gateway every etcd >= 3.4 serves on the client port,
with only the standard library.  Blocking waits follow the reference's watch-before-check pattern
(src/etha/kvstore/etcd.py:81-123): open a `/v3/watch` stream on the key or prefix, wait for its `created`
answer, look at the current state with one `range`, and then sleep on the stream until an event arrives —
no polling while nothing changes.  A gateway without the watch endpoint makes the wait fall back to polling.
`wait_for_keys` ranges a prefix, so it needs no `candidate_keys`; values are stored raw (bytes), as in the
reference.
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


_NO_WATCH = object()  # the gateway offers no usable watch stream: the caller polls instead


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

    # ---- watch ----------------------------------------------------------------------------------
    def _wait_with_watch(self, key: bytes, range_end: bytes | None, check, timeout: float):
        """Watch-before-check: `check()` is evaluated once the watch exists and again after every event on the
        watched key range; returns its first non-None result.  Raises TimeoutError; returns the sentinel `_NO_WATCH`
        if the gateway has no watch endpoint."""
        import http.client
        import socket

        deadline = time.monotonic() + timeout
        conn = http.client.HTTPConnection(self.host, self.port, timeout=min(self._timeout, max(timeout, 0.05)))
        try:
            create = {"key": _b64(key)}
            if range_end is not None:
                create["range_end"] = _b64(range_end)
            try:
                conn.request("POST", "/v3/watch", body=json.dumps({"create_request": create}),
                             headers={"Content-Type": "application/json"})
                resp = conn.getresponse()
                if resp.status != 200:
                    return _NO_WATCH
                first = resp.readline()
                if not first or not json.loads(first).get("result", {}).get("created"):
                    return _NO_WATCH
            except (OSError, ValueError, http.client.HTTPException):
                return _NO_WATCH
            while True:
                got = check()
                if got is not None:
                    return got
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError
                sock = conn.sock or getattr(getattr(resp.fp, "raw", None), "_sock", None)
                if sock is None:
                    return _NO_WATCH
                sock.settimeout(left)
                try:
                    line = resp.readline()  # blocks until the next event (or the deadline)
                except (socket.timeout, TimeoutError):
                    raise TimeoutError from None
                except OSError:
                    return _NO_WATCH
                if not line:
                    return _NO_WATCH  # the stream ended: let the caller poll
        finally:
            conn.close()

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
        try:
            got = self._wait_with_watch(self._prefixed(key, component).encode(), None,
                                        lambda: self.get(key, component=component), timeout)
        except TimeoutError:
            raise TimeoutError(f"Timeout waiting for key: {key}") from None
        if got is not _NO_WATCH:
            return got
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

    def wait_for_value(self, key: str, expected: str, timeout: float = 3600.0, *, component: str | None = None) -> bytes:
        want = expected.encode()
        t0 = time.monotonic()

        def check():
            v = self.get(key, component=component)
            return v if v == want else None

        try:
            got = self._wait_with_watch(self._prefixed(key, component).encode(), None, check, timeout)
        except TimeoutError:
            raise TimeoutError(f"Timeout waiting for key '{key}' to have value '{expected}'") from None
        if got is not _NO_WATCH:
            return got
        return super().wait_for_value(key, expected, max(timeout - (time.monotonic() - t0), 0.0), component=component)

    def wait_for_keys(self, key_pattern, expected_count, value="1", timeout=3600.0, candidate_keys=None, *, component=None):
        pattern = self._prefixed(key_pattern, component)
        prefix = (pattern[: pattern.find("*")] if "*" in pattern else pattern).encode()
        t0 = time.monotonic()

        def check():
            found = self.poll_keys(key_pattern, value, candidate_keys, component=component)
            return found[:expected_count] if len(found) >= expected_count else None

        try:
            got = self._wait_with_watch(prefix, _prefix_end(prefix), check, timeout)
        except TimeoutError:
            n = len(self.poll_keys(key_pattern, value, candidate_keys, component=component))
            raise TimeoutError(f"Timeout waiting for {expected_count} keys matching '{key_pattern}', got {n}") from None
        if got is not _NO_WATCH:
            return got
        return super().wait_for_keys(key_pattern, expected_count, value, max(timeout - (time.monotonic() - t0), 0.0),
                                     candidate_keys, component=component)

    def close(self, cleanup: bool = True) -> None:
        if self._closed:
            return
        if cleanup:
            n = self._delete_prefix(f"{self.namespace}/")
            logger.info("EtcdStore: deleted %d keys under %s/", n, self.namespace)
        self._closed = True
