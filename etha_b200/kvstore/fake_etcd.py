"""A tiny in-process etcd v3 JSON gateway (put / range / deleterange) for tests and for boxes with no
etcd binary.  Not a consensus store: one process, one dict, enough to exercise `EtcdStore`.

Answers are shaped like the real gateway's proto3 JSON: 64-bit integers are strings (`"count": "3"`,
`"deleted": "1"`, `"revision": "17"`) and fields holding a default value are left out altogether (no `kvs` for an
empty range, no `value` for an empty value, no `deleted` when nothing was deleted)."""

from __future__ import annotations

import base64
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


class FakeEtcdGateway:
    def __init__(self, host: str = "127.0.0.1", port: int = 0):
        self._data: dict[bytes, bytes] = {}
        self._lock = threading.Lock()
        self._revision = 1
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):  # silence
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                op = self.path.rsplit("/", 1)[-1]
                out = outer._handle(op, body)
                raw = json.dumps(out).encode()
                self.send_response(200)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                self.wfile.write(raw)

        self._server = ThreadingHTTPServer((host, port), Handler)
        self.host, self.port = self._server.server_address[:2]
        self._thread = threading.Thread(target=self._server.serve_forever, daemon=True)

    def _select(self, body: dict) -> list[bytes]:
        key = base64.b64decode(body.get("key", ""))
        end = base64.b64decode(body["range_end"]) if "range_end" in body else None
        if end is None:
            return [key] if key in self._data else []
        if end == b"\0":
            return sorted(k for k in self._data if k >= key)
        return sorted(k for k in self._data if key <= k < end)

    def _handle(self, op: str, body: dict) -> dict:
        with self._lock:
            header = {"header": {"cluster_id": "1", "member_id": "1", "revision": str(self._revision), "raft_term": "2"}}
            if op == "put":
                self._revision += 1
                self._data[base64.b64decode(body["key"])] = base64.b64decode(body.get("value", ""))
                return header
            if op == "range":
                keys = self._select(body)
                limit = int(body.get("limit", 0))
                if limit:
                    keys = keys[:limit]
                enc = lambda b: base64.b64encode(b).decode("ascii")
                out = dict(header)
                if keys:
                    out["kvs"] = [dict({"key": enc(k), "mod_revision": str(self._revision)},
                                       **({"value": enc(self._data[k])} if self._data[k] else {})) for k in keys]
                    out["count"] = str(len(keys))
                return out
            if op == "deleterange":
                keys = self._select(body)
                for k in keys:
                    del self._data[k]
                if keys:
                    self._revision += 1
                return dict(header, **({"deleted": str(len(keys))} if keys else {}))
        return {"error": f"unknown op {op}"}

    def start(self) -> "FakeEtcdGateway":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._server.shutdown()
        self._server.server_close()
