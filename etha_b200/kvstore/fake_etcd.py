"""A tiny in-process etcd v3 JSON gateway (put / range / deleterange / watch) for tests and for boxes with no
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
        self._watchers: list = []
        self._stopping = False
        outer = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"  # as the real gateway: keep-alive answers and chunked watch streams

            def log_message(self, *a):  # silence
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                op = self.path.rsplit("/", 1)[-1]
                if op == "watch":
                    return outer._serve_watch(self, body)
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

    def _serve_watch(self, handler, body: dict) -> None:
        """`/v3/watch`: a chunked stream of JSON lines, first `created`, then one line per matching put / delete."""
        import queue

        req = body.get("create_request", {})
        key = base64.b64decode(req.get("key", ""))
        end = base64.b64decode(req["range_end"]) if "range_end" in req else None
        q: "queue.Queue[dict]" = queue.Queue()
        match = (lambda k: k == key) if end is None else (lambda k: key <= k and (end == b"\0" or k < end))
        with self._lock:
            self._watchers.append((match, q))
        handler.send_response(200)
        handler.send_header("Content-Type", "application/json")
        handler.send_header("Transfer-Encoding", "chunked")
        handler.end_headers()

        def send(obj) -> bool:
            raw = json.dumps(obj).encode() + b"\n"
            try:
                handler.wfile.write(f"{len(raw):x}\r\n".encode() + raw + b"\r\n")
                handler.wfile.flush()
                return True
            except OSError:
                return False

        try:
            if not send({"result": {"header": {"revision": str(self._revision)}, "created": True}}):
                return
            while not self._stopping:
                try:
                    ev = q.get(timeout=0.2)
                except queue.Empty:
                    continue
                if not send({"result": {"header": {"revision": str(self._revision)}, "events": [ev]}}):
                    return
        finally:
            handler.close_connection = True
            with self._lock:
                self._watchers = [w for w in self._watchers if w[1] is not q]

    def _notify(self, key: bytes, value: bytes | None) -> None:
        enc = lambda b: base64.b64encode(b).decode("ascii")
        kv = {"key": enc(key), "mod_revision": str(self._revision)}
        if value:
            kv["value"] = enc(value)
        ev = {"kv": kv} if value is not None else {"type": "DELETE", "kv": kv}
        for match, q in self._watchers:
            if match(key):
                q.put(ev)

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
                self._notify(base64.b64decode(body["key"]), base64.b64decode(body.get("value", "")))
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
                    self._notify(k, None)
                if keys:
                    self._revision += 1
                return dict(header, **({"deleted": str(len(keys))} if keys else {}))
        return {"error": f"unknown op {op}"}

    def start(self) -> "FakeEtcdGateway":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stopping = True
        self._server.shutdown()
        self._server.server_close()
