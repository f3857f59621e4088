#!/usr/bin/env python
"""Micro-benchmark of the KV store backends (counterpart of the reference's bench/kvstore_benchmark.py): per-operation
latency of set / get / exists / set_bytes / get_bytes / wait_for_key / wait_for_keys on TCPStore and on etcd (a real
gateway with --etcd-host/--etcd-port, otherwise the in-process fake gateway).

    python bench/kvstore_benchmark.py --iters 2000 --payload 4096
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from etha_b200.kvstore import EtcdStore, TorchTCPStore  # noqa: E402
from etha_b200.kvstore.fake_etcd import FakeEtcdGateway  # noqa: E402


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def timed(fn, n: int) -> dict:
    samples = []
    for i in range(n):
        t0 = time.perf_counter()
        fn(i)
        samples.append((time.perf_counter() - t0) * 1e6)
    samples.sort()
    return {"mean_us": round(sum(samples) / n, 2), "p50_us": round(samples[n // 2], 2), "p99_us": round(samples[int(n * 0.99) - 1], 2)}


def bench_store(store, name: str, iters: int, payload: int) -> None:
    blob = os.urandom(payload)
    keys = [f"k{i}" for i in range(iters)]
    cands = [f"pair:p/rank:{r}/side" for r in range(8)]
    for k in cands:
        store.set(k, "1")
    ops = {
        "set": lambda i: store.set(keys[i], "1"),
        "get": lambda i: store.get(keys[i]),
        "exists": lambda i: store.exists(keys[i]),
        "set_bytes": lambda i: store.set_bytes("b" + keys[i], blob),
        "get_bytes": lambda i: store.get_bytes("b" + keys[i]),
        "wait_for_key(existing)": lambda i: store.wait_for_key(keys[i], timeout=5.0),
        "wait_for_keys(8 existing)": lambda i: store.wait_for_keys("pair:p/rank:*/side", 8, timeout=5.0, candidate_keys=cands),
    }
    for op, fn in ops.items():
        print(json.dumps({"backend": name, "op": op, "iters": iters, "payload_bytes": payload if "bytes" in op else None,
                          **timed(fn, iters)}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=1000)
    ap.add_argument("--payload", type=int, default=4096)
    ap.add_argument("--backends", default="tcp,etcd")
    ap.add_argument("--etcd-host", default=None)
    ap.add_argument("--etcd-port", type=int, default=2379)
    args = ap.parse_args()
    if "tcp" in args.backends:
        s = TorchTCPStore("127.0.0.1", free_port(), world_size=1, is_master=True, timeout=30.0, wait_for_workers=False, namespace="bench")
        bench_store(s, "tcp", args.iters, args.payload)
        s.close()
    if "etcd" in args.backends:
        gw = None
        if args.etcd_host is None:
            gw = FakeEtcdGateway().start()
            host, port, label = gw.host, gw.port, "etcd(fake gateway)"
        else:
            host, port, label = args.etcd_host, args.etcd_port, "etcd"
        s = EtcdStore(host, port, namespace="bench")
        bench_store(s, label, args.iters, args.payload)
        s.close(cleanup=True)
        if gw:
            gw.stop()


if __name__ == "__main__":
    main()
