"""KV store abstraction for distributed coordination (reference: src/etha/kvstore/__init__.py:11-59)."""

import os
from typing import Literal

from .base import KVStore
from .etcd import EtcdStore
from .tcp import TorchTCPStore


def create_store(
    host: str = "localhost",
    port: int | None = None,
    backend: Literal["etcd", "tcp"] = "tcp",
    timeout: float = 3600.0,
    namespace: str = "default",
    component: str = "tensorbus",
) -> KVStore:
    """`tcp`: rank 0 (env RANK) hosts a TCPStore for WORLD_SIZE clients on `port` (default 29500);
    `etcd`: connect to an etcd v3 gateway on `port` (default 2379)."""
    rank = int(os.environ.get("RANK", 0))
    if backend == "etcd":
        return EtcdStore(host=host, port=port or 2379, timeout=timeout, cleanup=False, namespace=namespace, component=component)
    world_size = int(os.environ.get("WORLD_SIZE", 1))
    return TorchTCPStore(
        host=host,
        port=port or 29500,
        world_size=world_size,
        is_master=(rank == 0),
        timeout=timeout,
        wait_for_workers=True,
        namespace=namespace,
        component=component,
    )


__all__ = ["KVStore", "EtcdStore", "TorchTCPStore", "create_store"]
