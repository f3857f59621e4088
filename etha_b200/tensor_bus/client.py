"""Worker-side client of the tensor bus (API of the reference: src/etha/tensor_bus/client.py:30-406).

A worker (trainer rank, inference worker) talks to the agent that owns its GPU through the agent's
command queue; every command carries the name of a fresh POSIX semaphore the agent posts when it is
done.  Tensors are not copied: a CUDA tensor travels as a 64-byte IPC handle plus offset/shape/strides
(`TensorDesc`), a CPU tensor as a shared-memory file name (torch's file-system sharing).

Differences from the reference, on purpose:
* after a command completes the client looks for `error:{semaphore}` in the agent's state store and
  raises `TensorBusError` — in the reference a failed command looks like success (the semaphore is
  posted either way and the agent dies);
* the heartbeat is written by a dedicated agent thread, so a long command does not make it stale.
"""

from __future__ import annotations

import logging
import os
import pickle
import time
import uuid
import weakref
from typing import Literal

import torch

from ..ops.hostlib import O_CREAT, BusyError, Semaphore
from .command_queue import CommandQueue
from .commands import CleanupBatch, InitPair, QueryStatus, RegisterTensors, Transfer
from .state_store import StateStore

logger = logging.getLogger(__name__)

HEARTBEAT_FRESH_S = 5.0


class TensorBusError(RuntimeError):
    """The agent reported that a command failed."""


def generate_semaphore_name(command_type: str, context_id: str) -> str:
    safe = context_id.replace("/", "_").replace(":", "_")
    return f"/command_{command_type}_{safe}_{os.getpid()}_{uuid.uuid4().hex}"


def encode_tensor(t: torch.Tensor, peer=None, arena=None) -> bytes:
    """Serialise a handle to `t` for the agent (never the data).  A tensor inside the client's replicated arena
    carries, next to its descriptor, where the agent can fetch the arena's file descriptor."""
    t = t.detach()
    if t.is_cuda:
        from ..parallel.peer import PeerMemory

        if arena is not None and arena.contains(t):
            import dataclasses

            return pickle.dumps(("cuda", dataclasses.replace(arena.arena.describe(t), arena=arena.ticket())))
        peer = peer or PeerMemory(t.device)
        return pickle.dumps(("cuda", peer.describe(t)))
    # CPU: move the storage to a named shared-memory file any process can open
    import torch.multiprocessing as tmp

    if tmp.get_sharing_strategy() != "file_system":
        tmp.set_sharing_strategy("file_system")
    if not t.is_shared():
        t.share_memory_()
    manager, handle, size = t.untyped_storage()._share_filename_cpu_()
    meta = (manager, handle, size, t.storage_offset(), tuple(t.shape), tuple(t.stride()), str(t.dtype).replace("torch.", ""))
    return pickle.dumps(("cpu", meta))


class ReplicatedArena:
    """Worker-owned block of VMM device memory for tensors every consumer holds in full (Replicate targets).

    Memory from `cudaMalloc` cannot be bound to an NVSwitch multicast object; this arena can.  The worker carves its
    replicated tensors out of it (`TensorBusClient.empty_replicated`), the agent fetches the arena's file descriptor
    once (a Unix socket next to the arena, `SCM_RIGHTS`), binds it into a multicast team with the other agents of the
    batch, and producers then write all replicas with one `multimem.st` pass.  Every consumer must allocate the same
    tensors in the same order, so that a tensor sits at the same offset in every replica's arena."""

    def __init__(self, nbytes: int, device):
        import socket
        import tempfile
        import threading

        from ..parallel.arena import VmmArena

        from ..ops import device_info

        # sized in multiples of the multicast granularity, so that the agents can bind it to a multicast object
        with torch.cuda.device(device):
            multicast = device_info()["multicast"]
        self.arena = VmmArena(nbytes, device, n_team=8 if multicast else 0)
        self._cursor = 0
        self._path = os.path.join(tempfile.gettempdir(), f"etha_arena_{os.getpid()}_{uuid.uuid4().hex[:12]}.sock")
        self._srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._srv.bind(self._path)
        self._srv.listen(8)
        self._srv.settimeout(0.2)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._serve, daemon=True)
        self._thread.start()

    def _serve(self) -> None:
        import socket

        while not self._stop.is_set():
            try:
                conn, _ = self._srv.accept()
            except (TimeoutError, OSError):
                continue
            with conn:
                try:
                    socket.send_fds(conn, [b"fd"], [self.arena.fd])
                    conn.settimeout(5.0)
                    conn.recv(1)  # the agent confirms it holds its duplicate
                except OSError:
                    pass

    def empty(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = dtype.itemsize
        for s in shape:
            n *= int(s)
        off = self._cursor
        if off + n > self.arena.size:
            raise MemoryError(f"replicated arena of {self.arena.size} bytes is full ({off} used, {n} requested): "
                              "create the client with a larger replicated_arena_bytes")
        self._cursor = (off + n + 255) // 256 * 256
        return self.arena.tensor(off, tuple(shape), dtype)

    def contains(self, t: torch.Tensor) -> bool:
        return t.is_cuda and self.arena.va <= t.data_ptr() < self.arena.va + self.arena.size

    def ticket(self) -> dict:
        return {"socket": self._path, "size": self.arena.size, "pid": os.getpid(), "device_index": self.arena.device.index,
                "va": self.arena.va}

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=1.0)
        self._srv.close()
        try:
            os.unlink(self._path)
        except OSError:
            pass
        self.arena.close()


class BatchHandler:
    """Handle of one `register_tensors` call; all its pairs transfer together."""

    def __init__(self, client: "TensorBusClient", batch_id: str, pair_names: list[str]):
        self._client_ref = weakref.ref(client)
        self.batch_id = batch_id
        self.pair_names = pair_names
        self._closed = False
        self._pending = None  # completion of a non-blocking registration

    def wait(self, timeout: float = 30.0) -> "BatchHandler":
        """Wait for a registration started with `blocking=False`."""
        if self._pending is not None:
            self._pending.acquire(timeout)
            self._pending = None
        return self

    @property
    def client(self) -> "TensorBusClient":
        c = self._client_ref()
        if c is None:
            raise RuntimeError("TensorBusClient has been garbage collected. BatchHandler is no longer valid.")
        return c

    def transfer(self, transfer_type: Literal["send", "recv"], blocking: bool = False, timeout: float = 30.0):
        """Start one direction of the batch. Returns the completion handle (`.acquire(timeout)` waits)."""
        return self.client.transfer(self.batch_id, transfer_type, blocking=blocking, timeout=timeout)

    def query_transfer_signal(self, blocking: bool = True, timeout: float = 30.0) -> bool:
        return self.client.query_transfer_signal(self.batch_id, blocking=blocking, timeout=timeout)

    def close(self, blocking: bool = True, timeout: float = 30.0) -> None:
        if self._closed:
            return
        self._closed = True
        client = self.client
        try:
            client._execute_command_with_semaphore(
                CleanupBatch(batch_id=self.batch_id), "cleanup_batch", f"batch_{self.batch_id}", blocking=blocking, timeout=timeout
            )
        finally:
            client._release_batch(self.batch_id)

    def __del__(self):
        try:
            self.close(blocking=False)
        except Exception:
            pass


class Completion:
    """What a non-blocking command returns: wait with `acquire(timeout)`; errors surface there."""

    def __init__(self, client: "TensorBusClient", sem: Semaphore, what: str):
        self._client, self._sem, self._what = client, sem, what
        self.name = sem.name

    def acquire(self, timeout: float | None = None) -> None:
        try:
            self._sem.acquire(timeout)
        except BusyError as e:
            raise TimeoutError(f"{self._what}: no answer from the agent within {timeout}s ({self.name})") from e
        finally:
            pass
        self._sem.close()
        self._client._raise_if_failed(self.name, self._what)

    wait = acquire

    def close(self) -> None:
        self._sem.close()


class TensorBusClient:
    def __init__(
        self,
        agent_rank: int,
        lmdb_command_queue_path: str | None = None,
        agent_state_lmdb_path: str | None = None,
        connection_timeout: float = 30.0,
        replicated_arena_bytes: int | None = None,
    ):
        self.agent_rank = agent_rank
        self.replicated_arena_bytes = replicated_arena_bytes or int(os.environ.get("TENSOR_BUS_REPLICATED_ARENA_BYTES", 256 << 20))
        self._arena: ReplicatedArena | None = None
        if agent_state_lmdb_path is None:
            agent_state_lmdb_path = os.environ.get("TENSOR_BUS_STATE_PATH")
        if agent_state_lmdb_path is None:
            raise ValueError("agent_state_lmdb_path (or TENSOR_BUS_STATE_PATH) is required")
        self.agent_state_lmdb_path = agent_state_lmdb_path
        self.state: StateStore | None = None
        self._connect_agent(agent_state_lmdb_path, connection_timeout)
        if lmdb_command_queue_path is None:
            lmdb_command_queue_path = os.environ.get("TENSOR_BUS_COMMAND_QUEUE_PATH")
        self.command_queue = CommandQueue(lmdb_command_queue_path)
        self._peer = None
        self._keepalive: dict[str, list[torch.Tensor]] = {}
        self._handlers: dict[str, weakref.ref] = {}

    # ---- plumbing ------------------------------------------------------------------------------
    def _raise_if_failed(self, sem_name: str, what: str) -> None:
        err = self.state.pop_error(sem_name) if self.state is not None else None
        if err:
            raise TensorBusError(f"{what} failed on agent {self.agent_rank}: {err}")

    def _execute_command_with_semaphore(self, command, command_type: str, context_id: str, blocking: bool = False,
                                        timeout: float = 30.0) -> Completion:
        name = generate_semaphore_name(command_type, context_id)
        sem = Semaphore(name, O_CREAT, 0)
        command.semaphore_name = name
        command.timestamp = time.time()
        self.command_queue.enqueue(command)
        done = Completion(self, sem, f"{command_type} '{context_id}'")
        if blocking:
            done.acquire(timeout)
        return done

    def _connect_agent(self, path: str, timeout: float) -> None:
        deadline = time.time() + timeout
        while not os.path.exists(path):
            if time.time() > deadline:
                raise ConnectionError(
                    f"Agent state file not found at {path} after {timeout}s. Is the agent running and is AGENT_RANK correct?"
                )
            time.sleep(0.05)
        last_err = None
        while time.time() <= deadline:
            try:
                if self.state is None:
                    self.state = StateStore(path, readonly=True)
                age = self.state.heartbeat_age()
                if age is not None and age < HEARTBEAT_FRESH_S:
                    logger.info("TensorBusClient[%s]: agent alive (heartbeat %.2fs old)", self.agent_rank, age)
                    return
            except Exception as e:  # file still being created
                last_err = e
            time.sleep(0.05)
        if self.state is not None:
            self.state.close()
            self.state = None
        raise ConnectionError(
            f"Agent at {path} is not responding after {timeout}s: heartbeat too old or missing ({last_err}). "
            "The agent may have crashed."
        )

    # ---- API -----------------------------------------------------------------------------------
    def init_pair(self, pair_name: str, local_name: str, remote_name: str, expected_world_size: int, device_mesh=None,
                  placements=None, blocking: bool = True, timeout: float = 30.0):
        """Declare this rank's side of `pair_name`; returns once both sides are complete and planned.

        With `blocking=False` the completion handle is returned instead: several pairs can then be declared in
        any order on the two sides and awaited afterwards (the agent progresses all handshakes concurrently)."""
        mesh_payload = placements_payload = None
        if device_mesh is not None:
            m = getattr(device_mesh, "mesh", device_mesh)
            shape = tuple(int(s) for s in m.shape)
            # the shape is what the reference ships; the rank ids in mesh order let the agent honour a mesh whose
            # ranks are not ascending (an agent that only knows the shape payload assumes ascending order)
            ids = [int(x) for x in m.reshape(-1).tolist()] if hasattr(m, "reshape") else None
            mesh_payload = memoryview(pickle.dumps({"shape": shape, "ids": ids}))
        if placements is not None:
            placements_payload = memoryview(pickle.dumps(tuple(placements)))
        msg = InitPair(pair_name=pair_name, local_name=local_name, expected_world_size=expected_world_size,
                       remote_name=remote_name, mesh_shape_payload=mesh_payload, placements_payload=placements_payload)
        done = self._execute_command_with_semaphore(msg, "register", pair_name, blocking=blocking, timeout=timeout)
        if not blocking:
            return done
        if self.state.matched(pair_name) != "matched":
            raise RuntimeError(f"Pair '{pair_name}' is not matched")
        return None

    def register_tensors(self, batch_id: str, tensors: list[tuple[torch.Tensor, str]], bucket_size: int | None = None,
                         timeout: float = 30.0, blocking: bool = True) -> BatchHandler:
        """Register `(tensor, pair_name)` entries as one batch; order within a pair pairs them with the remote side.

        Blocks until every rank of both sides has registered (the reference always blocks).  A process that drives
        several clients passes `blocking=False` to each and then calls `handler.wait(timeout)` on the handlers."""
        if not tensors:
            raise ValueError("tensors list cannot be empty")
        if any(t.is_cuda for t, _ in tensors) and self._peer is None:
            from ..parallel.peer import PeerMemory

            self._peer = PeerMemory(next(t.device for t, _ in tensors if t.is_cuda))
        payload = [(pair, memoryview(encode_tensor(t, self._peer, self._arena))) for t, pair in tensors]
        # the registered tensors must outlive the registration: kept until the batch handler is closed
        self._keepalive.setdefault(batch_id, []).extend(t for t, _ in tensors)
        msg = RegisterTensors(batch_id=batch_id, tensors=payload, bucket_size=bucket_size)
        done = self._execute_command_with_semaphore(msg, "register_tensors", f"batch_{batch_id}", blocking=blocking,
                                                    timeout=timeout)
        # an older handle of the same batch id no longer owns the registration (the agent replaced it): its close or
        # garbage collection must not clean up the new one
        old = self._handlers.get(batch_id)
        old = old() if old is not None else None
        if old is not None:
            old._closed = True
        handler = BatchHandler(self, batch_id, list(dict.fromkeys(pair for _, pair in tensors)))
        self._handlers[batch_id] = weakref.ref(handler)
        handler._pending = None if blocking else done
        return handler

    def empty_replicated(self, shape, dtype: torch.dtype, device=None) -> torch.Tensor:
        """An uninitialised CUDA tensor in this client's replicated arena: register it as a `Replicate` target and
        producers write every replica with one NVLS multicast store instead of one store per replica.  (Tensors
        allocated any other way still work: their fan-out is one peer store per replica.)"""
        if self._arena is None:
            dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
            self._arena = ReplicatedArena(self.replicated_arena_bytes, dev)
        return self._arena.empty(shape, dtype)

    def transfer(self, batch_id: str, transfer_type: Literal["send", "recv"], blocking: bool = False, timeout: float = 30.0):
        msg = Transfer(batch_id=batch_id, transfer_type=transfer_type)
        return self._execute_command_with_semaphore(msg, "transfer", f"batch_{batch_id}_{transfer_type}", blocking=blocking,
                                                    timeout=timeout)

    def query_transfer_signal(self, batch_id: str, blocking: bool = True, timeout: float = 30.0) -> bool:
        """True once the sending side has started (or finished) a transfer the receiver has not consumed yet."""
        msg = QueryStatus(batch_id=batch_id, state_name="transfer_signal")
        self._execute_command_with_semaphore(msg, "query", f"batch_{batch_id}", blocking=blocking, timeout=timeout)
        return self.state.signal(batch_id, "transfer_signal")

    def _release_batch(self, batch_id: str) -> None:
        """Stop pinning the tensors of a closed batch (and their IPC exports' keep-alive references)."""
        tensors = self._keepalive.pop(batch_id, [])
        if self._peer is not None and tensors:
            self._peer.forget(tensors)

    def close(self) -> None:
        self._keepalive.clear()
        if self._arena is not None:
            # the agent keeps its own handle on the memory: closing here only ends this process's mapping
            self._arena.close()
            self._arena = None
        self.command_queue.close(destroy=False)
        if self.state is not None:
            self.state.close()
            self.state = None
