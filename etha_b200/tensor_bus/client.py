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


def encode_tensor(t: torch.Tensor, peer=None) -> bytes:
    """Serialise a handle to `t` for the agent (never the data)."""
    t = t.detach()
    if t.is_cuda:
        from ..parallel.peer import PeerMemory

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
    ):
        self.agent_rank = agent_rank
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
        payload = [(pair, memoryview(encode_tensor(t, self._peer))) for t, pair in tensors]
        # the registered tensors must outlive the registration: kept until the batch handler is closed
        self._keepalive.setdefault(batch_id, []).extend(t for t, _ in tensors)
        msg = RegisterTensors(batch_id=batch_id, tensors=payload, bucket_size=bucket_size)
        done = self._execute_command_with_semaphore(msg, "register_tensors", f"batch_{batch_id}", blocking=blocking,
                                                    timeout=timeout)
        handler = BatchHandler(self, batch_id, list(dict.fromkeys(pair for _, pair in tensors)))
        handler._pending = None if blocking else done
        return handler

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
        self.command_queue.close(destroy=False)
        if self.state is not None:
            self.state.close()
            self.state = None
