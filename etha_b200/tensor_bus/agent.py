"""Tensor bus agent: the daemon that owns one GPU's side of every transfer.

Same role, constructor and command set as the reference's agent (src/etha/tensor_bus/agent.py:73-798),
re-organised around three ideas:

* **no collective in any handler.**  Rendezvous, descriptor exchange, the pre-transfer barrier and
  completion all go through the KV store, planning is analytic, and no process sub-group is ever
  created — so handlers need no lock-step discipline across agents, and a side that never shows up
  produces a timeout error instead of a hung collective;
* **handlers are resumable jobs** (generators that yield while they wait), so the command loop keeps
  turning: several `InitPair` handshakes progress concurrently in any order, and the heartbeat (written by
  its own thread) never goes stale during a long command;
* **failures are reported**: the error text is stored under `error:{semaphore}` before the semaphore is
  posted, and the agent stays alive.

On GPUs the data path is the peer-to-peer executor (`etha_b200.comm.p2p`): workers hand over IPC
descriptors, agents exchange them and each producing agent launches one copy table per transfer.  On CPU
tensors (tests, gloo) the bucket executor is used.
"""

from __future__ import annotations

import logging
import os
import pickle
import threading
import time
import traceback
import uuid
from typing import Generator

import torch
import torch.distributed as dist

from ..kvstore import KVStore, create_store
from ..ops.hostlib import ExistentialError, Semaphore
from .batch_state import BatchState
from .command_queue import CommandQueue
from .commands import CleanupBatch, InitPair, QueryStatus, RegisterTensors, Transfer
from .agent_handlers import AgentHandlers
from .pair_state import PairState
from .state_store import StateStore

logger = logging.getLogger(__name__)

TIME_INTERVAL = 0.001  # command-loop tick
HOT_JOB_S = 0.05  # a job younger than this is polled without sleeping (a transfer is a few store round trips + the copy)
HEARTBEAT_PERIOD = 0.2
ERROR_TTL_S = 120.0  # a failed command's message is kept this long for its client to read, then deleted

_DTYPES = {str(d).replace("torch.", ""): d for d in [
    torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16, torch.int32,
    torch.int64, torch.bool,
]}


def decode_tensor(payload: bytes):
    """Inverse of `client.encode_tensor`: ("cuda", TensorDesc) stays a descriptor, ("cpu", ...) becomes a tensor
    over the worker's shared-memory file."""
    kind, meta = pickle.loads(payload)
    if kind == "cuda":
        return "cuda", meta
    import torch.multiprocessing as tmp

    if tmp.get_sharing_strategy() != "file_system":
        tmp.set_sharing_strategy("file_system")
    manager, handle, size, offset, shape, stride, dtype = meta
    storage = torch.UntypedStorage._new_shared_filename_cpu(manager, handle, size)
    t = torch.empty(0, dtype=_DTYPES[dtype]).set_(storage, offset, shape, stride)
    return "cpu", t


class _Job:
    def __init__(self, command, gen: Generator, concurrent: bool):
        self.command, self.gen, self.concurrent = command, gen, concurrent
        self.started = time.monotonic()


class TensorBusAgent(AgentHandlers):
    def __init__(
        self,
        rank: int,
        world_size: int,
        store_host: str,
        store_port: int,
        lmdb_command_queue_path: str,
        lmdb_state_path: str,
        store_timeout: float = 3600.0,
        store_backend: str = "tcp",
        store_namespace: str | None = None,
        store: KVStore | None = None,
        device: str | torch.device | None = None,
    ):
        self.rank, self.world_size = rank, world_size
        self.store_timeout = store_timeout
        use_cuda = torch.cuda.is_available() if device is None else torch.device(device).type == "cuda"
        if use_cuda:
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            self.device = torch.device("cuda", local)
        else:
            self.device = torch.device("cpu")
        if not dist.is_initialized():
            backend = "cuda:nccl,cpu:gloo" if use_cuda else "gloo"
            dist.init_process_group(backend=backend, rank=rank, world_size=world_size)
        if store_namespace is None:
            box = [uuid.uuid4().hex[:8] if rank == 0 else None]
            dist.broadcast_object_list(box, src=0, device=torch.device("cpu"))
            store_namespace = box[0]
        self.namespace = store_namespace
        self.store: KVStore = store or create_store(
            host=store_host, port=store_port, timeout=store_timeout, backend=store_backend, namespace=store_namespace
        )
        self.command_queue = CommandQueue(lmdb_command_queue_path)
        self.lmdb_state_path = str(lmdb_state_path)
        self.state = StateStore(self.lmdb_state_path)
        self.state.beat()
        self.pairs: dict[str, PairState] = {}
        self.batches: dict[str, BatchState] = {}
        self._jobs: list[_Job] = []
        self._errors: list[tuple[float, str]] = []  # (time stored, semaphore name) of error keys in the state store
        self.error_ttl_s = ERROR_TTL_S
        self._stop = threading.Event()
        self._peer = None
        self._worker_arenas: dict[tuple, object] = {}  # (worker pid, address) -> imported replicated arena
        self._hb = threading.Thread(target=self._heartbeat_loop, daemon=True)
        self._hb.start()
        logger.info("Agent %s/%s up on %s, namespace %s", rank, world_size, self.device, store_namespace)

    # ---- loop -------------------------------------------------------------------------------------
    def _heartbeat_loop(self) -> None:
        while not self._stop.is_set():
            try:
                self.state.beat()
            except Exception:
                pass
            self._stop.wait(HEARTBEAT_PERIOD)

    def run(self, max_idle_s: float | None = None) -> None:
        """Serve commands until `stop()`; `max_idle_s` ends the loop after that long without any command (tests)."""
        last = time.monotonic()
        while not self._stop.is_set():
            # idle: block on the queue semaphore for a tick; with jobs in flight poll fast, a transfer's barrier and
            # completion are a handful of store round trips and should not pay a millisecond sleep each
            if not self._jobs:
                tick = TIME_INTERVAL
            else:  # a sleep costs at least 60-100 us of timer slack: too much between the polls of a 5 ms transfer
                now = time.monotonic()
                tick = 0.0 if any(now - j.started < HOT_JOB_S for j in self._jobs) else 0.00005
            busy = self.step(block_s=tick)
            if busy:
                last = time.monotonic()
            elif max_idle_s is not None and time.monotonic() - last > max_idle_s:
                break

    def stop(self) -> None:
        self._stop.set()

    def _can_start(self, concurrent: bool) -> bool:
        if not self._jobs:
            return True
        return concurrent and all(j.concurrent for j in self._jobs)

    def step(self, block_s: float = 0.0) -> bool:
        """One tick: maybe start the next command, advance every running job. Returns True if anything is in flight."""
        # another command can only start next to running ones if all of them are handshakes: do not look otherwise
        nxt = self.command_queue.peek() if (self._jobs and all(j.concurrent for j in self._jobs)) else None
        if not self._jobs or (nxt is not None and self._can_start(isinstance(nxt, InitPair))):
            msg = self.command_queue.dequeue(block=not self._jobs, timeout=block_s)
            if msg is not None:
                self._start(msg)
        elif block_s:
            time.sleep(block_s)
        for job in list(self._jobs):
            self._advance(job)
        # clients open the state store read-only, so the agent removes error messages once they are old enough to
        # have been read (the store has a fixed number of slots)
        while self._errors and time.monotonic() - self._errors[0][0] > self.error_ttl_s:
            self.state.delete(f"error:{self._errors.pop(0)[1]}")
        return bool(self._jobs)

    def _start(self, command) -> None:
        handlers = {
            InitPair: self._init_pair_job,
            RegisterTensors: self._register_tensors_job,
            Transfer: self._transfer_job,
            QueryStatus: self._query_status_job,
            CleanupBatch: self._cleanup_batch_job,
        }
        h = handlers.get(type(command))
        if h is None:
            logger.warning("Agent %s: unknown command %r", self.rank, type(command))
            return
        self._jobs.append(_Job(command, h(command), isinstance(command, InitPair)))

    def _advance(self, job: _Job) -> None:
        try:
            next(job.gen)
            if time.monotonic() - job.started > self.store_timeout:
                raise TimeoutError(f"{type(job.command).__name__} did not complete within {self.store_timeout}s")
            return
        except StopIteration:
            pass
        except Exception as e:  # report, stay alive
            logger.error("Agent %s: %s failed: %s\n%s", self.rank, type(job.command).__name__, e, traceback.format_exc())
            if job.command.semaphore_name:
                self.state.set_error(job.command.semaphore_name, f"{type(e).__name__}: {e}")
                self._errors.append((time.monotonic(), job.command.semaphore_name))
        self._jobs.remove(job)
        if job.command.semaphore_name:
            self._release_semaphore(job.command.semaphore_name)

    def _release_semaphore(self, name: str) -> None:
        try:
            sem = Semaphore(name)
        except ExistentialError:
            logger.warning("Agent %s: semaphore %s not found", self.rank, name)
            return
        try:
            sem.release()
        finally:
            sem.close()
            try:
                sem.unlink()
            except ExistentialError:
                pass

    @staticmethod
    def _extract_rank(key: str) -> int:
        i = key.find("/rank:")
        if i < 0:
            raise ValueError(f"No rank found in key: {key}")
        return int(key[i + 6 :].split("/")[0])

    def close(self, destroy: bool = True) -> None:
        self._stop.set()
        self._hb.join(timeout=1.0)
        for batch_id in list(self.batches):  # leave multicast teams and release mappings in order
            try:
                self._drop_batch(self.batches.pop(batch_id))
            except Exception:
                logger.exception("Agent %s: releasing batch %s failed", self.rank, batch_id)
        for arena in self._worker_arenas.values():
            arena.close()
        self._worker_arenas.clear()
        self.command_queue.close(destroy=destroy)
        self.state.close()
        if destroy:
            try:
                os.unlink(self.lmdb_state_path)
            except OSError:
                pass
        if self._peer is not None:
            self._peer.close()
        self.store.close()
        if dist.is_initialized():
            dist.destroy_process_group()
