"""Persistent bounded command queue between worker processes and their agent.

Same behaviour as the reference's LMDB queue (src/etha/tensor_bus/command_queue.py:23-396): msgpack
commands in FIFO order, fixed capacity (default 50 000), contents survive close/reopen, three named
POSIX semaphores (`/cq_{stem}` queued items, `/cq_space_{stem}` free slots, `/cq_ready_{stem}` leader
election between processes opening the same path).  Storage is a memory-mapped ring in a plain file
(`etha_b200/ops/csrc/shmq.cpp`) instead of an LMDB environment.
"""

from __future__ import annotations

import logging
import os
from pathlib import Path

import msgspec

from ..ops.hostlib import O_CREX, BusyError, ExistentialError, Semaphore, ShmQueue, unlink_semaphore
from .commands import Message

logger = logging.getLogger(__name__)


class QueueFullError(Exception):
    """The queue holds `capacity` commands (non-blocking enqueue, or the wait for space timed out)."""


class CommandQueue:
    _encoder = msgspec.msgpack.Encoder()
    _decoder = msgspec.msgpack.Decoder(Message)

    def __init__(self, lmdb_path: str = "/tmp/tensor_bus.lmdb", capacity: int = 50000, data_bytes: int = 1 << 28):
        self.lmdb_path = Path(lmdb_path)
        self.capacity = capacity
        stem = self.lmdb_path.stem
        self.sem_name = f"/cq_{stem}"
        self.space_sem_name = f"/cq_space_{stem}"
        self.ready_name = f"/cq_ready_{stem}"
        self._sem: Semaphore | None = None
        self._space_sem: Semaphore | None = None
        self._q: ShmQueue | None = None
        try:
            ready = Semaphore(self.ready_name, O_CREX, 0)  # whoever creates it initialises the rest
        except ExistentialError:
            ready = Semaphore(self.ready_name)
            ready.acquire()
            ready.release()  # pass the baton to the next follower
            ready.close()
            self._q = ShmQueue(str(self.lmdb_path), capacity, data_bytes)
            self.capacity = self._q.capacity
            self._sem = Semaphore(self.sem_name)
            self._space_sem = Semaphore(self.space_sem_name)
            return
        try:
            self._q = ShmQueue(str(self.lmdb_path), capacity, data_bytes)
            self.capacity = self._q.capacity
            queued = self._q.size()
            for name in (self.sem_name, self.space_sem_name):  # stale leftovers of a crashed owner
                try:
                    unlink_semaphore(name)
                except ExistentialError:
                    pass
            self._sem = Semaphore(self.sem_name, O_CREX, queued)
            self._space_sem = Semaphore(self.space_sem_name, O_CREX, self.capacity - queued)
            ready.release()
            ready.close()
        except Exception:
            for name in (self.sem_name, self.space_sem_name, self.ready_name):
                try:
                    unlink_semaphore(name)
                except Exception:
                    pass
            raise

    # ---- producer -------------------------------------------------------------------------
    def enqueue(self, msg: Message, *, block: bool = True, timeout: float | None = None) -> int:
        """Append `msg`; returns its position. Raises QueueFullError when no slot frees up in time."""
        try:
            self._space_sem.acquire(timeout if block else 0)
        except BusyError:
            raise QueueFullError(f"Queue is full (capacity={self.capacity})") from None
        data = self._encoder.encode(msg)
        pos = self._q.push(data)
        if pos < 0:
            self._space_sem.release()
            if pos == ShmQueue.TOO_BIG:
                raise ValueError(f"command of {len(data)} bytes does not fit the queue's data ring")
            raise QueueFullError(f"Queue is full (capacity={self.capacity}, data ring exhausted)")
        self._sem.release()
        return pos

    # ---- consumer -------------------------------------------------------------------------
    def _decode(self, data: bytes | None):
        if data is None:
            return None
        try:
            return self._decoder.decode(data)
        except msgspec.DecodeError:
            logger.warning("CommandQueue: dropped an undecodable command (%d bytes)", len(data))
            return None

    def dequeue(self, *, block: bool = False, timeout: float | None = None):
        """Oldest command or None. With `block`, waits up to `timeout` seconds for one to arrive."""
        if block:
            try:
                self._sem.acquire(timeout)
            except BusyError:
                return None
        else:
            # an item is taken only together with its semaphore count: a producer that has pushed but not yet posted
            # delivers on the next call, and the count never runs ahead of the ring
            try:
                self._sem.acquire(0)
            except BusyError:
                return None
        data = self._q.pop()
        if data is None:
            return None
        self._space_sem.release()
        return self._decode(data)

    def dequeue_batch(self, max_count: int = 32) -> list:
        out = []
        for _ in range(max_count):
            try:
                self._sem.acquire(0)
            except BusyError:
                break
            data = self._q.pop()
            if data is None:
                break
            self._space_sem.release()
            msg = self._decode(data)
            if msg is not None:
                out.append(msg)
        return out

    def peek(self):
        return self._decode(self._q.peek())

    def size(self) -> int:
        return self._q.size()

    def is_empty(self) -> bool:
        return self.size() == 0

    def clear(self, delete_commands: bool = True) -> None:  # noqa: ARG002
        self._q.clear()
        while True:
            try:
                self._sem.acquire(0)
            except BusyError:
                break
        while True:
            try:
                self._space_sem.acquire(0)
            except BusyError:
                break
        for _ in range(self.capacity):
            self._space_sem.release()

    def close(self, destroy: bool = True) -> None:
        """Close this process's handles; with `destroy` (default) also remove the file and the semaphores.
        Processes sharing the queue pass `destroy=False`; the last one destroys."""
        if destroy:
            for name in (self.sem_name, self.space_sem_name, self.ready_name):
                try:
                    unlink_semaphore(name)
                except Exception:
                    pass
        for attr in ("_sem", "_space_sem"):
            s = getattr(self, attr)
            if s is not None:
                s.close()
                setattr(self, attr, None)
        if self._q is not None:
            self._q.close()
            self._q = None
        if destroy:
            try:
                os.unlink(self.lmdb_path)
            except OSError:
                pass

    def __repr__(self) -> str:
        return f"CommandQueue(path={self.lmdb_path}, size={self.size() if self._q else 'closed'})"
