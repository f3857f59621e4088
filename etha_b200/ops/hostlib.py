"""ctypes bindings of `libetha_b200_host.so`: POSIX named semaphores, shared-memory queue and KV store.

`Semaphore` follows the call surface of `posix_ipc.Semaphore` that the reference relies on
(src/etha/tensor_bus/client.py:157-180, src/etha/tensor_bus/command_queue.py:38-80): `acquire(timeout)`,
`release()`, `close()`, `unlink()`, plus the `BusyError` / `ExistentialError` exceptions.
"""

from __future__ import annotations

import ctypes as C
import errno
import os
import threading

from . import build

O_CREAT = 1
O_EXCL = 2
O_CREX = O_CREAT | O_EXCL


class SemaphoreError(OSError):
    pass


class BusyError(SemaphoreError):
    """The semaphore could not be acquired within the timeout."""


class ExistentialError(SemaphoreError):
    """The named object does not exist (open/unlink) or already exists (exclusive create)."""


_lock = threading.Lock()
_lib = None


def host_lib() -> C.CDLL:
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        lib = C.CDLL(build.build_host_lib())
        vp, i32, u32, u64, i64 = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64, C.c_int64
        lib.etha_sem_open.argtypes = [C.c_char_p, i32, C.c_uint, C.POINTER(i32)]
        lib.etha_sem_open.restype = vp
        lib.etha_sem_post.argtypes = [vp]
        lib.etha_sem_wait.argtypes = [vp, C.c_double]
        lib.etha_sem_value.argtypes = [vp, C.POINTER(i32)]
        lib.etha_sem_close.argtypes = [vp]
        lib.etha_sem_unlink.argtypes = [C.c_char_p]
        lib.etha_q_open.argtypes = [C.c_char_p, u64, u64, C.POINTER(i32)]
        lib.etha_q_open.restype = vp
        lib.etha_q_push.argtypes = [vp, C.c_char_p, u64]
        lib.etha_q_push.restype = i64
        lib.etha_q_front.argtypes = [vp, C.c_char_p, u64, C.POINTER(u64), i32]
        lib.etha_q_size.argtypes = [vp]
        lib.etha_q_size.restype = i64
        lib.etha_q_capacity.argtypes = [vp]
        lib.etha_q_capacity.restype = u64
        lib.etha_q_clear.argtypes = [vp]
        lib.etha_q_close.argtypes = [vp]
        lib.etha_kv_open.argtypes = [C.c_char_p, i32, i32, u64, C.POINTER(i32)]
        lib.etha_kv_open.restype = vp
        lib.etha_kv_put.argtypes = [vp, C.c_char_p, u32, C.c_char_p, u32]
        lib.etha_kv_get.argtypes = [vp, C.c_char_p, u32, C.c_char_p, u32, C.POINTER(u32)]
        lib.etha_kv_del.argtypes = [vp, C.c_char_p, u32]
        lib.etha_kv_count.argtypes = [vp]
        lib.etha_kv_count.restype = i64
        lib.etha_kv_close.argtypes = [vp]
        _lib = lib
        return lib


class Semaphore:
    """A POSIX named semaphore (`/name`)."""

    def __init__(self, name: str, flags: int = 0, initial_value: int = 0):
        if not name.startswith("/"):
            raise ValueError("semaphore names start with '/'")
        self.name = name
        err = C.c_int(0)
        self._h = host_lib().etha_sem_open(name.encode(), flags, initial_value, C.byref(err))
        if not self._h:
            if err.value in (errno.ENOENT, errno.EEXIST):
                raise ExistentialError(err.value, os.strerror(err.value), name)
            raise SemaphoreError(err.value, os.strerror(err.value), name)

    def _handle(self):
        if not self._h:
            raise ExistentialError(errno.EBADF, "semaphore is closed", self.name)
        return self._h

    def acquire(self, timeout: float | None = None) -> None:
        """Decrement, waiting at most `timeout` seconds (None: forever, 0: do not wait). Raises BusyError."""
        rc = host_lib().etha_sem_wait(self._handle(), -1.0 if timeout is None else float(max(timeout, 0.0)))
        if rc == 1:
            raise BusyError(errno.EAGAIN, "semaphore busy", self.name)
        if rc < 0:
            raise SemaphoreError(-rc, os.strerror(-rc), self.name)

    def release(self) -> None:
        rc = host_lib().etha_sem_post(self._handle())
        if rc < 0:
            raise SemaphoreError(-rc, os.strerror(-rc), self.name)

    @property
    def value(self) -> int:
        out = C.c_int(0)
        host_lib().etha_sem_value(self._handle(), C.byref(out))
        return out.value

    def close(self) -> None:
        if self._h:
            host_lib().etha_sem_close(self._h)
            self._h = None

    def unlink(self) -> None:
        unlink_semaphore(self.name)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def unlink_semaphore(name: str) -> None:
    rc = host_lib().etha_sem_unlink(name.encode())
    if rc == -errno.ENOENT:
        raise ExistentialError(errno.ENOENT, "no such semaphore", name)
    if rc < 0:
        raise SemaphoreError(-rc, os.strerror(-rc), name)


class ShmQueue:
    """Bounded FIFO of byte strings in a memory-mapped file (no blocking: see CommandQueue for that)."""

    FULL_COUNT, FULL_BYTES, TOO_BIG = -1, -2, -3

    def __init__(self, path: str, capacity: int = 50000, data_bytes: int = 1 << 28):
        err = C.c_int(0)
        self._h = host_lib().etha_q_open(str(path).encode(), capacity, data_bytes, C.byref(err))
        if not self._h:
            raise OSError(err.value, os.strerror(err.value), str(path))
        self._buf = C.create_string_buffer(1 << 16)

    def push(self, data: bytes) -> int:
        return int(host_lib().etha_q_push(self._h, data, len(data)))

    def _front(self, consume: bool) -> bytes | None:
        n = C.c_uint64(0)
        rc = host_lib().etha_q_front(self._h, self._buf, len(self._buf), C.byref(n), int(consume))
        if rc == -3:
            self._buf = C.create_string_buffer(int(n.value) * 2)
            rc = host_lib().etha_q_front(self._h, self._buf, len(self._buf), C.byref(n), int(consume))
        if rc == 1:
            return None
        if rc != 0:
            raise OSError(f"queue read failed ({rc})")
        return self._buf.raw[: n.value]

    def pop(self) -> bytes | None:
        return self._front(True)

    def peek(self) -> bytes | None:
        return self._front(False)

    def size(self) -> int:
        return int(host_lib().etha_q_size(self._h))

    @property
    def capacity(self) -> int:
        return int(host_lib().etha_q_capacity(self._h))

    def clear(self) -> None:
        host_lib().etha_q_clear(self._h)

    def close(self) -> None:
        if self._h:
            host_lib().etha_q_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ShmKV:
    """Small key -> bytes store in a memory-mapped file; one writer process, lock-free readers."""

    MAX_VALUE = 2048

    def __init__(self, path: str, create: bool = True, readonly: bool = False, nslots: int = 4096):
        err = C.c_int(0)
        self._h = host_lib().etha_kv_open(str(path).encode(), int(create), int(readonly), nslots, C.byref(err))
        if not self._h:
            raise OSError(err.value, os.strerror(err.value), str(path))
        self._buf = C.create_string_buffer(self.MAX_VALUE)

    def put(self, key: bytes, value: bytes) -> None:
        rc = host_lib().etha_kv_put(self._h, key, len(key), value, len(value))
        if rc != 0:
            raise OSError(-rc, os.strerror(-rc))

    def get(self, key: bytes) -> bytes | None:
        n = C.c_uint32(0)
        rc = host_lib().etha_kv_get(self._h, key, len(key), self._buf, len(self._buf), C.byref(n))
        if rc == 1:
            return None
        if rc != 0:
            raise OSError(-rc, os.strerror(-rc))
        return self._buf.raw[: n.value]

    def delete(self, key: bytes) -> bool:
        return host_lib().etha_kv_del(self._h, key, len(key)) == 0

    def __len__(self) -> int:
        return int(host_lib().etha_kv_count(self._h))

    def close(self) -> None:
        if self._h:
            host_lib().etha_kv_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
