"""VMM arenas and NVLS multicast teams.

`VmmArena` is a block of device memory allocated with the CUDA virtual-memory API, so that (a) other
processes can map it from a file descriptor and (b) it can be bound to an NVSwitch multicast object.
`NvlsTeam` binds one equally sized arena per member GPU to one multicast object and maps it: a
`multimem.st` to `team.mc_va + off` then lands at `arena.va + off` on EVERY member — a Replicate target is
written with a single pass over the source and one store per 16 bytes, whatever the number of replicas.

Every member GPU must bind memory (an unbound member would fault on the first multicast store), so
producers that are not replicas bind a scratch arena of the same size.  Tear-down order matters on a
shared machine: unmap, unbind, release, and only then let the process exit — `close()` does that and is
also registered with `atexit`.

The reference has no counterpart (NCCL broadcast on a sub-group, src/etha/comm/transfer.py:33-41).
"""

from __future__ import annotations

import atexit
import ctypes as C
import os
import socket
import threading
from typing import Callable, Sequence

import torch

from ..ops import lib as L
from .peer import PeerMemory, RegionDesc, TensorDesc


def _lib():
    lib = L.cuda_lib()
    if not getattr(lib, "_vmm_ready", False):
        u64, i32, vp = C.c_uint64, C.c_int, C.c_void_p
        P = C.POINTER
        lib.etha_vmm_granularity.argtypes = [i32, P(u64)]
        lib.etha_vmm_alloc.argtypes = [u64, P(u64), P(u64), P(i32)]
        lib.etha_vmm_import.argtypes = [i32, u64, P(u64), P(u64)]
        lib.etha_vmm_unmap_release.argtypes = [u64, u64, u64]
        lib.etha_mc_create.argtypes = [i32, u64, P(u64), P(i32)]
        lib.etha_mc_import.argtypes = [i32, P(u64)]
        lib.etha_mc_add_device.argtypes = [u64]
        lib.etha_mc_bind.argtypes = [u64, u64, u64, u64, u64]
        lib.etha_mc_bind_addr.argtypes = [u64, u64, u64, u64]
        lib.etha_mc_map.argtypes = [u64, u64, P(u64)]
        lib.etha_mc_unbind.argtypes = [u64, u64, u64]
        lib.etha_close_fd.argtypes = [i32]
        lib._vmm_ready = True
    return lib


def granularity(n_devices: int = 0) -> int:
    out = C.c_uint64()
    L.check(_lib().etha_vmm_granularity(n_devices, C.byref(out)), "vmm_granularity")
    return int(out.value)


class _RawCudaBuffer:
    """Exposes a raw device range to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class VmmArena:
    def __init__(self, size: int, device: torch.device | int, n_team: int = 0):
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        with torch.cuda.device(self.device):
            g = granularity(n_team)
            self.size = (int(size) + g - 1) // g * g
            h, va, fd = C.c_uint64(), C.c_uint64(), C.c_int(-1)
            L.check(_lib().etha_vmm_alloc(self.size, C.byref(h), C.byref(va), C.byref(fd)), "vmm_alloc")
        self.handle, self.va, self.fd = int(h.value), int(va.value), int(fd.value)
        self._bytes = torch.as_tensor(_RawCudaBuffer(self.va, self.size, self), device=self.device)
        self._closed = False
        atexit.register(self.close)

    def tensor(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = dtype.itemsize
        for s in shape:
            n *= s
        if offset % 16 or offset + n > self.size:
            raise ValueError("arena view out of range or not 16-byte aligned")
        return self._bytes.narrow(0, offset, n).view(dtype).view(tuple(shape))

    def describe(self, t: torch.Tensor) -> TensorDesc:
        """Descriptor of a view of this arena; peers resolve it through `PeerMemory.adopt_mapping`."""
        region = RegionDesc(os.getpid(), self.device.index, self.va, self.size, b"vmm")
        return TensorDesc(region, t.data_ptr() - self.va, tuple(t.shape), tuple(t.stride()), str(t.dtype).replace("torch.", ""))

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        self._bytes = None
        if self.fd >= 0:
            _lib().etha_close_fd(self.fd)
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            _lib().etha_vmm_unmap_release(self.handle, self.va, self.size)


class ImportedArena:
    """Another process's `VmmArena`, mapped here from its file descriptor.  Has what `NvlsTeam` needs of an arena
    (handle, address, size, a descriptor to pass on), so an agent can bind its worker's memory to a multicast object."""

    def __init__(self, fd: int, size: int, device: torch.device | int):
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.size, self.fd = int(size), int(fd)
        with torch.cuda.device(self.device):
            h, va = C.c_uint64(), C.c_uint64()
            L.check(_lib().etha_vmm_import(self.fd, self.size, C.byref(h), C.byref(va)), "vmm_import")
        self.handle, self.va = int(h.value), int(va.value)
        self.imported = True  # bound to a multicast object by address, not by handle
        self._closed = False
        atexit.register(self.close)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        _lib().etha_close_fd(self.fd)
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            _lib().etha_vmm_unmap_release(self.handle, self.va, self.size)


def exchange_fds(rank: int, ranks: Sequence[int], fds: Sequence[int], tag: str, barrier: Callable[[], None],
                 directory: str = "/tmp") -> dict[int, list[int]]:
    """All-to-all hand-over of file descriptors between the processes `ranks` of one machine (SCM_RIGHTS over
    Unix sockets).  `barrier` must synchronise exactly those processes.  Returns peer rank -> received fds."""
    ranks = list(ranks)
    path = lambda r: os.path.join(directory, f"etha_fd_{tag}_{r}.sock")
    try:
        os.unlink(path(rank))
    except OSError:
        pass
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(path(rank))
    srv.listen(len(ranks))
    peers = [r for r in ranks if r != rank]

    def serve():
        for _ in peers:
            conn, _addr = srv.accept()
            with conn:
                socket.send_fds(conn, [rank.to_bytes(4, "little")], list(fds))
                conn.recv(1)  # the peer confirms it holds its duplicates before we go on

    th = threading.Thread(target=serve, daemon=True)
    th.start()
    barrier()
    got: dict[int, list[int]] = {}
    for r in peers:
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
            c.connect(path(r))
            msg, rfds, _flags, _addr = socket.recv_fds(c, 16, max(len(fds), 1) + 4)
            got[int.from_bytes(msg[:4], "little")] = list(rfds)
            c.send(b"k")
    th.join(timeout=60)
    barrier()
    srv.close()
    try:
        os.unlink(path(rank))
    except OSError:
        pass
    return got


class TeamUnavailable(RuntimeError):
    """The multicast team could not be formed (some member could not bind its memory); every member has left it
    again and the caller should use plain peer stores."""


class NvlsTeam:
    """One multicast object over the arenas of `ranks` (one process and one GPU each, same machine).

    Collective: every member constructs it with its own arena (all arenas have the same size).  After
    construction `mc_va` is this member's mapping of the multicast object and every peer's arena is mapped
    for plain peer access too (`peer_va[rank]`).
    """

    def __init__(self, rank: int, ranks: Sequence[int], arena: VmmArena, tag: str, all_gather: Callable[[object], list],
                 peer: PeerMemory | None = None):
        """`all_gather(obj)` returns every member's object in the order of `ranks` (e.g. `all_gather_object` on a
        gloo group of exactly these processes); it also serves as the barrier."""
        self.rank, self.ranks, self.arena = rank, list(ranks), arena
        barrier = lambda: all_gather(0)
        self.mc_handle = self.mc_va = 0
        self.peer_va: dict[int, int] = {rank: arena.va}
        self._imports: list[tuple[int, int]] = []
        self._closed = False
        lib = _lib()
        root = self.ranks[0]
        with torch.cuda.device(arena.device):
            mc_fd = -1
            if rank == root:
                h, fd = C.c_uint64(), C.c_int(-1)
                L.check(lib.etha_mc_create(len(self.ranks), arena.size, C.byref(h), C.byref(fd)), "mc_create")
                self.mc_handle, mc_fd = int(h.value), int(fd.value)
            # one exchange carries both the arena fd of every member and (from the root) the multicast fd
            mine = [arena.fd] + ([mc_fd] if rank == root else [])
            got = exchange_fds(rank, self.ranks, mine, tag, barrier)
            for r, fds in got.items():
                h, va = C.c_uint64(), C.c_uint64()
                L.check(lib.etha_vmm_import(fds[0], arena.size, C.byref(h), C.byref(va)), "vmm_import")
                self._imports.append((int(h.value), int(va.value)))
                self.peer_va[r] = int(va.value)
                if r == root and rank != root:
                    mh = C.c_uint64()
                    L.check(lib.etha_mc_import(fds[1], C.byref(mh)), "mc_import")
                    self.mc_handle = int(mh.value)
                for fd in fds:
                    lib.etha_close_fd(fd)
            if mc_fd >= 0:
                lib.etha_close_fd(mc_fd)
            L.check(lib.etha_mc_add_device(self.mc_handle), "mc_add_device")
            barrier()  # every device is part of the team before anybody binds
            # an arena this process created is bound by its allocation handle; one it imported from another process
            # (an agent binding its worker's arena) is bound by the address it is mapped at.  Whether binding worked is
            # agreed on by all members before anybody maps or stores: one failure dissolves the team everywhere.
            problem = None
            rc = lib.etha_mc_bind(self.mc_handle, 0, arena.handle, 0, arena.size) if not getattr(arena, "imported", False) else -1
            if rc != 0:
                first = L.last_error() if not getattr(arena, "imported", False) else "imported allocation"
                rc = lib.etha_mc_bind_addr(self.mc_handle, 0, arena.va, arena.size)
                if rc != 0:
                    problem = f"rank {rank}: binding to the multicast object failed (by handle: {first}; by address: {L.last_error()})"
            self._bound = problem is None
            problems = [p for p in all_gather(problem) if p]
            if not problems:
                va = C.c_uint64()
                rc = lib.etha_mc_map(self.mc_handle, arena.size, C.byref(va))
                if rc == 0:
                    self.mc_va = int(va.value)
                problems = [p for p in all_gather(None if rc == 0 else f"rank {rank}: mapping the multicast object failed: {L.last_error()}") if p]
            if problems:
                self.close()
                raise TeamUnavailable("; ".join(problems))
        # descriptors of views of a peer's arena (`VmmArena.describe`) resolve to the mappings made here
        owners = all_gather((os.getpid(), arena.device.index, arena.va))
        self.owner_va = {r: o[2] for r, o in zip(self.ranks, owners)}
        self.replicas: list[int] | None = None  # members that really consume (None: all); the others bind scratch
        if peer is not None:
            peer.register_arena(arena)
            for r, (pid, dev_index, va) in zip(self.ranks, owners):
                if r != rank:
                    peer.adopt_mapping((pid, dev_index, va), self.peer_va[r])
        atexit.register(self.close)

    def close(self) -> None:
        """Unmap and unbind before the process goes away (a bound member that dies disturbs its peers)."""
        if self._closed:
            return
        self._closed = True
        lib = _lib()
        with torch.cuda.device(self.arena.device):
            torch.cuda.synchronize()
            if self.mc_va:
                lib.etha_vmm_unmap_release(0, self.mc_va, self.arena.size)
            if self.mc_handle:
                if getattr(self, "_bound", True):
                    lib.etha_mc_unbind(self.mc_handle, 0, self.arena.size)
                lib.etha_vmm_unmap_release(self.mc_handle, 0, 0)
            for h, va in self._imports:
                lib.etha_vmm_unmap_release(h, va, self.arena.size)
