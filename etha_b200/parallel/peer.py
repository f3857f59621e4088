"""Peer pointers: describe local device tensors so that other processes can address them, and map theirs.

An agent (or a rank of a torchrun job) exports the allocation behind each registered tensor once as a
64-byte CUDA IPC handle, ships `(handle, offset, shape, strides, dtype)` to its peers over the control
plane and maps the handles it receives; the copy kernels then use the mapped addresses directly over
NVLink.  Within one process (a rank that holds both roles, or several logical ranks sharing a GPU) the
owner's own addresses are used and nothing is mapped.

The reference shares tensors only worker -> agent, by pickling whole tensors through torch's CUDA-IPC
reducer and rebuilding them on `LOCAL_RANK` (src/etha/tensor_bus/client.py:314, src/etha/tensor_bus/
agent.py:608, src/etha/tensor_bus/utils.py:14-69); agents never see each other's memory there.
"""

from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch

from ..ops import lib as L
from ..ops.table import SliceRef

_DTYPE_NAMES = {str(d).replace("torch.", ""): d for d in [
    torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16,
    torch.int32, torch.int64, torch.bool, torch.float8_e4m3fn, torch.float8_e5m2,
]}


@dataclass(frozen=True)
class RegionDesc:
    """One exported device allocation."""

    pid: int
    device_index: int
    base: int  # address in the owner's address space
    size: int
    handle: bytes  # cudaIpcMemHandle_t

    @property
    def key(self) -> tuple:
        return (self.pid, self.device_index, self.base)


@dataclass(frozen=True)
class TensorDesc:
    """A (possibly strided) tensor inside an exported allocation."""

    region: RegionDesc
    offset: int  # bytes from region.base to element [0, ..., 0]
    shape: tuple[int, ...]
    strides: tuple[int, ...]  # elements
    dtype: str
    # set for a view of a worker's replicated (VMM) arena: {"socket", "size", "pid", "device_index", "va"} tells the
    # agent where to fetch the arena's file descriptor
    arena: dict | None = None

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPE_NAMES[self.dtype]


class PeerExportError(RuntimeError):
    """A tensor's memory cannot be shared with other processes."""


class PeerMemory:
    """Per-process registry of exported and mapped allocations.

    Exported regions are remembered by base address but always carry the handle CUDA returned for the current
    allocation; mappings of other processes' regions are keyed by `(owner pid, handle bytes)`, so an allocation
    that was freed and re-created at the same address is opened afresh instead of reusing a dead mapping.
    Mappings are reference counted by their users (`retain` / `release`): the last release closes the mapping."""

    def __init__(self, device: torch.device | int | None = None):
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.pid = os.getpid()
        self._lib = L.cuda_lib()
        self._exported: dict[int, RegionDesc] = {}  # base -> desc
        self._mapped: dict[tuple, int] = {}  # map key -> local base
        self._by_owner_base: dict[tuple, tuple] = {}  # (pid, device, base) -> map key of the current mapping
        self._refs: dict[tuple, int] = {}  # map key -> users
        self._keepalive: dict[int, torch.Tensor] = {}
        self._arenas: list = []  # VMM arenas of this process: their views are described without an IPC handle

    # ---- owner side -----------------------------------------------------------------------
    def register_arena(self, arena) -> None:
        self._arenas.append(arena)

    def describe(self, t: torch.Tensor, keepalive: bool = True) -> TensorDesc:
        if not t.is_cuda:
            raise ValueError("only CUDA tensors can be exported")
        for arena in self._arenas:
            if arena.va <= t.data_ptr() < arena.va + arena.size:
                return arena.describe(t)
        with torch.cuda.device(t.device):
            handle = C.create_string_buffer(64)
            base, size = C.c_uint64(), C.c_uint64()
            storage_ptr = t.untyped_storage().data_ptr()
            rc = self._lib.etha_ipc_export(storage_ptr, handle, C.byref(base), C.byref(size))
        if rc != 0:
            raise PeerExportError(
                f"cannot export the memory of a {tuple(t.shape)} {t.dtype} tensor on {t.device} for other processes "
                f"({L.last_error()}). CUDA IPC handles exist only for plain cudaMalloc allocations: memory from "
                "torch's expandable segments (PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True), from a VMM pool "
                "(cuMemCreate / cuMemMap) or from cudaMallocAsync cannot be exported this way. Allocate the registered "
                "tensors with the default caching allocator, or place them in an etha_b200.parallel.arena.VmmArena "
                "(shared by file descriptor)."
            )
        region = self._exported.get(base.value)
        if region is None or region.size != size.value or region.handle != handle.raw:
            # first export of this address, or the allocation behind it was replaced: the fresh handle wins
            region = RegionDesc(self.pid, t.device.index, base.value, size.value, handle.raw)
            self._exported[base.value] = region
        if keepalive:
            self._keepalive[id(t)] = t
        return TensorDesc(region, t.data_ptr() - base.value, tuple(t.shape), tuple(t.stride()),
                          str(t.dtype).replace("torch.", ""))

    def describe_local_only(self, t: torch.Tensor) -> TensorDesc:
        """Descriptor usable only inside this process (no IPC handle is created)."""
        st = t.untyped_storage()
        region = RegionDesc(self.pid, t.device.index if t.is_cuda else -1, st.data_ptr(), st.nbytes(), b"")
        self._keepalive[id(t)] = t
        return TensorDesc(region, t.data_ptr() - st.data_ptr(), tuple(t.shape), tuple(t.stride()),
                          str(t.dtype).replace("torch.", ""))

    def forget(self, tensors) -> None:
        """Stop keeping `tensors` alive (their batch was cleaned up)."""
        for t in tensors:
            self._keepalive.pop(id(t), None)

    # ---- peer side ------------------------------------------------------------------------
    @staticmethod
    def _map_key(region: RegionDesc) -> tuple:
        if region.handle and len(region.handle) == 64:
            return (region.pid, region.handle)
        return region.key  # VMM arena or test double: identified by owner and address

    def map_region(self, region: RegionDesc) -> int:
        """Address of `region.base` in this process (maps the allocation on first use)."""
        if region.pid == self.pid:
            return region.base
        key = self._map_key(region)
        local = self._mapped.get(key)
        if local is None:
            if not region.handle or region.handle == b"vmm":
                raise ValueError("region of another process has no IPC handle and no adopted mapping")
            stale = self._by_owner_base.get(region.key)
            if stale is not None and stale != key:
                self._close(stale)  # the owner re-allocated this address: the old mapping points at freed memory
            with torch.cuda.device(self.device):
                out = C.c_uint64()
                L.check(self._lib.etha_ipc_open(region.handle, C.byref(out)), "ipc_open")
            local = out.value
            self._mapped[key] = local
            self._by_owner_base[region.key] = key
        return local

    def retain(self, regions) -> list[tuple]:
        """Count one more user of the mappings of `regions` (mapping them if needed); returns the keys to hand
        back to `release`."""
        keys = []
        for region in regions:
            if region.pid == self.pid or not region.handle or len(region.handle) != 64:
                continue
            self.map_region(region)
            key = self._map_key(region)
            self._refs[key] = self._refs.get(key, 0) + 1
            keys.append(key)
        return keys

    def release(self, keys) -> None:
        """Drop one user per key; a mapping nobody uses any more is closed."""
        for key in keys:
            n = self._refs.get(key, 0) - 1
            if n > 0:
                self._refs[key] = n
                continue
            self._refs.pop(key, None)
            self._close(key)

    def _close(self, key: tuple) -> None:
        local = self._mapped.pop(key, None)
        if local is not None:
            self._lib.etha_ipc_close(local)
        for owner_base, k in list(self._by_owner_base.items()):
            if k == key:
                del self._by_owner_base[owner_base]

    @property
    def n_mapped(self) -> int:
        return len(self._mapped)

    def adopt_mapping(self, region_key: tuple, local_base: int) -> None:
        """Register a mapping made elsewhere (a VMM arena imported from a file descriptor): descriptors whose
        region has this `(pid, device_index, base)` key resolve to `local_base`."""
        self._mapped[tuple(region_key)] = int(local_base)

    def slice_ref(self, desc: TensorDesc, index: tuple[slice, ...] = ()) -> SliceRef:
        """`SliceRef` of `tensor[index]` (unit-step slices) for the tensor described by `desc`."""
        base = self.map_region(desc.region)
        dt = desc.torch_dtype
        off = desc.offset
        for sl, stride in zip(index, desc.strides):
            off += (sl.start or 0) * stride * dt.itemsize
        return SliceRef(base + off, desc.strides, dt, base, base + desc.region.size)

    def as_tensor(self, desc: TensorDesc) -> torch.Tensor:
        """A torch view of a described tensor in this process's address space (maps the region if needed).
        Used when a library call needs a tensor object, e.g. the NCCL fallback across nodes."""
        base = self.map_region(desc.region)
        dt = desc.torch_dtype
        span = 1 + sum((n - 1) * abs(st) for n, st in zip(desc.shape, desc.strides)) if all(desc.shape) else 0

        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (max(span, 1) * dt.itemsize,), "typestr": "|u1",
                                        "data": (base + desc.offset, False), "version": 2}
        flat = torch.as_tensor(raw, device=self.device).view(dt)
        return flat.as_strided(desc.shape, desc.strides)

    def close(self) -> None:
        for local in self._mapped.values():
            self._lib.etha_ipc_close(local)  # mappings adopted from elsewhere are unknown to it and left alone
        self._mapped.clear()
        self._by_owner_base.clear()
        self._refs.clear()
        self._keepalive.clear()
