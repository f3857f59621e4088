"""Native ops: sm_100a copy/convert/reduce kernels, flag kernels, table packer, IPC helpers."""

from __future__ import annotations

import torch

from . import lib as _L
from .lib import STATUS_BAD_OP, STATUS_OK, STATUS_TIMEOUT, cuda_lib
from .table import CopyTable, SliceRef, dtype_code

FLAG_LAUNCH_COUNT = [0]  # set_flags / wait_flags kernels launched in this process

__all__ = [
    "CopyTable",
    "SliceRef",
    "dtype_code",
    "cuda_lib",
    "local_copy",
    "set_flags",
    "wait_flags",
    "device_info",
    "STATUS_OK",
    "STATUS_TIMEOUT",
    "STATUS_BAD_OP",
]


def local_copy(src: torch.Tensor, dst: torch.Tensor, stream: torch.cuda.Stream | None = None) -> None:
    """`dst[...] = src` (any strides, fp32/bf16/fp16 conversion) through the copy kernels."""
    t = CopyTable(dst.device)
    t.add_copy(src, dst)
    t.finalize()
    t.launch(stream)
    # the table's device arrays must outlive the kernel: tie them to the stream
    for buf in t.device_buffers():
        buf.record_stream(stream or torch.cuda.current_stream(dst.device))


def set_flags(addresses: torch.Tensor, epoch: int, stream: torch.cuda.Stream | None = None) -> None:
    """Store `epoch` (release, system scope) to every uint32 flag whose address is in `addresses` (int64, device)."""
    s = (stream or torch.cuda.current_stream(addresses.device)).cuda_stream
    _L.check(cuda_lib().etha_set_flags(addresses.data_ptr(), addresses.numel(), epoch & 0xFFFFFFFF, s), "set_flags")
    FLAG_LAUNCH_COUNT[0] += 1


def wait_flags(
    flags: torch.Tensor,
    which: torch.Tensor,
    epoch: int,
    status: torch.Tensor,
    timeout_s: float = 2.0,
    stream: torch.cuda.Stream | None = None,
) -> None:
    """Enqueue a bounded wait until `flags[which[i]] >= epoch` for all i.

    `status` (int32[2], device or pinned-mapped) receives `[STATUS_OK | STATUS_TIMEOUT, index of the
    first missing flag]`.  The wait gives up after `timeout_s`; the context stays usable.
    """
    s = (stream or torch.cuda.current_stream(flags.device)).cuda_stream
    rc = cuda_lib().etha_wait_flags(
        flags.data_ptr(), which.data_ptr(), which.numel(), epoch & 0xFFFFFFFF, int(timeout_s * 1e9), status.data_ptr(), s
    )
    _L.check(rc, "wait_flags")
    FLAG_LAUNCH_COUNT[0] += 1


def device_info() -> dict:
    import ctypes as C

    sm, maj, mnr, mc = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    _L.check(cuda_lib().etha_device_info(C.byref(sm), C.byref(maj), C.byref(mnr), C.byref(mc)), "device_info")
    return {"sm_count": sm.value, "cc": (maj.value, mnr.value), "multicast": bool(mc.value)}
