"""ctypes bindings of `libetha_b200_cuda.so` (kernels, table packer, IPC helpers)."""

from __future__ import annotations

import ctypes as C
import os
import threading

from . import build

MAX_SRC = 8
MAX_DST = 8
MAX_DIMS = 4

DT_RAW, DT_F32, DT_BF16, DT_F16 = 0, 1, 2, 3
RED_CODES = {"sum": 0, "avg": 1, "max": 2, "min": 3, "product": 4}
FLAG_MULTIMEM = 1
STATUS_OK, STATUS_TIMEOUT, STATUS_BAD_OP = 0, 1, 2


class OpSpec(C.Structure):
    _fields_ = [
        ("ndim", C.c_int32),
        ("shape", C.c_int64 * 8),
        ("src_stride", C.c_int64 * 8),
        ("dst_stride", C.c_int64 * 8),
        ("src_itemsize", C.c_int32),
        ("dst_itemsize", C.c_int32),
        ("src_dtype", C.c_int32),
        ("dst_dtype", C.c_int32),
        ("nsrc", C.c_int32),
        ("ndst", C.c_int32),
        ("src", C.c_uint64 * MAX_SRC),
        ("dst", C.c_uint64 * MAX_DST),
        ("src_lo", C.c_uint64 * MAX_SRC),
        ("src_hi", C.c_uint64 * MAX_SRC),
        ("dst_lo", C.c_uint64 * MAX_DST),
        ("dst_hi", C.c_uint64 * MAX_DST),
        ("red_size", C.c_int32 * 2),
        ("red_op", C.c_int32 * 2),
        ("flags", C.c_int32),
        ("tile_bytes", C.c_int32),
    ]


class DmaCopy(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("dst", "src", "width", "height", "dpitch", "spitch")]


_lock = threading.Lock()
_lib = None


def cuda_lib() -> C.CDLL:
    """Load (building first if the sources are newer) the CUDA library. Raises if it cannot be built."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        # ETHA_CUDA_LIB selects a pre-built library (e.g. one compiled with other tuning macros)
        path = os.environ.get("ETHA_CUDA_LIB") or build.build_cuda_lib()
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
        lib.etha_last_error.restype = C.c_char_p
        lib.etha_sizeof_op.restype = i32
        lib.etha_pack_op.argtypes = [C.POINTER(OpSpec), vp, C.c_char_p, i32]
        lib.etha_pack_op.restype = i32
        lib.etha_op_tiles.argtypes = [vp]
        lib.etha_op_tiles.restype = u32
        lib.etha_op_class.argtypes = [vp]
        lib.etha_op_class.restype = i32
        lib.etha_general_ctas_per_sm.restype = i32
        lib.etha_op_bulk_ok.argtypes = [vp]
        lib.etha_op_bulk_ok.restype = i32
        lib.etha_m2n_run_noalloc.argtypes = [C.POINTER(OpSpec), u32, i32, vp]
        lib.etha_m2n_run_noalloc.restype = i32
        lib.etha_m2n_noalloc_status.argtypes = [C.POINTER(u32), vp]
        lib.etha_m2n_noalloc_status.restype = i32
        lib.etha_op_stream_key.argtypes = [vp]
        lib.etha_op_stream_key.restype = i32
        lib.etha_stream_ctas_per_sm.restype = i32
        lib.etha_m2n_typed_launch.argtypes = [vp, vp, u32, i32, i32, vp, vp, u32, u32, i32, vp]
        lib.etha_m2n_typed_launch.restype = i32
        lib.etha_m2n_launch.argtypes = [vp, vp, u32, i32, i32, i32, vp, vp, u32, u32, i32, vp]
        lib.etha_m2n_launch.restype = i32
        lib.etha_set_flags.argtypes = [vp, u32, u32, vp]
        lib.etha_set_flags.restype = i32
        lib.etha_wait_flags.argtypes = [vp, vp, u32, u32, u64, vp, vp]
        lib.etha_wait_flags.restype = i32
        lib.etha_ipc_export.argtypes = [u64, C.c_char_p, C.POINTER(u64), C.POINTER(u64)]
        lib.etha_ipc_export.restype = i32
        lib.etha_ipc_open.argtypes = [C.c_char_p, C.POINTER(u64)]
        lib.etha_ipc_open.restype = i32
        lib.etha_ipc_close.argtypes = [u64]
        lib.etha_ipc_close.restype = i32
        lib.etha_copy_engine_d2d.argtypes = [u64, u64, u64, vp]
        lib.etha_copy_engine_d2d.restype = i32
        lib.etha_op_dma_copies.argtypes = [vp, C.POINTER(DmaCopy)]
        lib.etha_op_dma_copies.restype = i32
        lib.etha_dma_plan_create.argtypes = [C.POINTER(DmaCopy), u32, i32, i32, C.POINTER(vp)]
        lib.etha_dma_plan_create.restype = i32
        lib.etha_dma_plan_launch.argtypes = [vp, vp]
        lib.etha_dma_plan_launch.restype = i32
        lib.etha_dma_plan_join.argtypes = [vp, vp]
        lib.etha_dma_plan_join.restype = i32
        lib.etha_dma_plan_destroy.argtypes = [vp]
        lib.etha_dma_plan_destroy.restype = i32
        lib.etha_enable_peer_access.argtypes = [i32]
        lib.etha_enable_peer_access.restype = i32
        lib.etha_device_info.argtypes = [C.POINTER(i32)] * 4
        lib.etha_device_info.restype = i32
        if hasattr(lib, "etha_m2n_bulk_launch"):
            lib.etha_m2n_bulk_launch.argtypes = [vp, vp, u32, i32, vp, vp, u32, u32, i32, vp]
            lib.etha_m2n_bulk_launch.restype = i32
        _lib = lib
        return lib


def last_error() -> str:
    return (cuda_lib().etha_last_error() or b"").decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")
