"""Host-side table packer: collapsing, unit selection, bounds validation (no GPU needed)."""

import ctypes as C

import pytest
import torch

from etha_b200.ops import lib as L
from etha_b200.ops.table import CopyTable, SliceRef


class OpView(C.Structure):
    _fields_ = [
        ("src", C.c_uint64 * 8), ("dst", C.c_uint64 * 8), ("src_stride", C.c_int64 * 4), ("dst_stride", C.c_int64 * 4),
        ("extent", C.c_uint32 * 4), ("div_mul", C.c_uint32 * 5), ("div_shr", C.c_uint32 * 5),
        ("inner_units", C.c_uint32), ("total_units", C.c_uint32), ("tile_units", C.c_uint32),
        ("unit_bytes_src", C.c_uint32), ("unit_bytes_dst", C.c_uint32),
        ("ndim", C.c_uint8), ("nsrc", C.c_uint8), ("ndst", C.c_uint8), ("mode", C.c_uint8),
        ("src_dtype", C.c_uint8), ("dst_dtype", C.c_uint8), ("unit_elems", C.c_uint8), ("flags", C.c_uint8),
        ("red_size", C.c_uint8 * 2), ("red_op", C.c_uint8 * 2), ("pad", C.c_uint32 * 5),
    ]


def pack(shape, sstr, dstr, sdt=torch.bfloat16, ddt=torch.bfloat16, sptr=1 << 20, dptr=1 << 24, nsrc=1, **kw):
    t = CopyTable(torch.device("cpu"))
    srcs = [SliceRef(sptr + i * (1 << 30), tuple(sstr), sdt) for i in range(nsrc)]
    t.add(shape, srcs, [SliceRef(dptr, tuple(dstr), ddt)], **kw)
    assert len(t._packed) == 1
    cls, tiles, raw, *_ = t._packed[0]
    return cls, tiles, OpView.from_buffer_copy(raw)


def test_struct_size_matches_native():
    assert L.cuda_lib().etha_sizeof_op() == C.sizeof(OpView)


def test_contiguous_collapses_to_one_run():
    cls, tiles, op = pack((1024, 4096), (4096, 1), (4096, 1))
    assert (op.ndim, op.unit_bytes_src, op.inner_units, op.total_units) == (0, 16, 1024 * 4096 // 8, 1024 * 4096 // 8)
    assert cls == 0 and tiles == (op.total_units + op.tile_units - 1) // op.tile_units


def test_column_slice_is_rows_of_a_matrix():
    # Shard(0) source [1024, 4096] cut into 4 column blocks -> contiguous [1024, 1024]
    cls, _, op = pack((1024, 1024), (4096, 1), (1024, 1))
    assert (cls, op.ndim, op.extent[0], op.inner_units) == (0, 1, 1024, 128)
    assert (op.src_stride[0], op.dst_stride[0]) == (8192, 2048)


def test_three_strided_dims_go_to_general_class():
    cls, _, op = pack((4, 8, 32), (1024, 64, 1), (2048, 128, 1))
    assert cls == 1 and op.ndim == 2


def test_unit_shrinks_with_alignment():
    _, _, op = pack((7, 33), (64, 1), (33, 1))  # 66-byte rows of bf16: 2-byte units
    assert op.unit_bytes_src == 2
    _, _, op = pack((8, 64), (64, 1), (64, 1), sptr=(1 << 20) + 8)  # base only 8-byte aligned
    assert op.unit_bytes_src == 8
    _, _, op = pack((16,), (2,), (1,))  # inner stride != 1: element-wise
    assert op.unit_bytes_src == 2 and op.ndim == 1 and op.inner_units == 1


def test_conversion_and_reduce_modes():
    cls, _, op = pack((64, 64), (64, 1), (64, 1), sdt=torch.float32, ddt=torch.bfloat16)
    assert (cls, op.mode, op.unit_elems, op.unit_bytes_src, op.unit_bytes_dst) == (1, 1, 8, 32, 16)
    cls, _, op = pack((64, 64), (64, 1), (64, 1), sdt=torch.float32, ddt=torch.float32, nsrc=4,
                      reduce_sizes=(2, 2), reduce_ops=("sum", "max"))
    assert (cls, op.mode, op.nsrc, tuple(op.red_size), tuple(op.red_op)) == (1, 2, 4, (2, 2), (0, 2))


def test_rejects_out_of_bounds_and_unsupported():
    t = CopyTable(torch.device("cpu"))
    src = SliceRef(4096, (64, 1), torch.float32, lo=4096, hi=4096 + 64 * 64 * 4)
    bad_dst = SliceRef(1 << 20, (64, 1), torch.float32, lo=1 << 20, hi=(1 << 20) + 64 * 64 * 4 - 4)
    with pytest.raises(ValueError, match="outside its allocation"):
        t.add((64, 64), [src], [bad_dst])
    with pytest.raises(ValueError, match="conversion|no conversion"):
        t.add((64,), [SliceRef(4096, (1,), torch.int32)], [SliceRef(8192, (1,), torch.float32)])
    with pytest.raises(ValueError):
        t.add((2, 2, 2, 2, 2, 2), [SliceRef(4096, (1000, 300, 90, 27, 8, 2), torch.float32)],
              [SliceRef(1 << 20, (32, 16, 8, 4, 2, 1), torch.float32)])


def test_fast_division_magic():
    # the packer's magic numbers must reproduce floor division for every dividend below 2^31 we try
    import random

    random.seed(0)
    for d in [1, 2, 3, 5, 7, 128, 448, 1000, 4095, 4096, 4097, 65535, 1 << 20, (1 << 30) - 1]:
        _, _, op = pack((2, d), (2 * d, 1), (d + 8, 1), sdt=torch.uint8, ddt=torch.uint8, sptr=1 << 20, dptr=(1 << 24) + 1)
        mul, shr = op.div_mul[4], op.div_shr[4]
        assert op.inner_units == d
        for n in [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d] + [random.randrange(1 << 31) for _ in range(200)]:
            if n >= 1 << 31:
                continue
            q = n if mul == 0 else ((n * mul) >> 32) >> shr
            assert q == n // d, (d, n)
