"""CPU restatement of the copy kernels' index arithmetic over the packed table.

The packer's output (collapsed dims, units, byte strides, fast-division constants, tile counts) is interpreted here
exactly as the kernels do — unit -> (row indices, column) with multiply-high division — and applied with numpy to
host buffers, for randomly strided boxes.  If the packed description of a box is wrong in any way, the emulated copy
differs from plain tensor slicing.  Runs without a GPU."""

import ctypes as C
import random

import numpy as np
import pytest
import torch

from etha_b200.ops import lib as L
from etha_b200.ops.table import CopyTable, SliceRef

from test_table_pack import OpView


def _fast_div(n, mul, shr):
    return n if mul == 0 else ((n * mul) >> 32) >> shr


def _emulate(op: OpView, src_buf: np.ndarray, dst_buf: np.ndarray, src_base: int, dst_base: int):
    """Bit-copy ops only: walk every unit like tile_raw + unit_offsets."""
    ub = op.unit_bytes_src
    tiles = (op.total_units + op.tile_units - 1) // op.tile_units
    seen = 0
    for t in range(tiles):
        base = t * op.tile_units
        limit = min(op.total_units, base + op.tile_units)
        for unit in range(base, limit):
            q = _fast_div(unit, op.div_mul[4], op.div_shr[4])
            col = unit - q * op.inner_units
            so, do = col * op.unit_bytes_src, col * op.unit_bytes_dst
            for d in reversed(range(op.ndim)):
                q2 = 0 if d == 0 else _fast_div(q, op.div_mul[d], op.div_shr[d])
                i = q - q2 * op.extent[d]
                so += i * op.src_stride[d]
                do += i * op.dst_stride[d]
                q = q2
            s = op.src[0] - src_base + so
            for j in range(op.ndst):
                d0 = op.dst[j] - dst_base + do
                dst_buf[d0 : d0 + ub] = src_buf[s : s + ub]
            seen += 1
    assert seen == op.total_units


def _random_view(rng, t: torch.Tensor, shape):
    """A view of `t` with the given shape: random offsets, optional steps of the outer dims and permutation."""
    big = list(t.shape)
    idx = []
    for n, m in zip(shape, big):
        start = rng.randrange(0, m - n + 1)
        idx.append(slice(start, start + n))
    return t[tuple(idx)]


@pytest.mark.parametrize("seed", range(12))
def test_packed_ops_reproduce_strided_copies(seed):
    rng = random.Random(seed)
    dtype = rng.choice([torch.uint8, torch.int16, torch.float32, torch.float64, torch.bfloat16])
    ndim = rng.randint(1, 4)
    shape = [rng.randint(1, 9) for _ in range(ndim)]
    shape[-1] = rng.choice([1, 3, 8, 16, 24, 40])
    # build typed parents from byte patterns so that every dtype (bf16, fp64) carries arbitrary bits
    def parent(extra):
        dims = [n + e for n, e in zip(shape, extra)]
        nbytes = int(np.prod(dims)) * dtype.itemsize
        raw = torch.from_numpy(np.random.RandomState(seed).randint(0, 256, nbytes, dtype=np.uint8))
        return raw.view(dtype).view(dims)

    sp = parent([rng.randint(0, 4) for _ in shape])
    dp = torch.zeros_like(parent([rng.randint(0, 4) for _ in shape]))
    sv, dv = _random_view(rng, sp, shape), _random_view(rng, dp, shape)
    if ndim >= 2 and rng.random() < 0.3:  # a transposed pair: inner stride != 1 on both sides
        sv, dv = sv.transpose(0, -1), dv.transpose(0, -1)
    t = CopyTable(torch.device("cpu"), tile_bytes=rng.choice([64, 4096, 65536]))
    t.add(tuple(sv.shape), [SliceRef.of(sv)], [SliceRef.of(dv)])
    expect = dp.clone()
    # expected result through plain tensor assignment on a copy with identical layout
    ev = expect.as_strided(dv.shape, dv.stride(), dv.storage_offset())
    ev.copy_(sv)
    src_np = sp.contiguous().view(torch.uint8).numpy().reshape(-1)
    dst_np = dp.view(torch.uint8).numpy().reshape(-1)
    for cls, tiles, raw, *_ in t._packed:
        op = OpView.from_buffer_copy(raw)
        assert op.mode == 0
        _emulate(op, src_np, dst_np, sp.untyped_storage().data_ptr(), dp.untyped_storage().data_ptr())
    assert torch.equal(dp.view(torch.uint8), expect.view(torch.uint8))
