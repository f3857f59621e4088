"""Copy-engine lowering of table ops, checked on the host: the 1-D / pitched 2-D copies an op is turned into move
exactly the op's box, ops a DMA engine cannot run are left to the kernels, and the byte-budget selection takes the
largest candidates first while keeping table order."""

import numpy as np
import pytest
import torch

from etha_b200.ops import lib as L
from etha_b200.ops.table import CopyTable, SliceRef

BASE_S, BASE_D = 1 << 40, 2 << 40


def _table(**kw):
    t = CopyTable.__new__(CopyTable)
    CopyTable.__init__(t, torch.device("cpu"), **kw)
    return t


def _ref(base, view: torch.Tensor, storage_bytes: int, origin: torch.Tensor) -> SliceRef:
    off = view.data_ptr() - origin.data_ptr()
    return SliceRef(base + off, tuple(view.stride()), view.dtype, base, base + storage_bytes)


def _apply(copies, src_buf: np.ndarray, dst_buf: np.ndarray):
    for c in copies:
        for row in range(c.height):
            s = c.src - BASE_S + row * c.spitch
            d = c.dst - BASE_D + row * c.dpitch
            dst_buf[d : d + c.width] = src_buf[s : s + c.width]


@pytest.mark.parametrize("case", ["contiguous", "column_block", "into_column_block", "odd_bytes"])
def test_copies_move_exactly_the_box(case):
    src = torch.randn(64, 96).to(torch.bfloat16)
    dst = torch.zeros(64, 96, dtype=torch.bfloat16)
    sv, dv = {"contiguous": (src, dst), "column_block": (src[:, 32:64], dst.view(-1)[: 64 * 32].view(64, 32)),
              "into_column_block": (src.view(-1)[: 64 * 32].view(64, 32), dst[:, 16:48]),
              "odd_bytes": (src[3:10, 1:8], dst[5:12, 2:9])}[case]
    t = _table(dma_min_bytes=0)
    t.add(tuple(sv.shape), [_ref(BASE_S, sv, src.numel() * 2, src)], [_ref(BASE_D, dv, dst.numel() * 2, dst)], dma_ok=True)
    assert len(t._dma_candidates) == 1
    taken = t._select_dma()
    assert taken == {0} and t.dma_bytes == sv.numel() * 2
    s_np = src.view(torch.uint8).numpy().reshape(-1).copy()
    d_np = np.zeros(dst.numel() * 2, dtype=np.uint8)
    _apply(t._dma, s_np, d_np)
    want = torch.zeros_like(dst)
    want_view = {"contiguous": want, "column_block": want.view(-1)[: 64 * 32].view(64, 32), "into_column_block": want[:, 16:48],
                 "odd_bytes": want[5:12, 2:9]}[case]
    want_view.copy_(sv)
    assert np.array_equal(d_np, want.view(torch.uint8).numpy().reshape(-1))


def test_ops_a_dma_engine_cannot_run_stay_with_the_kernels():
    a = torch.randn(32, 64)
    b16 = torch.zeros(32, 64, dtype=torch.bfloat16)
    cube_s, cube_d = torch.randn(4, 8, 16), torch.zeros(4, 8, 16)
    t = _table(dma_min_bytes=0)
    ref = lambda base, x, origin: _ref(base, x, origin.numel() * origin.element_size(), origin)
    t.add((32, 64), [ref(BASE_S, a, a)], [ref(BASE_D, b16, b16)], dma_ok=True)  # conversion
    t.add((32, 64), [ref(BASE_S, a, a), ref(BASE_S + (1 << 30), a, a)], [ref(BASE_D, a, a)], (2,), ("sum",), dma_ok=True)  # collapse
    t.add((4, 4, 8), [ref(BASE_S, cube_s[:, :4, :8], cube_s)], [ref(BASE_D, cube_d[:, 4:, 8:], cube_d)], dma_ok=True)  # 2 strided dims
    t.add((32, 64), [ref(BASE_S, a, a)], [ref(BASE_D, a, a)], dma_ok=False)  # a local destination
    assert not t._dma_candidates and len(t._packed) == 4
    t2 = _table(dma_min_bytes=1 << 20)
    t2.add((32, 64), [ref(BASE_S, a, a)], [ref(BASE_D, a, a)], dma_ok=True)  # below the size floor
    assert not t2._dma_candidates


def test_selection_takes_the_largest_first_within_the_budget_and_keeps_table_order():
    big = torch.zeros(1 << 20, dtype=torch.uint8)
    t = _table(dma_min_bytes=1024, dma_fraction=0.7)
    sizes = [100_000, 400_000, 50_000, 300_000, 150_000]  # 1 000 000 bytes delivered: budget 700 000
    off = 0
    for n in sizes:
        v = big[off : off + n]
        t.add((n,), [_ref(BASE_S, v, big.numel(), big)], [_ref(BASE_D, v, big.numel(), big)], dma_ok=True)
        off += n
    taken = t._select_dma()
    assert taken == {1, 3}  # 400 000 + 300 000; 150 000 would exceed the budget, and so would every smaller one
    assert t.dma_bytes == 700_000 and [c.width for c in t._dma] == [400_000, 300_000]
    # a fan-out op becomes one copy per destination
    t3 = _table(dma_min_bytes=0)
    v = big[:4096]
    t3.add((4096,), [_ref(BASE_S, v, big.numel(), big)], [_ref(BASE_D, v, big.numel(), big), _ref(BASE_D + 8192, v, big.numel(), big)],
           dma_ok=True)
    t3._select_dma()
    assert [(c.dst - BASE_D, c.width, c.height) for c in t3._dma] == [(0, 4096, 1), (8192, 4096, 1)]
