"""The allocation-free entry point (`etha_m2n_run_noalloc`, no_alloc.h) against the table API.

A weight-sync hook inside an inference worker often cannot allocate: the worker has given the free device
memory to its KV-cache pool.  Such a caller passes only its own source and destination tensors; the op table
and the counters live in an array inside the loaded library.  The test drives the exported C symbol through
ctypes, twice in a row with different work (the array keeps whatever the first call left), and compares bit
for bit with `CopyTable`, which is how every other kernel test in this suite compares.
"""

import ctypes as C

import pytest
import torch

from etha_b200.ops import CopyTable, SliceRef
from etha_b200.ops import lib as L
from etha_b200.ops.table import dtype_code

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_OPS = 64


def _spec(shape, srcs, dsts, red_sizes=(), red_ops=()):
    """Fill one M2NOpSpec from tensor views (sources share shape/strides; destinations too)."""
    s = L.OpSpec()
    s.ndim = len(shape)
    for i, n in enumerate(shape):
        s.shape[i] = n
        s.src_stride[i] = srcs[0].stride(i)
        s.dst_stride[i] = dsts[0].stride(i)
    s.src_itemsize, s.dst_itemsize = srcs[0].dtype.itemsize, dsts[0].dtype.itemsize
    s.src_dtype, s.dst_dtype = dtype_code(srcs[0].dtype), dtype_code(dsts[0].dtype)
    s.nsrc, s.ndst = len(srcs), len(dsts)
    for i, t in enumerate(srcs):
        r = SliceRef.of(t)
        s.src[i], s.src_lo[i], s.src_hi[i] = r.ptr, r.lo, r.hi
    for i, t in enumerate(dsts):
        r = SliceRef.of(t)
        s.dst[i], s.dst_lo[i], s.dst_hi[i] = r.ptr, r.lo, r.hi
    sizes = list(red_sizes) or [len(srcs)]
    ops = list(red_ops) or ["sum"]
    s.red_size[0], s.red_size[1] = sizes[0], (sizes[1] if len(sizes) > 1 else 1)
    s.red_op[0] = L.RED_CODES[ops[0]]
    s.red_op[1] = L.RED_CODES[ops[1]] if len(ops) > 1 else 0
    s.tile_bytes = 65536
    return s


def _entry():
    lib = L.cuda_lib()
    fn = lib.etha_m2n_run_noalloc
    fn.argtypes = [C.POINTER(L.OpSpec), C.c_uint32, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    st = lib.etha_m2n_noalloc_status
    st.argtypes = [C.POINTER(C.c_uint32), C.c_void_p]
    st.restype = C.c_int
    return fn, st


def _workload(seed):
    """(specs for the no-alloc call, outputs it writes, table doing the same work, outputs of the table)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape, dtype=torch.bfloat16: torch.randn(*shape, generator=g).to(dtype).to(DEV)
    a = rnd(1024, 1024)  # contiguous copy (fast kernel, one run)
    b = rnd(512, 4096)  # column block -> contiguous rows (fast kernel, matrix rows)
    c = rnd(256, 520, dtype=torch.float32)  # fp32 -> bf16 conversion (general kernel)
    d0, d1 = rnd(256, 520), rnd(256, 520)  # two pending values collapsed in fp32 (general kernel)
    e = rnd(7, 33)  # odd sizes: 2-byte units
    outs = lambda: [
        torch.zeros(1024, 1024, dtype=torch.bfloat16, device=DEV),
        torch.zeros(512, 1024, dtype=torch.bfloat16, device=DEV),
        torch.zeros(256, 520, dtype=torch.bfloat16, device=DEV),
        torch.zeros(256, 520, dtype=torch.bfloat16, device=DEV),
        torch.zeros(7, 33, dtype=torch.bfloat16, device=DEV),
        torch.zeros(7, 33, dtype=torch.bfloat16, device=DEV),
    ]
    o, r = outs(), outs()
    work = lambda out: [
        ((1024, 1024), [a], [out[0]], (), ()),
        ((512, 1024), [b[:, 1024:2048]], [out[1]], (), ()),
        ((256, 520), [c], [out[2]], (), ()),
        ((256, 520), [d0, d1], [out[3]], (2,), ("sum",)),
        ((7, 33), [e], [out[4], out[5]], (), ()),
    ]
    specs = (L.OpSpec * 5)(*[_spec(*w) for w in work(o)])
    table = CopyTable(DEV)
    for shape, srcs, dsts, sizes, ops in work(r):
        table.add(shape, [SliceRef.of(t) for t in srcs], [SliceRef.of(t) for t in dsts], sizes, ops)
    table.finalize()
    return specs, o, table, r, (a, b, c, d0, d1, e)


def test_no_alloc_entry_point_matches_table_api_twice():
    run, status = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    for seed in (1, 2):  # second call reuses the array with the first call's contents in it
        specs, got, table, want, keep = _workload(seed)
        rc = run(specs, len(specs), 0, stream)
        assert rc == 0, L.last_error()
        table.launch()
        torch.cuda.synchronize()
        word = C.c_uint32(99)
        assert status(C.byref(word), stream) == 0 and word.value == 0
        assert table.error_word() == 0
        for g_, w_ in zip(got, want):
            assert torch.equal(g_, w_)
        assert torch.equal(got[0], keep[0]) and got[3].abs().sum() > 0


def test_no_alloc_entry_point_rejects_oversized_requests():
    run, _ = _entry()
    src = torch.ones(64, device=DEV)
    dst = torch.zeros(64, device=DEV)
    specs = (L.OpSpec * (MAX_OPS + 1))(*[_spec((64,), [src], [dst]) for _ in range(MAX_OPS + 1)])
    rc = run(specs, MAX_OPS + 1, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -100 and "at most 64" in L.last_error()
    assert float(dst.sum()) == 0.0, "a refused call must not launch anything"
    # exactly the maximum is accepted
    rc = run(specs, MAX_OPS, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(dst, src)
