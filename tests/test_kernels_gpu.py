"""sm_100a copy / convert / reduce / flag kernels against plain PyTorch (fp32 reference arithmetic)."""

import pytest
import torch

from etha_b200 import ops
from etha_b200.comm.ir import PartialFamily, reduce_family_values
from etha_b200.ops import CopyTable, SliceRef

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, dtype, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype.is_floating_point:
        return torch.randn(shape, generator=g).to(dtype).to(DEV)
    return torch.randint(-100, 100, shape, generator=g).to(dtype).to(DEV)


def _run(table):
    table.finalize()
    table.launch()
    torch.cuda.synchronize()
    assert table.error_word() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int8, torch.int64, torch.float64])
@pytest.mark.parametrize("shape", [(1024, 4096), (333, 77), (5,), (1, 1), (3, 4, 5, 6)])
def test_contiguous_copy(dtype, shape):
    src = _rand(shape, dtype)
    dst = torch.zeros_like(src)
    t = CopyTable(DEV)
    t.add_copy(src, dst)
    _run(t)
    assert torch.equal(src, dst)


def test_many_ops_one_launch_llama_like_slices():
    # FSDP Shard(0) shard of o_proj [1024, 4096] -> four column blocks landing as contiguous rows of the
    # consumers' [4096, 1024] shards; plus q_proj-like contiguous pieces and a 2 KiB norm slice.
    src = _rand((1024, 4096), torch.bfloat16, 1)
    outs = [torch.zeros(4096, 1024, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    norm_src = _rand((1024,), torch.bfloat16, 2)
    norm_dst = [torch.zeros(4096, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    t = CopyTable(DEV)
    for j in range(4):
        t.add_copy(src[:, 1024 * j : 1024 * (j + 1)], outs[j][2048:3072])
    t.add((1024,), [SliceRef.of(norm_src)], [SliceRef.of(d[1024:2048]) for d in norm_dst])
    _run(t)
    for j in range(4):
        assert torch.equal(outs[j][2048:3072], src[:, 1024 * j : 1024 * (j + 1)])
        assert outs[j][:2048].abs().sum() == 0 and outs[j][3072:].abs().sum() == 0
        assert torch.equal(norm_dst[j][1024:2048], norm_src) and norm_dst[j][:1024].abs().sum() == 0


def test_slice_view_does_not_touch_neighbours():
    wide_src = _rand((8, 32, 64), torch.float32, 3)
    wide_dst = _rand((8, 32, 64), torch.float32, 4)
    keep = wide_dst.clone()
    t = CopyTable(DEV)
    t.add_copy(wide_src[:, :16, :], wide_dst[:, :16, :])
    _run(t)
    assert torch.equal(wide_dst[:, :16], wide_src[:, :16]) and torch.equal(wide_dst[:, 16:], keep[:, 16:])


@pytest.mark.parametrize("shape,sl", [((7, 33), None), ((64, 130), (slice(None), slice(1, 129))), ((129,), (slice(1, 128),))])
def test_unaligned_boxes(shape, sl):
    src = _rand(shape, torch.bfloat16, 5)
    dst = torch.zeros_like(src)
    sv, dv = (src, dst) if sl is None else (src[sl], dst[sl])
    t = CopyTable(DEV)
    t.add_copy(sv, dv)
    _run(t)
    want = torch.zeros_like(src)
    (want if sl is None else want[sl]).copy_(sv)
    assert torch.equal(dst, want)


def test_transposed_source():
    src = _rand((96, 160), torch.float16, 6)
    dst = torch.zeros(160, 96, dtype=torch.float16, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(src.t(), dst)
    _run(t)
    assert torch.equal(dst, src.t())


@pytest.mark.parametrize("sdt,ddt", [
    (torch.float32, torch.bfloat16), (torch.float32, torch.float16), (torch.bfloat16, torch.float32),
    (torch.float16, torch.float32), (torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16),
])
@pytest.mark.parametrize("shape", [(512, 1024), (33, 7)])
def test_conversion_matches_torch(sdt, ddt, shape):
    src = _rand(shape, sdt, 7) * 3.7
    dst = torch.zeros(shape, dtype=ddt, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(src, dst)
    _run(t)
    assert torch.equal(dst, src.to(ddt))


@pytest.mark.parametrize("sizes,opnames", [((4,), ("sum",)), ((2,), ("avg",)), ((3,), ("max",)), ((3,), ("min",)),
                                          ((2,), ("product",)), ((2, 2), ("sum", "sum")), ((2, 3), ("sum", "max")),
                                          ((2, 2), ("avg", "avg")), ((8,), ("sum",))])
@pytest.mark.parametrize("sdt,ddt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
def test_partial_collapse_matches_reference_arithmetic(sizes, opnames, sdt, ddt):
    n = 1
    for s in sizes:
        n *= s
    srcs = [_rand((256, 520), sdt, 100 + i) for i in range(n)]
    dst = torch.zeros(256, 520, dtype=ddt, device=DEV)
    t = CopyTable(DEV)
    t.add_reduce(srcs, dst, sizes, opnames)
    _run(t)
    fam = PartialFamily(ranks=tuple(range(n)), sizes=tuple(sizes), ops=tuple(opnames))
    want = reduce_family_values([s.cpu() for s in srcs], fam, sdt).to(ddt)
    assert torch.equal(dst.cpu(), want)
    for s, i in zip(srcs, range(n)):
        assert torch.equal(s, _rand((256, 520), sdt, 100 + i)), "sources must stay untouched"


def test_reduce_scalar_path_and_fanout():
    srcs = [_rand((9, 13), torch.float32, 200 + i) for i in range(3)]
    dsts = [torch.zeros(9, 13, dtype=torch.float32, device=DEV) for _ in range(2)]
    t = CopyTable(DEV)
    t.add((9, 13), [SliceRef.of(s) for s in srcs], [SliceRef.of(d) for d in dsts], (3,), ("sum",))
    _run(t)
    want = (srcs[0] + srcs[1]) + srcs[2]
    assert torch.equal(dsts[0], want) and torch.equal(dsts[1], want)


def test_flags_published_after_copy_and_bounded_wait():
    src = _rand((2048, 2048), torch.bfloat16, 9)
    dst = torch.zeros_like(src)
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    addrs = torch.tensor([flags.data_ptr() + 4 * 2, flags.data_ptr() + 4 * 5], dtype=torch.int64, device=DEV)
    status = torch.full((2,), 77, dtype=torch.int32, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(src, dst)
    t.finalize()
    t.launch(signals=addrs, epoch=3)
    ops.wait_flags(flags, torch.tensor([2, 5], dtype=torch.int32, device=DEV), 3, status, timeout_s=2.0)
    torch.cuda.synchronize()
    assert status.tolist()[0] == ops.STATUS_OK
    assert flags.tolist() == [0, 0, 3, 0, 0, 3, 0, 0]
    assert torch.equal(src, dst)
    # second launch reuses the arrival counter
    t.launch(signals=addrs, epoch=4)
    torch.cuda.synchronize()
    assert flags.tolist()[2] == 4


def test_wait_gives_up_and_reports_missing_flag():
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    flags[0] = 1
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops.wait_flags(flags, torch.tensor([0, 3], dtype=torch.int32, device=DEV), 1, status, timeout_s=0.2)
    torch.cuda.synchronize()
    assert status.tolist() == [ops.STATUS_TIMEOUT, 1]
    # the context is still usable
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_local_copy_helper():
    a = _rand((100, 200), torch.float32, 11)
    b = torch.zeros(100, 200, dtype=torch.bfloat16, device=DEV)
    ops.local_copy(a, b)
    torch.cuda.synchronize()
    assert torch.equal(b, a.to(torch.bfloat16))


@pytest.mark.parametrize("shape,cols", [((4096, 4096), None), ((2048, 4096), (1024, 2048)), ((777, 1024), None), ((64, 8192), (256, 4352))])
def test_tma_bulk_kernel_matches_ldst(shape, cols):
    src = _rand(shape, torch.bfloat16, 21)
    sv = src if cols is None else src[:, cols[0]:cols[1]]
    dst = torch.zeros(sv.shape, dtype=torch.bfloat16, device=DEV)
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    addrs = torch.tensor([flags.data_ptr() + 4], dtype=torch.int64, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(sv, dst)
    t.finalize()
    assert t.n_bulk_ops == t.n_ops[0] == 1
    for epoch in (1, 2):
        dst.zero_()
        t.launch(signals=addrs, epoch=epoch, bulk=True)
        torch.cuda.synchronize()
        assert t.error_word() == 0 and flags.tolist() == [0, epoch]
        assert torch.equal(dst, sv)


def test_tma_bulk_many_ops_and_fallback():
    srcs = [_rand((512 + 64 * i, 2048), torch.bfloat16, 30 + i) for i in range(9)]
    dsts = [torch.zeros_like(s) for s in srcs]
    t = CopyTable(DEV)
    for s, d in zip(srcs, dsts):
        t.add_copy(s, d)
    t.finalize()
    t.launch(bulk=True)
    torch.cuda.synchronize()
    assert t.n_bulk_ops == 9 and all(torch.equal(s, d) for s, d in zip(srcs, dsts))
    # a fan-out is read once per stage and stored to every replica by the TMA kernel
    a, b1, b2 = _rand((256, 256), torch.float32, 40), torch.zeros(256, 256, device=DEV), torch.zeros(256, 256, device=DEV)
    t2 = CopyTable(DEV)
    t2.add((256, 256), [SliceRef.of(a)], [SliceRef.of(b1), SliceRef.of(b2)])
    t2.finalize()
    assert t2.n_bulk_ops == 1
    t2.launch(bulk=True)
    torch.cuda.synchronize()
    assert t2.error_word() == 0 and torch.equal(a, b1) and torch.equal(a, b2)


def test_tma_bulk_mixed_table_splits_per_op():
    """Rows shorter than 512 bytes stay with the LD/ST kernel, everything else of the fast class goes through the
    TMA ring; the flag is published by whichever kernel runs last."""
    wide = _rand((1024, 4096), torch.bfloat16, 50)          # strided source rows of 2 KiB -> contiguous destination
    narrow = _rand((4096, 512), torch.bfloat16, 51)         # 128-byte rows: not TMA-capable
    vec = _rand((1024,), torch.bfloat16, 52)                # one 2 KiB run, three replicas
    d_wide = torch.zeros(1024, 1024, dtype=torch.bfloat16, device=DEV)
    d_narrow = torch.zeros(4096, 512, dtype=torch.bfloat16, device=DEV)
    reps = [torch.zeros(1024, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    flags = torch.zeros(1, dtype=torch.int32, device=DEV)
    addrs = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(narrow[:, 64:128], d_narrow[:, 64:128])
    t.add_copy(wide[:, 1024:2048], d_wide)
    t.add((1024,), [SliceRef.of(vec)], [SliceRef.of(r) for r in reps])
    t.finalize()
    assert t.n_ops[0] == 3 and t.n_bulk_ops == 2
    t.launch(signals=addrs, epoch=7, bulk=True)
    torch.cuda.synchronize()
    assert t.error_word() == 0 and flags.tolist() == [7]
    assert torch.equal(d_wide, wide[:, 1024:2048])
    assert all(torch.equal(r, vec) for r in reps)
    assert torch.equal(d_narrow[:, 64:128], narrow[:, 64:128]) and int(d_narrow[:, :64].count_nonzero()) == 0


@pytest.mark.parametrize("sdt,ddt", [
    (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.float16, torch.bfloat16),
    (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32),
])
@pytest.mark.parametrize("nsrc,opname", [(1, "sum"), (2, "sum"), (2, "avg"), (4, "sum"), (4, "max"), (2, "product"), (4, "min")])
@pytest.mark.parametrize("rows", [False, True])
def test_streaming_instances_equal_general_kernel(sdt, ddt, nsrc, opname, rows):
    """The per-(dtype pair, source count) streaming kernels must give the general kernel's bits: same accumulation
    order, same single rounding.  `rows`: source is a column block of a wider matrix (the matrix-row box form)."""
    if nsrc == 1 and sdt == ddt:
        pytest.skip("a same-dtype copy is a bit copy, not a typed op")
    if nsrc > 1 and sdt != ddt and torch.float32 not in (sdt, ddt):
        pytest.skip("collapses between the two 16-bit types have no streaming instance (general kernel)")
    wide = [_rand((384, 1024), sdt, 300 + i) * 1.7 for i in range(nsrc)]
    srcs = [w[:, 256:768] if rows else w[:, :512].contiguous() for w in wide]
    outs = {}
    for streaming in (True, False):
        dsts = [torch.zeros(384, 512, dtype=ddt, device=DEV) for _ in range(2)]
        t = CopyTable(DEV)
        t.stream_typed = streaming
        t.add((384, 512), [SliceRef.of(s) for s in srcs], [SliceRef.of(d) for d in dsts], (nsrc,) if nsrc > 1 else (),
              (opname,) if nsrc > 1 else ())
        t.finalize()
        assert t.n_typed_ops == (1 if streaming else 0)
        t.launch()
        torch.cuda.synchronize()
        assert t.error_word() == 0 and torch.equal(dsts[0], dsts[1])
        outs[streaming] = dsts[0]
    assert torch.equal(outs[True].view(torch.uint8), outs[False].view(torch.uint8))
    if nsrc == 1:
        assert torch.equal(outs[True], srcs[0].to(ddt))
    else:
        fam = PartialFamily(ranks=tuple(range(nsrc)), sizes=(nsrc,), ops=(opname,))
        want = reduce_family_values([s.cpu() for s in srcs], fam, sdt).to(ddt)
        assert torch.equal(outs[True].cpu(), want)


def test_streaming_and_general_ops_share_one_table():
    """A table with two streaming keys, a general-class op (3 sources) and bit copies: every class runs, the last
    kernel publishes the flag."""
    a32 = _rand((256, 512), torch.float32, 400)
    b16 = [_rand((256, 512), torch.bfloat16, 401 + i) for i in range(3)]
    raw = _rand((100, 64), torch.int32, 405)
    o_cvt = torch.zeros(256, 512, dtype=torch.bfloat16, device=DEV)
    o_red2 = torch.zeros(256, 512, dtype=torch.bfloat16, device=DEV)
    o_red3 = torch.zeros(256, 512, dtype=torch.bfloat16, device=DEV)
    o_raw = torch.zeros_like(raw)
    flags = torch.zeros(1, dtype=torch.int32, device=DEV)
    addrs = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=DEV)
    t = CopyTable(DEV)
    t.add_copy(a32, o_cvt)
    t.add_reduce(b16[:2], o_red2, (2,), ("sum",))
    t.add_reduce(b16, o_red3, (3,), ("sum",))
    t.add_copy(raw, o_raw)
    t.finalize()
    assert t.n_typed_ops == 2 and t.n_ops == [1, 3]
    t.launch(signals=addrs, epoch=5)
    torch.cuda.synchronize()
    assert t.error_word() == 0 and flags.tolist() == [5]
    assert torch.equal(o_cvt, a32.to(torch.bfloat16)) and torch.equal(o_raw, raw)
    assert torch.equal(o_red2, (b16[0].float() + b16[1].float()).to(torch.bfloat16))
    assert torch.equal(o_red3, ((b16[0].float() + b16[1].float()) + b16[2].float()).to(torch.bfloat16))
