"""Peer-to-peer executor on one GPU: every logical rank lives in this process (no IPC), so the whole
plan -> copy table -> kernels -> flags path runs against the same expectations as the CPU matrix."""

import math

import pytest
import torch
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from etha_b200.comm.baselines import local_slice_of
from etha_b200.comm.p2p import P2PBatch, PairLayout, link_local

from test_reshard_cpu import CASES_8, _make_source_local

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
R = Replicate()


def _run_case(case, overlap, src_dtype=torch.float32, tgt_dtype=torch.float32):
    sshape, splc, tshape, tplc, shape, slice_view = case
    ns, nt = math.prod(sshape), math.prod(tshape)
    smesh = torch.arange(ns).view(sshape)
    t0 = 0 if overlap else ns
    tmesh = torch.arange(t0, t0 + nt).view(tshape)
    ranks = sorted(set(smesh.reshape(-1).tolist()) | set(tmesh.reshape(-1).tolist()))
    eff = tuple(R if isinstance(p, Partial) else p for p in splc)
    wide = list(shape)
    if slice_view:
        wide[1] *= 2
    logical, contribs = _make_source_local(0, smesh, splc, tuple(wide), src_dtype, slice_view)
    g = torch.Generator().manual_seed(99)
    tgt_init_full = torch.randn(tuple(wide), generator=g).to(tgt_dtype)
    layout = PairLayout(smesh, splc, tmesh, tplc)

    batches, srcs, tgts, backs = [], {}, {}, {}
    for r in ranks:
        src = tgt = None
        if r in smesh.reshape(-1).tolist():
            base = (contribs[r] if contribs is not None else local_slice_of(logical, smesh, eff, r)).clone().to(DEV)
            src = base[:, : shape[1]] if slice_view else base
            srcs[r] = (src, src.clone())
        if r in tmesh.reshape(-1).tolist():
            back = local_slice_of(tgt_init_full, tmesh, tplc, r).clone().to(DEV)
            tgt = back[:, : shape[1]] if slice_view else back
            tgts[r], backs[r] = tgt, back
        b = P2PBatch(r, ranks, DEV)
        b.add(layout, src, tgt)
        batches.append(b)
    link_local(batches)
    for _ in range(2):  # two transfers: epochs advance, arrival counters are reused
        for b in batches:
            b.begin()
            b.send()
        for b in batches:
            b.recv(timeout_s=2.0)
        torch.cuda.synchronize()
        for b in batches:
            b.check()
    for r, (src, snap) in srcs.items():
        assert torch.equal(src, snap), "source modified"
    for r, tgt in tgts.items():
        want = local_slice_of(logical, tmesh, tplc, r)
        want = (want[:, : shape[1]] if slice_view else want).to(tgt_dtype).to(DEV)
        assert torch.equal(tgt, want), f"rank {r}: max diff {(tgt.float() - want.float()).abs().max()}"
        if slice_view:
            untouched = local_slice_of(tgt_init_full, tmesh, tplc, r)[:, shape[1]:].to(DEV)
            assert torch.equal(backs[r][:, shape[1]:], untouched)


@pytest.mark.parametrize("case", CASES_8, ids=[str(i) for i in range(len(CASES_8))])
def test_reshard_matrix_disjoint(case):
    _run_case(case, overlap=False)


@pytest.mark.parametrize("case", CASES_8, ids=[str(i) for i in range(len(CASES_8))])
def test_reshard_matrix_overlapping(case):
    _run_case(case, overlap=True)


UNEVEN = [
    ((2,), (Shard(0),), (2,), (Shard(1),), (1000, 333), False),
    ((2,), (Shard(0),), (2,), (Shard(1),), (7, 4096), False),
    ((2, 2), (Shard(0), Shard(1)), (3,), (Shard(0),), (10, 7), False),
    ((2,), (Partial(),), (2,), (Shard(0),), (5, 3), False),
]


@pytest.mark.parametrize("case", UNEVEN, ids=[str(i) for i in range(len(UNEVEN))])
def test_uneven_shards(case):
    _run_case(case, overlap=False)


@pytest.mark.parametrize("sd,td", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_dtype_pairs(sd, td):
    _run_case(CASES_8[12], False, sd, td)  # 2-D shard swap
    _run_case(CASES_8[5], False, sd, td)  # Partial -> Replicate: fp32 accumulation, one rounding


def test_timeout_is_reported_not_fatal():
    # a consumer whose producer never sends: the bounded wait reports which producer is missing
    layout = PairLayout(torch.tensor([0]), (R,), torch.tensor([1]), (R,))
    src = torch.ones(64, device=DEV)
    tgt = torch.zeros(64, device=DEV)
    a, b = P2PBatch(0, [0, 1], DEV), P2PBatch(1, [0, 1], DEV)
    a.add(layout, src, None)
    b.add(layout, None, tgt)
    link_local([a, b])
    b.begin()
    b.recv(timeout_s=0.2)
    torch.cuda.synchronize()
    from etha_b200.comm.p2p import TransferTimeout

    with pytest.raises(TransferTimeout, match="producer rank 0"):
        b.check()
    # the late producer still completes the same epoch and a fresh wait succeeds
    a.begin()
    a.send()
    b.recv(timeout_s=2.0)
    torch.cuda.synchronize()
    b.check()
    assert torch.equal(tgt, src)


def test_weight_sync_tiny_model_single_gpu():
    from etha_b200.models import fsdp_layout, tiny_llama, vllm_tp_layout
    from etha_b200.models.sync import WeightSync

    mesh = torch.tensor([0])
    ws = WeightSync(tiny_llama(), 0, [0], DEV, mesh, mesh, fsdp_layout(), vllm_tp_layout()).build()
    ws.sync()
    torch.cuda.synchronize()
    ws.check()
    assert ws.verify() == 0
