"""Analytic planner against (a) DTensor's own shard arithmetic, (b) plans recorded from the reference."""

import itertools
import json
import math

import pytest
import torch
from torch.distributed.tensor._utils import _compute_local_shape_and_global_offset
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from etha_b200.comm import M2MMap, Transport, plan_m2m
from etha_b200.comm.ir import partial_family


def oracle_routes(smesh, splc, tmesh, tplc):
    """Brute force with DTensor's offset arithmetic: who owns which cell of the lcm grid."""
    eff = tuple(Replicate() if isinstance(p, Partial) else p for p in splc)
    ndim = max([p.dim for p in list(eff) + list(tplc) if isinstance(p, Shard)], default=0) + 1

    def counts(mesh, plc):
        c = [1] * ndim
        for n, p in zip(mesh.shape, plc):
            if isinstance(p, Shard):
                c[p.dim] *= n
        return c

    sc, tc = counts(smesh, eff), counts(tmesh, tplc)
    grid = tuple(math.lcm(a, b) for a, b in zip(sc, tc))
    s_coords = list(itertools.product(*[range(n) for n in smesh.shape]))
    t_coords = list(itertools.product(*[range(n) for n in tmesh.shape]))
    s_info = {}
    for c in s_coords:
        shape, off = _compute_local_shape_and_global_offset(grid, tuple(smesh.shape), list(c), eff)
        s_info[c] = (shape, off)
    non_shard = [i for i, p in enumerate(eff) if not isinstance(p, Shard)]
    table = {}
    for j, tcoord in enumerate(t_coords):
        fam = s_coords[j % len(s_coords)]
        tshape, toff = _compute_local_shape_and_global_offset(grid, tuple(tmesh.shape), list(tcoord), tplc)
        for tcell in itertools.product(*[range(n) for n in tshape]):
            g = [o + c for o, c in zip(toff, tcell)]
            owner = None
            for c in s_coords:
                if any(c[i] != fam[i] for i in non_shard):
                    continue
                shape, off = s_info[c]
                if all(o <= x < o + n for x, o, n in zip(g, off, shape)):
                    owner = c
                    scell = tuple(x - o for x, o in zip(g, off))
            assert owner is not None
            table.setdefault((int(smesh[owner]), scell), []).append((int(tmesh[tcoord]), tuple(tcell)))
    return table, grid, sc, tc


CASES = [
    ((2,), (Shard(0),), (2,), (Shard(1),)),
    ((4,), (Shard(0),), (4,), (Shard(1),)),
    ((4,), (Shard(0),), (4,), (Replicate(),)),
    ((4,), (Replicate(),), (4,), (Shard(0),)),
    ((1, 2, 2), (Replicate(), Shard(0), Shard(0)), (4,), (Shard(0),)),
    ((2, 2), (Replicate(), Shard(0)), (2, 2), (Replicate(), Shard(0))),
    ((1, 4), (Replicate(), Replicate()), (2, 2), (Replicate(), Shard(0))),
    ((2, 2), (Shard(0), Shard(0)), (4,), (Shard(0),)),
    ((2, 3), (Shard(0), Shard(1)), (3, 2), (Shard(1), Shard(0))),
    ((2, 2), (Shard(1), Replicate()), (8,), (Shard(0),)),
    ((2, 2, 2), (Replicate(), Shard(0), Shard(1)), (2, 1, 1, 2), (Replicate(), Replicate(), Replicate(), Shard(1))),
    ((3,), (Shard(0),), (2,), (Shard(0),)),
    ((6,), (Shard(2),), (4,), (Shard(0),)),
]


@pytest.mark.parametrize("sshape,splc,tshape,tplc", CASES)
def test_matches_dtensor_arithmetic(sshape, splc, tshape, tplc):
    ns, nt = math.prod(sshape), math.prod(tshape)
    smesh = torch.arange(ns).view(sshape)
    tmesh = torch.arange(ns, ns + nt).view(tshape)
    m = plan_m2m(smesh, splc, tmesh, tplc)
    table, grid, sc, tc = oracle_routes(smesh, splc, tmesh, tplc)
    assert m.source_num_slicers == [g // c for g, c in zip(grid, sc)]
    assert m.target_num_slicers == [g // c for g, c in zip(grid, tc)]
    got = {(r.src.rank, r.src.cell): sorted((d.rank, d.cell) for d in r.dsts) for r in m.routes}
    assert got == {k: sorted(v) for k, v in table.items()}
    keys = [(r.src.rank, r.src.cell) for r in m.routes]
    assert keys == sorted(keys)
    for r in m.routes:
        want = Transport.NONE if not r.dsts else (Transport.P2P if len(r.dsts) == 1 else Transport.BROADCAST)
        assert r.kind is want


def test_wire_format_matches_recorded_reference_plan():
    # JSON produced by the reference for Shard(0)x2 (ranks 0-1) -> Shard(1)x2 (ranks 2-3)
    recorded = {
        "routes": [
            {"src": {"rank": 0, "cell": [0, 0]}, "dsts": [{"rank": 2, "cell": [0, 0]}], "kind": "p2p"},
            {"src": {"rank": 0, "cell": [0, 1]}, "dsts": [{"rank": 3, "cell": [0, 0]}], "kind": "p2p"},
            {"src": {"rank": 1, "cell": [0, 0]}, "dsts": [{"rank": 2, "cell": [1, 0]}], "kind": "p2p"},
            {"src": {"rank": 1, "cell": [0, 1]}, "dsts": [{"rank": 3, "cell": [1, 0]}], "kind": "p2p"},
        ],
        "source_num_slicers": [1, 2],
        "target_num_slicers": [2, 1],
        "source_partial_reductions": [],
    }
    m = plan_m2m([0, 1], (Shard(0),), [2, 3], (Shard(1),))
    assert json.loads(m.to_json()) == recorded
    again = M2MMap.from_msgpack(m.to_msgpack())
    assert again.routes == m.routes and again.source_num_slicers == m.source_num_slicers
    assert M2MMap.from_json(json.dumps(recorded)).routes == m.routes


def test_partial_primaries_and_shadows_qwen_layout():
    # source mesh [[0,1],[2,3]] (Partial, Shard(0)) -> 4 ranks Shard(0): primaries follow j mod S
    m = plan_m2m([[0, 1], [2, 3]], (Partial(), Shard(0)), [4, 5, 6, 7], (Shard(0),))
    assert m.source_partial_reductions == [(0, "sum")]
    shipping = {(r.src.rank, r.src.cell): [d.rank for d in r.dsts] for r in m.routes if r.dsts}
    assert shipping == {(0, (0,)): [4], (0, (1,)): [5], (3, (0,)): [6], (3, (1,)): [7]}
    shadows = sorted((r.src.rank, r.src.cell) for r in m.routes if r.kind is Transport.NONE)
    assert shadows == [(1, (0,)), (1, (1,)), (2, (0,)), (2, (1,))]


def test_transitive_family_asymmetric_double_partial():
    # (2,3) mesh, both dims Partial, 2 replicate targets: all six ranks join every shipped cell
    m = plan_m2m(torch.arange(6).view(2, 3), (Partial(), Partial()), [6, 7], (Replicate(),))
    ranks_with_cell = sorted(r.src.rank for r in m.routes if r.src.cell == (0,))
    assert ranks_with_cell == [0, 1, 2, 3, 4, 5]
    assert sorted(r.src.rank for r in m.routes if r.dsts) == [0, 1]


def test_target_partial_rejected():
    with pytest.raises(NotImplementedError):
        plan_m2m([0, 1], (Shard(0),), [2, 3], (Partial(),))


def test_overlapping_meshes_plan():
    m = plan_m2m([0, 1], (Shard(0),), [0, 1], (Shard(1),))
    assert {(r.src.rank, d.rank) for r in m.routes for d in r.dsts} == {(0, 0), (0, 1), (1, 0), (1, 1)}


def test_partial_family_order():
    mesh = torch.arange(6).view(2, 3)
    fam = partial_family(mesh, [(0, "sum"), (1, "max")], 4)
    # first listed dim (mesh dim 0, size 2) varies fastest
    assert fam.ranks == (0, 3, 1, 4, 2, 5) and fam.sizes == (2, 3) and fam.ops == ("sum", "max")
    fam = partial_family(torch.arange(4).view(2, 2), [(1, "sum")], 2)
    assert fam.ranks == (2, 3)


# ---- property test: random meshes and placements against the DTensor-arithmetic oracle -------------------
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

_mesh_shape = st.lists(st.integers(1, 3), min_size=1, max_size=3).filter(lambda s: math.prod(s) <= 8)


def _placements(n, allow_partial):
    kinds = [st.just(Replicate()), st.builds(Shard, st.integers(0, 2))]
    if allow_partial:
        kinds.append(st.sampled_from([Partial(), Partial("max")]))
    return st.lists(st.one_of(*kinds), min_size=n, max_size=n).map(tuple)


@settings(max_examples=120, deadline=None)
@given(st.data())
def test_random_layouts_match_dtensor_arithmetic(data):
    ss = tuple(data.draw(_mesh_shape))
    ts = tuple(data.draw(_mesh_shape))
    sp = data.draw(_placements(len(ss), True))
    tp = data.draw(_placements(len(ts), False))
    ns, nt = math.prod(ss), math.prod(ts)
    overlap = data.draw(st.booleans())
    smesh = torch.arange(ns).view(ss)
    tmesh = torch.arange(0 if overlap else ns, (0 if overlap else ns) + nt).view(ts)
    m = plan_m2m(smesh, sp, tmesh, tp)
    table, grid, sc, tc = oracle_routes(smesh, sp, tmesh, tp)
    got = {(r.src.rank, r.src.cell): sorted((d.rank, d.cell) for d in r.dsts) for r in m.routes if r.dsts}
    assert got == {k: sorted(v) for k, v in table.items()}
    assert m.source_num_slicers == [g // c for g, c in zip(grid, sc)]
    # every consumer cell is delivered exactly once
    delivered = [(d.rank, d.cell) for r in m.routes for d in r.dsts]
    assert len(delivered) == len(set(delivered)) == nt * math.prod(m.target_num_slicers)
    # reduce-only entries exist exactly for the other members of a Partial family
    if any(isinstance(p, Partial) for p in sp):
        red = [(i, p.reduce_op) for i, p in enumerate(sp) if isinstance(p, Partial)]
        for r in [r for r in m.routes if r.dsts]:
            fam = partial_family(smesh, red, r.src.rank)
            for q in fam.ranks:
                assert any(x.src.rank == q and x.src.cell == r.src.cell for x in m.routes)
    else:
        assert all(r.dsts for r in m.routes)
