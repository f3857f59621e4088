"""MoE weight sync with the layouts of a real disaggregated RL job, one worker process (trainer or inference rank).

Trainer side (`--trainer-mesh AxB`, ranks 0..AB-1):
  * dense weights on the 2-D HSDP mesh (dp_replicate=A, dp_shard=B): `(Replicate, Shard(0))` for embeddings, the
    attention input projections and lm_head, `(Replicate, Shard(1))` for o_proj, `(Replicate, Replicate)` for
    router and norms;
  * stacked expert weights `[E, ...]` on the 3-D mesh (1, A, B) = (dp_replicate, dp_shard, ep) with
    `(Replicate, Shard(0), Shard(0))`: both dp_shard and ep cut the expert axis.
Inference side (`--inference-mesh CxD`, the following CD ranks): dense weights tensor-parallel on (dp=C, tp=D) with
`(Replicate, Shard(0))` / `(Replicate, Shard(1))`, experts expert-parallel on the 1-D mesh of all CD ranks.

Eight named pairs, one per layout class, as in the reference's example (examples/vllm_weight_sync/common.py:117-126,
trainer.py:150-170).  Fused tensors are registered as slice VIEWS and never copied: the inference rank owns one fused
`qkv_proj` per layer and registers its q, k and v row blocks, the trainer owns a fused `gate_up_proj` per layer and
registers the gate and up halves, which the inference rank receives into the swapped halves ([up; gate]) of its
`w13` (trainer.py:173-202, vllm_server.py:182-196).  Every fused buffer carries guard rows that must stay untouched.

Each round is gated on control keys in the agents' store, like the reference's loop (trainer.py:217-249,
vllm_server.py:293-325): the trainer perturbs its weights, sends, publishes `trainer_version`, and waits until every
inference rank has bumped `inference_version/{rank}` after receiving and verifying that round.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
from torch.distributed.tensor.placement_types import Replicate, Shard  # noqa: E402

from etha_b200.kvstore import TorchTCPStore  # noqa: E402
from etha_b200.models.sync import local_shape_and_offset  # noqa: E402
from etha_b200.tensor_bus.bootstrap import bootstrap_client  # noqa: E402

R = Replicate()
# model: a small MoE decoder; every dim divides by 4
LAYERS, HIDDEN, HEADS, KV_HEADS, HEAD_DIM, EXPERTS, FFN, VOCAB = 2, 128, 8, 4, 16, 8, 64, 512
GUARD = 3  # guard rows around fused buffers

# pair name -> (trainer placements, inference placements, "dense" | "moe")
PAIRS = {
    "embed_tokens": ((R, Shard(0)), (R, Shard(0)), "dense"),
    "qkv_proj": ((R, Shard(0)), (R, Shard(0)), "dense"),
    "o_proj": ((R, Shard(1)), (R, Shard(1)), "dense"),
    "router": ((R, R), (R, R), "dense"),
    "layernorm": ((R, R), (R, R), "dense"),
    "lm_head": ((R, Shard(0)), (R, Shard(0)), "dense"),
    "experts_gate_up": ((R, Shard(0), Shard(0)), (Shard(0),), "moe"),
    "experts_down": ((R, Shard(0), Shard(0)), (Shard(0),), "moe"),
}


def logical_tensors() -> list[tuple[str, str, tuple[int, ...]]]:
    """(name, pair, global shape) in the order both sides register them (sorted by pair, then name)."""
    out = [("embed_tokens", "embed_tokens", (VOCAB, HIDDEN)), ("lm_head", "lm_head", (VOCAB, HIDDEN)),
           ("norm", "layernorm", (HIDDEN,))]
    for i in range(LAYERS):
        p = f"layers.{i}."
        out += [
            (p + "q_proj", "qkv_proj", (HEADS * HEAD_DIM, HIDDEN)),
            (p + "k_proj", "qkv_proj", (KV_HEADS * HEAD_DIM, HIDDEN)),
            (p + "v_proj", "qkv_proj", (KV_HEADS * HEAD_DIM, HIDDEN)),
            (p + "o_proj", "o_proj", (HIDDEN, HEADS * HEAD_DIM)),
            (p + "input_layernorm", "layernorm", (HIDDEN,)),
            (p + "router", "router", (EXPERTS, HIDDEN)),
            (p + "experts.gate_proj", "experts_gate_up", (EXPERTS, FFN, HIDDEN)),
            (p + "experts.up_proj", "experts_gate_up", (EXPERTS, FFN, HIDDEN)),
            (p + "experts.down_proj", "experts_down", (EXPERTS, HIDDEN, FFN)),
        ]
    return sorted(out, key=lambda t: (t[1], t[0]))


def stable_hash_seed(name: str) -> int:
    h = 0
    for ch in name:
        h = (h * 131 + ord(ch)) % (2**31 - 1)
    return h


def full_value(name: str, shape, version: int) -> torch.Tensor:
    """Logical value of a parameter at a given version: seeded randn (the seed does not depend on the process),
    scaled by 2**-version, which is exact in bf16."""
    g = torch.Generator().manual_seed(stable_hash_seed(name))
    return (torch.randn(shape, generator=g) * 0.05).to(torch.bfloat16).float() * (0.5**version)


def shard_of(full: torch.Tensor, mesh: torch.Tensor, placements, rank: int) -> torch.Tensor:
    shape, off = local_shape_and_offset(tuple(full.shape), mesh, placements, rank)
    return full[tuple(slice(o, o + n) for o, n in zip(off, shape))]


class FusedBuffer:
    """Several parameters stacked along dim `dim` of one allocation, with guard rows before and after."""

    def __init__(self, parts: list[tuple[str, tuple[int, ...]]], dim: int, device, fill: float):
        lead = parts[0][1]
        total = sum(s[dim] for _, s in parts)
        shape = list(lead)
        shape[dim] = total + 2 * GUARD
        self.buf = torch.full(shape, fill, dtype=torch.bfloat16, device=device)
        self.dim, self.views, cur = dim, {}, GUARD
        for name, s in parts:
            self.views[name] = self.buf.narrow(dim, cur, s[dim])
            cur += s[dim]
        self.fill = fill

    def guards_intact(self) -> bool:
        n = self.buf.shape[self.dim]
        lo, hi = self.buf.narrow(self.dim, 0, GUARD), self.buf.narrow(self.dim, n - GUARD, GUARD)
        return bool((lo == self.fill).all() and (hi == self.fill).all())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", required=True, choices=["trainer", "inference"])
    ap.add_argument("--trainer-mesh", default="2x2")
    ap.add_argument("--inference-mesh", default="2x2")
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--path-prefix", required=True)
    ap.add_argument("--store-port", type=int, required=True)
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args()
    A, B = (int(x) for x in args.trainer_mesh.split("x"))
    Cc, D = (int(x) for x in args.inference_mesh.split("x"))
    T, I = A * B, Cc * D
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if args.device == "cuda" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    client, info = bootstrap_client(lambda r: (f"{args.path_prefix}{r}_command.lmdb", f"{args.path_prefix}{r}_state.lmdb"),
                                    connection_timeout=120.0)
    me = info.agent_rank
    trainer = args.role == "trainer"
    local_name, remote_name = ("trainer", "inference") if trainer else ("inference", "trainer")
    t_ranks, i_ranks = torch.arange(T), torch.arange(T, T + I)
    meshes = {  # (pair kind, side) -> mesh of agent ranks
        ("dense", True): t_ranks.view(A, B), ("moe", True): t_ranks.view(1, A, B),
        ("dense", False): i_ranks.view(Cc, D), ("moe", False): i_ranks.view(I),
    }
    # the control plane: plain keys on the agents' store (not part of the bus)
    control = TorchTCPStore("127.0.0.1", args.store_port, world_size=-1, is_master=False, wait_for_workers=False,
                            namespace="control", timeout=600.0)

    pending = []
    for pair, (tp_t, tp_i, kind) in PAIRS.items():
        mesh = meshes[(kind, trainer)]
        pending.append(client.init_pair(pair, local_name, remote_name, T if trainer else I, mesh, tp_t if trainer else tp_i,
                                        blocking=False))
    for p in pending:
        p.acquire(180.0)

    # ---- local tensors -------------------------------------------------------------------------------------
    tensors = logical_tensors()
    local: dict[str, torch.Tensor] = {}
    fused: list[FusedBuffer] = []

    def local_shape(name, pair, shape):
        tp_t, tp_i, kind = PAIRS[pair]
        return tuple(local_shape_and_offset(shape, meshes[(kind, trainer)], tp_t if trainer else tp_i, me)[0])

    by_name = {n: (p, s) for n, p, s in tensors}
    for i in range(LAYERS):
        p = f"layers.{i}."
        if trainer:  # fused gate_up: [E_local, 2*FFN (+guards), H], gate first
            parts = [(p + "experts.gate_proj", local_shape(p + "experts.gate_proj", "experts_gate_up", by_name[p + "experts.gate_proj"][1])),
                     (p + "experts.up_proj", local_shape(p + "experts.up_proj", "experts_gate_up", by_name[p + "experts.up_proj"][1]))]
            fb = FusedBuffer(parts, 1, dev, 7.0)
        else:  # fused qkv rows, and w13 with the halves swapped: [up; gate]
            parts = [(p + n, local_shape(p + n, "qkv_proj", by_name[p + n][1])) for n in ("q_proj", "k_proj", "v_proj")]
            fb = FusedBuffer(parts, 0, dev, 7.0)
            fused.append(fb)
            local.update(fb.views)
            parts = [(p + "experts.up_proj", local_shape(p + "experts.up_proj", "experts_gate_up", by_name[p + "experts.up_proj"][1])),
                     (p + "experts.gate_proj", local_shape(p + "experts.gate_proj", "experts_gate_up", by_name[p + "experts.gate_proj"][1]))]
            fb = FusedBuffer(parts, 1, dev, 7.0)
        fused.append(fb)
        local.update(fb.views)
    for name, pair, shape in tensors:
        if name not in local:
            local[name] = torch.zeros(local_shape(name, pair, shape), dtype=torch.bfloat16, device=dev)

    def expected(name, version):
        pair, shape = by_name[name]
        tp_t, tp_i, kind = PAIRS[pair]
        return shard_of(full_value(name, shape, version), meshes[(kind, trainer)], tp_t if trainer else tp_i, me).to(torch.bfloat16)

    if trainer:
        for name in local:
            local[name].copy_(expected(name, 0))
    batch = client.register_tensors("weights", [(local[name], pair) for name, pair, _ in tensors], timeout=300.0)

    # ---- gated rounds ----------------------------------------------------------------------------------------
    bad = 0
    for rnd in range(1, args.rounds + 1):
        if trainer:
            for name in local:  # "training": every weight changes (x 1/2, exact), in place, views included
                local[name].mul_(0.5)
            if dev.type == "cuda":
                torch.cuda.synchronize()
            batch.transfer("send", blocking=True, timeout=300.0)
            if me == 0:
                control.set("trainer_version", str(rnd))
            # the next round starts only after every inference rank has consumed this one
            for r in range(T, T + I):
                control.wait_for_value(f"inference_version/{r}", str(rnd), timeout=300.0)
        else:
            while not batch.query_transfer_signal(timeout=60.0):
                time.sleep(0.002)
            batch.transfer("recv", blocking=True, timeout=300.0)
            for name in local:
                if not torch.equal(local[name].cpu(), expected(name, rnd)):
                    bad += 1
            bad += sum(0 if fb.guards_intact() else 1 for fb in fused)
            control.set(f"inference_version/{me}", str(rnd))
    if trainer:
        bad += sum(0 if fb.guards_intact() else 1 for fb in fused)
    print(json.dumps({"role": args.role, "agent_rank": me, "rounds": args.rounds, "tensors": len(tensors), "pairs": len(PAIRS),
                      "mismatches": bad, "golden_match": bad == 0}), flush=True)
    batch.close()
    client.close()
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
