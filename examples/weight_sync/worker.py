"""One worker of the weight-sync example: a trainer rank (holds FSDP shards, sends) or an inference rank (a
stand-in for a vLLM worker: holds the tensor-parallel layout, receives and verifies).

Mirrors the roles of the reference's example (examples/vllm_weight_sync/trainer.py, vllm_server.py) without
vLLM, a checkpoint or the network: weights are random-initialised from per-tensor seeds, so the consumer can
regenerate what it must have received and compare bit for bit.
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

from etha_b200.models import fsdp_layout, vllm_tp_layout  # noqa: E402
from etha_b200.models.sync import full_tensor_for, local_shape_and_offset  # noqa: E402
from etha_b200.tensor_bus.bootstrap import bootstrap_client  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", required=True, choices=["trainer", "inference"])
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--side-size", type=int, required=True, help="ranks on each side")
    ap.add_argument("--syncs", type=int, default=3)
    ap.add_argument("--path-prefix", default="/tmp/agent_rank")
    ap.add_argument("--source-dtype", default="bfloat16")
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args()
    sys.path.insert(0, ROOT)
    from bench import model_of

    rank = int(os.environ["RANK"])  # rank within this side
    n = args.side_size
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if args.device == "cuda" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    naming = None if args.path_prefix == "/tmp/agent_rank" else (
        lambda r: (f"{args.path_prefix}{r}_command.lmdb", f"{args.path_prefix}{r}_state.lmdb"))
    client, info = bootstrap_client(naming, connection_timeout=60.0)
    trainer = args.role == "trainer"
    me, other = ("trainer", "inference") if trainer else ("inference", "trainer")
    model = model_of(args.model)
    s_rule, t_rule = fsdp_layout(), vllm_tp_layout()
    smesh, tmesh = torch.arange(n), torch.arange(n, 2 * n)  # agent ranks of the two sides
    src_dtype, dst_dtype = getattr(torch, args.source_dtype), torch.bfloat16

    # one pair per distinct (source placements, target placements)
    pairs: dict[tuple, str] = {}
    entries = []
    for k, spec in enumerate(model.tensors):
        sp, tp = tuple(s_rule(spec)), tuple(t_rule(spec))
        name = pairs.setdefault((sp, tp), f"pair{len(pairs)}")
        entries.append((k, spec, sp, tp, name))
    pending = [client.init_pair(name, me, other, n, smesh if trainer else tmesh, sp if trainer else tp, blocking=False)
               for (sp, tp), name in pairs.items()]
    for p in pending:
        p.acquire(120.0)

    agent_rank = info.agent_rank
    tensors = []
    for k, spec, sp, tp, name in entries:
        mesh, plc = (smesh, sp) if trainer else (tmesh, tp)
        shape, off = local_shape_and_offset(spec.shape, mesh, plc, agent_rank)
        if trainer:
            full = full_tensor_for(spec, k, 2, torch.float32, dev)
            t = full[tuple(slice(o, o + s) for o, s in zip(off, shape))].to(src_dtype).contiguous()
        else:
            t = torch.zeros(shape, dtype=dst_dtype, device=dev)
        tensors.append((t, name))
    batch = client.register_tensors("weights", tensors, timeout=300.0)

    times = []
    for it in range(args.syncs):
        t0 = time.perf_counter()
        if trainer:
            batch.transfer("send", blocking=True, timeout=300.0)
        else:
            while not batch.query_transfer_signal(timeout=60.0):
                time.sleep(0.002)
            batch.transfer("recv", blocking=True, timeout=300.0)
        times.append((time.perf_counter() - t0) * 1e3)
    bad = 0
    if not trainer:
        for (k, spec, sp, tp, name), (t, _) in zip(entries, tensors):
            full = full_tensor_for(spec, k, 2, torch.float32, dev).to(src_dtype).to(dst_dtype)
            shape, off = local_shape_and_offset(spec.shape, tmesh, tp, agent_rank)
            if not torch.equal(t, full[tuple(slice(o, o + s) for o, s in zip(off, shape))]):
                bad += 1
    dev_ms = client.state.get(f"batch:weights/state:last_{'send_device' if trainer else 'recv'}_ms")
    print(json.dumps({"role": args.role, "rank": rank, "agent_rank": agent_rank, "syncs": args.syncs,
                      "ms_per_sync_host": [round(x, 2) for x in times], "agent_ms_last": dev_ms.decode() if dev_ms else None,
                      "mismatching_tensors": bad, "golden_match": bad == 0}), flush=True)
    batch.close()
    client.close()
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
