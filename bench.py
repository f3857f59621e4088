#!/usr/bin/env python
"""Headline benchmark: full-model weight sync, trainer layout -> inference layout, on N GPUs of one node.

Metric: weight-sync GB/s (bytes the consumer ranks must end up holding / device time, max over ranks)
and sync latency per step, for Llama-3-8B bf16, FSDP `Shard(0)` over the first N/2 GPUs -> vLLM-style
TP over the other N/2 (N=1: producer and consumer share the GPU).  The total work is fixed as N grows
(strong scaling).  `--impl reference` runs the unmodified reference (its NCCL `bucket_comm`) from
`baseline/_ref` on the same configuration.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 20 --warmup 3
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "weight_sync_GBps"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "qwen2-7b", "mixtral-8x7b", "qwen3-0.6b", "tiny"])
    p.add_argument("--layout", default="fsdp-tp", choices=["fsdp-tp", "partial2x2-tp"],
                   help="fsdp-tp: Shard(0) over N/2 producers (stacked experts: expert parallel) -> TP over N/2 consumers; "
                        "partial2x2-tp: source mesh (2, N/4) with (Partial, Shard(0)) -> N/2 consumers, norms and "
                        "embeddings Replicate, linears TP (needs N >= 4)")
    p.add_argument("--nvls", type=int, default=0, help="1: Replicate targets live in a multicast-bound arena (multimem.st fan-out)")
    p.add_argument("--source-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--bulk", type=int, default=-1, help="1: TMA bulk kernel for the fast class, 0: LD/ST kernel, -1: default")
    p.add_argument("--engine", default="kernel", choices=["kernel", "dma-graph", "dma-streams"],
                   help="kernel (default): every copy by the sm_100a kernels; dma-*: the largest remote bit copies run on "
                        "the DMA engines next to the kernels (opt-in: +3.7 %% on 1+1 GPUs, but a 4+4 GPU run with it did "
                        "not finish within its time limit, so it is not the default)")
    p.add_argument("--dma-min-kb", type=int, default=1024)
    p.add_argument("--dma-fraction", type=float, default=0.7, help="share of the delivered bytes given to the DMA engines")
    p.add_argument("--ctas-per-sm", type=int, default=2)
    p.add_argument("--tile-kb", type=int, default=64)
    p.add_argument("--bucket-mb", type=int, default=256, help="reference arm: bucket size in MiB (0 = one message per chunk)")
    p.add_argument("--no-verify", action="store_true")
    p.add_argument("--bus", type=int, default=1, help="also time the sync through agents + TensorBusClient (0 to skip)")
    return p.parse_args()


def model_of(name: str):
    from etha_b200 import models

    return {
        "llama3-8b": models.llama3_8b,
        "qwen2-7b": models.qwen2_7b,
        "mixtral-8x7b": models.mixtral_8x7b,
        "qwen3-0.6b": models.qwen3_0p6b,
        "tiny": models.tiny_llama,
    }[name]()


def init_dist(n: int):
    """Returns (rank, world, gloo_group or None). One process per GPU; NCCL for in-stream barriers."""
    import torch
    import torch.distributed as dist

    if n == 1 and "RANK" not in os.environ:
        torch.cuda.set_device(0)
        return 0, 1, None
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dist.init_process_group("cuda:nccl,cpu:gloo", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, dist.group.WORLD


def max_over_ranks(value: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)  # gloo (cpu tensor)
    return float(t.item())


def meshes_for(n: int):
    import torch

    if n == 1:
        return torch.tensor([0]), torch.tensor([0]), "fsdp1->tp1 (producer and consumer share the GPU)"
    half = n // 2
    return torch.arange(half), torch.arange(half, n), f"fsdp{half}->tp{half}"


def layout_for(args, n: int):
    """(source mesh, target mesh, source rule, target rule, description, bytes the busiest GPU sends or receives)
    of the benchmark's layout; shared by both arms so that they run the same configuration."""
    import torch
    from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

    from etha_b200.models import fsdp_layout, vllm_tp_layout

    model = model_of(args.model)
    if args.layout == "fsdp-tp":
        smesh, tmesh, par = meshes_for(n)
        if "mixtral" in args.model:
            par = par.replace("fsdp", "ep+fsdp")
        k = max(n // 2, 1)
        return smesh, tmesh, fsdp_layout(), vllm_tp_layout(), par, model.numel * 2 / k
    if n < 4 or n % 4:
        raise SystemExit("layout partial2x2-tp needs 4 or 8 GPUs (a 2 x N/4 producer mesh and N/2 consumers)")
    half = n // 2
    smesh, tmesh = torch.arange(half).view(2, half // 2), torch.arange(half, n)
    tp_rule = vllm_tp_layout()

    def t_rule(t):
        return (Replicate(),) if t.kind in ("norm", "vocab", "router") else tp_rule(t)

    rep = sum(2 * torch.Size(t.shape).numel() for t in model.tensors if t.kind in ("norm", "vocab", "router"))
    # every consumer receives its 1/(N/2) of the TP tensors and all of the Replicate ones; the 2 x N/4 producers send
    # the same amount in total, so a consumer's ingress is the bound
    busiest = (model.numel * 2 - rep) / half + rep
    return (smesh, tmesh, lambda t: (Partial(), Shard(0)), t_rule,
            f"(Partial, Shard(0)) on 2x{half // 2} -> tp{half} (norms, embeddings Replicate)", busiest)


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from etha_b200 import ops
    from etha_b200.comm.p2p import PairLayout
    from etha_b200.models.sync import WeightSync
    from etha_b200.ops import table as table_mod
    from etha_b200.utils.clocks import ClockSampler
    from torch.distributed.tensor.placement_types import Replicate

    rank, world, group = init_dist(args.gpus)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = model_of(args.model)
    smesh, tmesh, s_rule, t_rule, par, busiest_bytes = layout_for(args, world)

    def exchange(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    # a version stamp travels with the weights: the producer uploads it from pinned host memory each
    # step, every consumer reads it back after the sync (this is the end-to-end check of a step)
    is_src = rank in smesh.reshape(-1).tolist()
    is_dst = rank in tmesh.reshape(-1).tolist()
    stamp_src = torch.zeros(16, dtype=torch.int64, device=dev) if is_src else None
    stamp_dst = torch.zeros(16, dtype=torch.int64, device=dev) if is_dst else None
    stamp_layout = PairLayout(smesh, (Replicate(),) * smesh.dim(), tmesh, (Replicate(),))
    ws = WeightSync(
        model, rank, list(range(world)), dev, smesh, tmesh, s_rule, t_rule, exchange=exchange,
        source_dtype=getattr(torch, args.source_dtype), nvls=bool(args.nvls) and world > 1,
        nvls_tag=f"bench{os.environ.get('MASTER_PORT', '0')}",
        extra=[(stamp_layout, stamp_src, stamp_dst)], tile_bytes=args.tile_kb * 1024,
        dma_min_bytes=args.dma_min_kb * 1024 if args.engine != "kernel" else None,
        dma_mode="graph" if args.engine == "dma-graph" else "streams", dma_fraction=args.dma_fraction,
    ).build()
    # TMA bulk kernel by default when producer and consumer share the GPU (it only serves local destinations)
    bulk = bool(args.bulk) if args.bulk >= 0 else (world == 1)
    kw = dict(ctas_per_sm=args.ctas_per_sm, bulk=bulk)
    stream = torch.cuda.current_stream()
    ready = torch.zeros(1, device=dev)

    def step():
        # in-stream readiness barrier: no producer starts before every consumer is in the step
        if world > 1:
            dist.all_reduce(ready)
        ws.sync(stream, timeout_s=20.0, **kw)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    ws.check()
    bad = 0 if args.no_verify else ws.verify()
    bad = int(max_over_ranks(float(bad), world))
    # every source value changes now (x 1/2, exact): the check after the timed loop can only pass if the timed
    # transfers themselves delivered the data
    ws.rescale_sources(0.5)

    # ---- device-timed region: K steps, events on the launching stream ---------------------------
    launches0 = table_mod.LAUNCH_COUNT[0] + ops.FLAG_LAUNCH_COUNT[0]
    sampler = ClockSampler(dev.index).start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ws.check()
    launches = table_mod.LAUNCH_COUNT[0] + ops.FLAG_LAUNCH_COUNT[0] - launches0
    if world > 1:  # kernels of this framework launched inside the timed region, summed over ranks
        t = torch.tensor([float(launches)], dtype=torch.float64)
        dist.all_reduce(t)
        launches = int(t.item())
    bad_after = 0 if args.no_verify else ws.verify()
    bad_after = int(max_over_ranks(float(bad_after), world))
    ms_total = max_over_ranks(e0.elapsed_time(e1), world)
    ms_step = ms_total / args.steps
    gbps = ws.payload_bytes / (ms_step * 1e-3) / 1e9

    # ---- the same K steps with every copy in the kernels (no DMA engine), for the record ---------------------
    kernels_only = None
    if ws.batch.table.n_dma_copies or int(max_over_ranks(float(ws.batch.table.n_dma_copies), world)):
        kw_k = dict(kw, dma=False)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(args.steps):
            if world > 1:
                dist.all_reduce(ready)
            ws.sync(stream, timeout_s=20.0, **kw_k)
        k1.record()
        torch.cuda.synchronize()
        ws.check()
        k_ms = max_over_ranks(k0.elapsed_time(k1), world) / args.steps
        kernels_only = {"ms_per_step": round(k_ms, 4), "value": round(ws.payload_bytes / (k_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                        "what": "same steps with dma=False: every copy issued by the sm_100a kernels"}

    # ---- end to end: pinned-host stamp upload, sync, stamp + status read back, host-visible completion ----
    pin_in = torch.zeros(16, dtype=torch.int64).pin_memory()
    pin_out = torch.zeros(16, dtype=torch.int64).pin_memory()
    pin_status = torch.zeros(2, dtype=torch.int32).pin_memory()
    h2d = pin_in.numel() * 8 if is_src else 0
    d2h = (pin_out.numel() * 8 + 8) if is_dst else 0
    stamp_errors = 0

    def e2e_step(k: int):
        nonlocal stamp_errors
        if is_src:
            pin_in.fill_(k)
            stamp_src.copy_(pin_in, non_blocking=True)
        step()
        if is_dst:
            pin_out.copy_(stamp_dst, non_blocking=True)
            pin_status.copy_(ws.batch._status, non_blocking=True)
        torch.cuda.synchronize()
        if is_dst and (int(pin_out[0]) != k or int(pin_status[0]) != 0):
            stamp_errors += 1

    for k in range(2):
        e2e_step(1000 + k)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for k in range(args.steps):
        e2e_step(k + 1)
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1), world) / args.steps
    stamp_errors = int(max_over_ranks(float(stamp_errors), world))
    e2e_gbps = ws.payload_bytes / (e2e_ms * 1e-3) / 1e9

    # ---- the same sync through the tensor bus: agents as separate processes, workers use TensorBusClient ----------
    bus = None
    if args.bus:
        bus = run_bus_e2e(args, rank, world, dev, ws, smesh, tmesh, stamp_src, stamp_dst, is_src, is_dst)

    link_nominal, hbm_copy = 900e9, 6535e9
    if world > 1:
        roof_ms = busiest_bytes / link_nominal * 1e3
        roof_what = "bytes the busiest GPU must send or receive / 900 GB/s (NVLink 5 nominal, one direction)"
    else:
        roof_ms = 2 * busiest_bytes / hbm_copy * 1e3
        roof_what = "bytes read + written / measured HBM copy bandwidth (6535 GB/s)"
    multicast_ops = int(max_over_ranks(float(ws.batch.multicast_ops), world))
    ws.close()
    result = {
        "metric": METRIC,
        "value": round(gbps, 2),
        "unit": "GB/s (1e9 bytes held by consumers / device time, max over ranks)",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random-init weights (randn*0.02, seeded per tensor), no checkpoint",
        "impl": "ours",
        "config": {
            "model": args.model,
            "global_batch": None,
            "seq_len": None,
            "parallelism": par,
            "layout": args.layout,
            "source_dtype": args.source_dtype,
            "tensors": len(model.tensors),
            "payload_bytes": ws.payload_bytes,
            "roofline_ms": round(roof_ms, 4),
            "roofline": roof_what,
            "frac_of_roofline": round(roof_ms / ms_step, 3),
            "nvls_multicast_ops": multicast_ops,
            "l2_policy": f"inputs larger than L2 ({ws.payload_bytes / 1e9:.1f} GB delivered per sync vs 126 MB)",
            "executor": "p2p copy table, " + ("TMA bulk kernel" if bulk else "LD/ST kernel")
                        + (f" + {ws.batch.table.n_dma_copies} DMA-engine copies ({args.engine})" if ws.batch.table.n_dma_copies else ""),
            "dma_copies_per_step_this_rank": ws.batch.table.n_dma_copies,
            "verified_bit_exact": (bad == 0) if not args.no_verify else None,
            "mismatching_tensors": bad,
            "verified_after_timed_region": (bad_after == 0) if not args.no_verify else None,
            "verification": "bit-exact after warm-up; then every source is halved on the device and the targets are "
                            "checked again after the timed loop against the halved values",
        },
        "e2e": {
            "value": round(e2e_gbps, 2),
            "unit": "GB/s",
            "ms_per_step": round(e2e_ms, 4),
            "h2d_bytes_per_step": int(max_over_ranks(float(h2d), world)),
            "d2h_bytes_per_step": int(max_over_ranks(float(d2h), world)),
            "what": "per step: version stamp uploaded from pinned host memory, full sync through WeightSync.sync(), "
                    "every consumer reads stamp + wait status back to pinned memory and the host checks them",
            "stamp_errors": stamp_errors,
        },
        "e2e_bus": bus,
        "kernels_only": kernels_only,
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if group is not None:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_bus_e2e(args, rank, world, dev, ws, smesh, tmesh, stamp_src, stamp_dst, is_src, is_dst) -> dict:
    """End to end through the public bus API: one agent process per GPU (two on the single GPU of N=1), this
    process attaches with TensorBusClient, registers the same shards and times transfer("send"|"recv") rounds.
    A failure here never invalidates the numbers above: it is reported in the returned dict."""
    import torch
    import torch.distributed as dist

    from etha_b200.models.bus_sync import BusItem, bus_roundtrip
    from torch.distributed.tensor.placement_types import Replicate

    steps = max(3, min(args.steps, 10))
    pin_in = torch.zeros(16, dtype=torch.int64).pin_memory()
    pin_out = torch.zeros(16, dtype=torch.int64).pin_memory()
    errors = [0]
    stream = torch.cuda.current_stream()

    def on_step(k, phase):
        if phase == "before_send":
            pin_in.fill_(k)
            stamp_src.copy_(pin_in, non_blocking=True)
            stream.synchronize()  # the agent reads the stamp from another process: it must have landed
        else:
            pin_out.copy_(stamp_dst, non_blocking=True)
            stream.synchronize()
            if int(pin_out[0]) != k:
                errors[0] += 1

    def share(obj):
        if world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=0, device=torch.device("cpu"))
        return box[0]

    items = [BusItem(e.source, e.target, tuple(e.layout.source_placements), tuple(e.layout.target_placements)) for e in ws.entries]
    items.append(BusItem(stamp_src, stamp_dst, (Replicate(),) * smesh.dim(), (Replicate(),)))
    src_agents = smesh.reshape(-1).tolist() if world > 1 else [0]
    dst_agents = tmesh.reshape(-1).tolist() if world > 1 else [1]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def stop():
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    out, failure = None, None
    try:
        out = bus_roundtrip(rank, world, dev.index, items, src_agents, dst_agents, steps=steps, warmup=2, share=share,
                            on_step=on_step, timeout=150.0, timer=(e0.record, stop),
                            source_mesh_shape=tuple(smesh.shape), target_mesh_shape=tuple(tmesh.shape))
    except Exception as e:  # reported, not fatal
        failure = f"{type(e).__name__}: {e}"[:300]
    ms = max_over_ranks(out["ms_per_step"] if out else float("inf"), world)
    bad = int(max_over_ranks(float(errors[0]), world))
    if ms == float("inf"):
        return {"unavailable": failure or "another rank failed"}
    return {
        "value": round(ws.payload_bytes / (ms * 1e-3) / 1e9, 2),
        "unit": "GB/s",
        "ms_per_step": round(ms, 4),
        "steps": steps,
        "agent_send_device_ms_last": out.get("agent_send_device_ms_last") if out else None,
        "h2d_bytes_per_step": 128,
        "d2h_bytes_per_step": 128,
        "stamp_errors": bad,
        "what": "TensorBusClient.init_pair/register_tensors once, then per step: stamp H2D from pinned memory, "
                "BatchHandler.transfer('send'|'recv') through command queue + agent + P2P kernels, stamp D2H and check",
    }


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        out = run_reference(args)
    else:
        out = run_ours(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
