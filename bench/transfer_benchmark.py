#!/usr/bin/env python
"""Transfer benchmark over the configurations of the study (counterpart of the reference's
bench/transfer_benchmark.py: layouts x sizes, effective throughput = bytes the target ranks must hold / time).

Run on N GPUs of one node (N=1: both roles on one GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29520 \
        bench/transfer_benchmark.py --config single --nvls 1

configs
  single   one bf16 [rows, 4096] tensor, sizes 1 MiB .. --max-mb, layouts Shard(0)->Shard(1), Shard(0)->Replicate,
           Replicate->Shard(0); producer mesh = first half of the ranks, consumer mesh = second half
  llama    Llama-3-8B, FSDP Shard(0) -> TP (same as bench.py)
  qwen2-partial   Qwen2-7B shapes, source mesh (2, N/4) with (Partial, Shard(0)) -> N/2 consumers; norms and embeddings
           Replicate (fused fp32 reduce + fan-out, NVLS when --nvls 1), linears TP
  mixtral  Mixtral-8x7B shapes, expert-parallel Shard(0) over stacked experts -> TP

Every number is device-timed with CUDA events on each rank, the maximum over ranks is reported, inputs exceed L2
for all but the smallest sizes (the size is printed), and each line carries the fraction of the NVLink roofline:
bytes the busiest GPU must send or receive / link bandwidth: first against the nominal 900 GB/s per direction, then
against the copy-engine peak recorded by `bench/link_bench.py` in `bench/link_peak.json`.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard  # noqa: E402

from bench import init_dist, max_over_ranks  # noqa: E402
from etha_b200.models import ModelSpec, TensorSpec, fsdp_layout, llama3_8b, mixtral_8x7b, qwen2_7b, vllm_tp_layout  # noqa: E402
from etha_b200.models.sync import WeightSync  # noqa: E402

LINK_NOMINAL, HBM_COPY = 900e9, 6535e9
with open(os.path.join(ROOT, "bench", "link_peak.json")) as _f:
    LINK_MEASURED = json.load(_f)["copy_engine_GBps"] * 1e9  # cudaMemcpyAsync onto a peer mapping, 1 GiB
_CASE = [0]  # every rank runs the cases in the same order, so the counter names the rendezvous sockets


def run_case(name, model, smesh, tmesh, s_rule, t_rule, args, rank, world, exchange, busiest_bytes, partial=False):
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = WeightSync(model, rank, list(range(world)), dev, smesh, tmesh, s_rule, t_rule, exchange=exchange,
                    nvls=bool(args.nvls) and world > 1, nvls_tag=f"tb{os.environ.get('MASTER_PORT', '0')}_{_CASE[0]}",
                    dma_min_bytes=(1 << 20) if args.engine == "dma-graph" else None, dma_fraction=0.7).build()
    _CASE[0] += 1
    ready = torch.zeros(1, device=dev)

    def step():
        if world > 1:
            dist.all_reduce(ready)
        ws.sync(timeout_s=20.0, bulk=(world == 1))

    try:
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        ws.check()
        bad = int(max_over_ranks(float(ws.verify() if args.verify else 0), world))
        ws.rescale_sources(0.5)  # the check after the timed loop can only pass if the timed transfers delivered the data
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        from etha_b200.utils.profiling import ProfilingSpec, maybe_enable_profiling

        spec = ProfilingSpec(enable_profiling=bool(args.profile), dump_folder=os.path.join(os.getcwd(), "profiling_traces"),
                             save_traces_folder=name.replace(' ', '_').replace('>', ''),
                             profile_freq=args.steps, warmup_steps=1, active_steps=max(args.steps - 2, 1))
        with maybe_enable_profiling(spec, rank=rank) as prof:
            e0.record()
            for _ in range(args.steps):
                step()
                if prof is not None:
                    prof.step()
            e1.record()
            torch.cuda.synchronize()
        ws.check()
        ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps
        bad_after = int(max_over_ranks(float(ws.verify() if args.verify else 0), world))
        mc = int(max_over_ranks(float(ws.batch.multicast_ops), world))
    finally:
        ws.close()
    if rank == 0:
        roof = busiest_bytes / (LINK_MEASURED if world > 1 else HBM_COPY / 2)
        print(json.dumps({
            "case": name, "n_gpus": world, "payload_MB": round(ws.payload_bytes / 2**20, 1), "ms": round(ms, 4),
            "GBps": round(ws.payload_bytes / ms / 1e6, 1), "roofline_ms_measured_link": round(roof * 1e3, 4),
            "frac_of_roofline_measured": round(roof * 1e3 / ms, 3),
            "frac_of_roofline_nominal": round(busiest_bytes / LINK_NOMINAL * 1e3 / ms, 3) if world > 1 else None,
            "multicast_ops": mc, "nvls": bool(args.nvls) and world > 1, "mismatching_tensors": bad if args.verify else None,
            "verified_after_timed_region": (bad_after == 0) if args.verify else None, "engine": args.engine,
            "under_profiler_not_a_benchmark_number": bool(args.profile),
        }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="single", choices=["single", "llama", "qwen2-partial", "mixtral"])
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--min-mb", type=int, default=1)
    ap.add_argument("--nvls", type=int, default=0)
    ap.add_argument("--verify", type=int, default=1)
    ap.add_argument("--layouts", default="S0->S1,S0->R,R->S0", help="comma-separated subset for --config single")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (0: full model)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: the unmodified reference's chunk / bucket / gather-broadcast methods (--config single)")
    ap.add_argument("--profile", type=int, default=0, help="1: wrap the timed steps in torch.profiler and write chrome traces")
    ap.add_argument("--engine", default="kernel", choices=["kernel", "dma-graph"])
    args = ap.parse_args()
    if args.impl == "reference":
        if args.config != "single":
            raise SystemExit("--impl reference covers --config single here; the model configurations run through bench.py --impl reference")
        from baseline.reference_arm import REF_DIR
        from baseline.reference_run import run_single

        run_single(args, REF_DIR)
        return
    rank, world, _ = init_dist(args.gpus)

    def exchange(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    half = max(world // 2, 1)
    smesh = torch.arange(half) if world > 1 else torch.tensor([0])
    tmesh = torch.arange(half, world) if world > 1 else torch.tensor([0])
    k = half

    def cut(model):
        if args.layers:
            keep = [t for t in model.tensors if ".layers." not in t.name or int(t.name.split(".layers.")[1].split(".")[0]) < args.layers]
            return ModelSpec(model.name + f"-{args.layers}L", keep)
        return model

    if args.config == "single":
        layouts = {
            "S0->S1": ((Shard(0),), (Shard(1),)),
            "S0->R": ((Shard(0),), (Replicate(),)),
            "R->S0": ((Replicate(),), (Shard(0),)),
        }
        mb = args.min_mb
        while mb <= args.max_mb:
            rows = mb * 2**20 // (4096 * 2)
            rows = max(rows // (8 * k) * (8 * k), 8 * k)
            nbytes = rows * 4096 * 2
            for lname, (sp, tp) in layouts.items():
                if lname not in args.layouts.split(","):
                    continue
                model = ModelSpec("one", [TensorSpec("w", (rows, 4096), "column")])
                # busiest GPU: S0->S1 and R->S0 move B/k per GPU; S0->R delivers B to every consumer
                busiest = nbytes if lname == "S0->R" else nbytes / k
                if world == 1:
                    busiest = nbytes
                if lname == "S0->R" and args.nvls and world > 1:
                    busiest = nbytes  # ingress of a consumer is still B; egress of a producer drops to B/k
                run_case(f"{lname} {mb}MiB", model, smesh, tmesh, lambda t, sp=sp: sp, lambda t, tp=tp: tp, args, rank, world,
                         exchange, busiest)
            mb *= 4
    elif args.config == "llama":
        m = cut(llama3_8b())
        run_case(m.name, m, smesh, tmesh, fsdp_layout(), vllm_tp_layout(), args, rank, world, exchange, m.numel * 2 / k)
    elif args.config == "mixtral":
        m = cut(mixtral_8x7b())
        run_case(m.name, m, smesh, tmesh, fsdp_layout(), vllm_tp_layout(), args, rank, world, exchange, m.numel * 2 / k)
    else:
        if world < 4:
            raise SystemExit("qwen2-partial needs at least 4 GPUs (2 x N/4 producers, N/2 consumers)")
        m = cut(qwen2_7b())
        smesh2 = torch.arange(half).view(2, half // 2)
        tp_rule = vllm_tp_layout()

        def t_rule(t):
            return (Replicate(),) if t.kind in ("norm", "vocab") else tp_rule(t)

        rep_bytes = sum(2 * torch.Size(t.shape).numel() for t in m.tensors if t.kind in ("norm", "vocab"))
        run_case(m.name + " (Partial, Shard(0)) -> TP/Replicate", m, smesh2, tmesh, lambda t: (Partial(), Shard(0)), t_rule, args,
                 rank, world, exchange, (m.numel * 2 - rep_bytes) / k + rep_bytes)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
