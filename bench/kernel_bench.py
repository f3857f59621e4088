#!/usr/bin/env python
"""Single-GPU micro-benchmark of the copy-table kernels (device-local source and destination).

Cases: `copy` (contiguous), `rows` (Shard(0) shard cut into 4 column blocks, the o_proj/down_proj
pattern), `cvt` (fp32 -> bf16), `reduce2` / `reduce4` (Partial collapse of 2 / 4 bf16 sources),
`fanout4` (one read, four destinations).  Buffers are larger than L2; timing uses CUDA events around
each launch after warm-up.  Prints one JSON line per case with achieved bytes/s against the measured
copy bandwidth in MEASURED_PEAKS.json (fallback 6.65 TB/s).

    python bench/kernel_bench.py --case all --mb 1024 --iters 10
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from etha_b200.ops import CopyTable, SliceRef  # noqa: E402


def peak_gbs() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def build_case(case: str, mb: int, dev, tile_kb: int, streaming: bool = True):
    n_rows = mb * 1024 * 1024 // (4096 * 2)
    t = CopyTable(dev, tile_bytes=tile_kb * 1024)
    t.stream_typed = streaming
    keep = []
    if case == "copy":
        src = torch.randn(n_rows, 4096, device=dev).to(torch.bfloat16)
        dst = torch.empty_like(src)
        t.add_copy(src, dst)
        traffic = 2 * src.numel() * 2
        check = lambda: torch.equal(src, dst)
    elif case == "rows":
        src = torch.randn(n_rows, 4096, device=dev).to(torch.bfloat16)
        dsts = [torch.empty(n_rows, 1024, dtype=torch.bfloat16, device=dev) for _ in range(4)]
        for j in range(4):
            t.add_copy(src[:, 1024 * j : 1024 * (j + 1)], dsts[j])
        traffic = 2 * src.numel() * 2
        check = lambda: all(torch.equal(dsts[j], src[:, 1024 * j : 1024 * (j + 1)]) for j in range(4))
    elif case == "cvt":
        src = torch.randn(n_rows, 4096, device=dev)
        dst = torch.empty(n_rows, 4096, dtype=torch.bfloat16, device=dev)
        t.add_copy(src, dst)
        traffic = src.numel() * 6
        check = lambda: torch.equal(dst, src.to(torch.bfloat16))
    elif case in ("reduce2", "reduce4"):
        k = int(case[-1])
        srcs = [torch.randn(n_rows, 4096, device=dev).to(torch.bfloat16) for _ in range(k)]
        dst = torch.empty_like(srcs[0])
        t.add_reduce(srcs, dst, (k,), ("sum",))
        traffic = (k + 1) * dst.numel() * 2
        def check():
            acc = srcs[0].float()
            for s in srcs[1:]:
                acc = acc + s.float()
            return torch.equal(dst, acc.to(torch.bfloat16))
    elif case == "fanout4":
        src = torch.randn(n_rows, 4096, device=dev).to(torch.bfloat16)
        dsts = [torch.empty_like(src) for _ in range(4)]
        t.add(tuple(src.shape), [SliceRef.of(src)], [SliceRef.of(d) for d in dsts])
        keep += [src] + dsts
        traffic = 5 * src.numel() * 2
        check = lambda: all(torch.equal(d, src) for d in dsts)
    else:
        raise ValueError(case)
    t.finalize()
    return t, traffic, check, keep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--mb", type=int, default=1024, help="size of the source tensor in MiB (bf16 [N, 4096])")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tile-kb", type=int, default=64)
    ap.add_argument("--ctas-per-sm", type=int, default=2)
    ap.add_argument("--bulk", type=int, default=0)
    ap.add_argument("--streaming", type=int, default=1, help="0: typed ops stay in the general kernel")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, how = peak_gbs()
    cases = ["copy", "rows", "cvt", "reduce2", "reduce4", "fanout4"] if args.case == "all" else [args.case]
    for case in cases:
        table, traffic, check, keep = build_case(case, args.mb, dev, args.tile_kb, bool(args.streaming))
        for _ in range(args.warmup):
            table.launch(ctas_per_sm=args.ctas_per_sm, bulk=bool(args.bulk))
        torch.cuda.synchronize()
        ok = bool(check())
        times = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            table.launch(ctas_per_sm=args.ctas_per_sm, bulk=bool(args.bulk))
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        med = times[len(times) // 2]
        gbs = traffic / (med * 1e-3) / 1e9
        print(json.dumps({
            "case": case, "mb": args.mb, "bulk": args.bulk, "ms_median": round(med, 4), "ms_min": round(times[0], 4),
            "dram_traffic_GBps": round(gbs, 1), f"frac_of_{how}_copy_bw": round(gbs / peak, 3), "correct": ok,
            "tile_kb": args.tile_kb, "ctas_per_sm": args.ctas_per_sm,
            "streaming_ops": getattr(table, "n_typed_ops", 0),
        }), flush=True)
        del table, keep


if __name__ == "__main__":
    main()
