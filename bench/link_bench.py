#!/usr/bin/env python
"""NVLink peak and per-message-class benchmark: one producer GPU stores into one consumer GPU.

Run on 2 GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29530 \
        bench/link_bench.py --mb 1024 --iters 20

Rank 0 is the producer, rank 1 the consumer; the consumer's buffer is opened by the producer as a peer pointer
(CUDA IPC), exactly as the executor does.  Engines compared on the same bytes:

  ce            copy engine (`cudaMemcpyAsync` device-to-device onto the peer mapping): the DMA reference
  ldst:C:T      `m2n_fast_kernel` (SM-issued 16-byte loads and peer stores), C CTAs per SM, T KiB tiles
  bulk          `m2n_bulk_kernel` (TMA bulk loads from local memory, plain bulk stores to the peer address)
  dma:graph     the table's copy-engine lowering: one CUDA graph of independent memcpy nodes
  dma:streams:K the same copies as asynchronous copies dealt over K side streams

Message classes (the shapes of a Llama-3-8B FSDP -> TP sync):

  contig        one contiguous run of --mb MiB                               (embeddings)
  chunks28m     the same bytes as separate 28 MiB runs                        (gate/up shards)
  rows2k        2 KiB source runs at 8 KiB pitch -> contiguous destination   (o_proj)
  rows7k        7 KiB source runs at 28 KiB pitch -> contiguous destination  (down_proj)
  norm2k        many separate 2 KiB messages                                 (norm shards)

Every copy-kernel launch ends with the system-scope fence and a release store to a flag in the consumer's
memory, so the timed interval covers delivery, not just issue.  Timing: CUDA events on the producer's stream,
median of --iters after warm-up; buffers exceed L2.  One JSON line per (class, engine).
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

from etha_b200.ops import CopyTable, SliceRef  # noqa: E402
from etha_b200.ops import lib as L  # noqa: E402
from etha_b200.parallel.peer import PeerMemory  # noqa: E402

LINK_NOMINAL = 900e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--classes", default="contig,chunks28m,rows2k,rows7k,norm2k")
    ap.add_argument("--engines", default="ce,ldst:2:64,bulk,dma:graph,dma:streams:8")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if world != 2:
        raise SystemExit("link_bench runs on exactly 2 ranks (producer, consumer)")
    peer = PeerMemory(dev)
    lib = L.cuda_lib()
    nbytes = args.mb << 20
    # both ranks allocate; only the consumer's buffer and flag are written remotely
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    flag = torch.zeros(4, dtype=torch.int32, device=dev)
    if rank == 0:
        buf.copy_(torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev))
    descs = [None, None]
    dist.all_gather_object(descs, {"buf": peer.describe(buf), "flag": peer.describe(flag)})
    results = []
    if rank == 0:
        dst = peer.slice_ref(descs[1]["buf"])
        dflag = peer.slice_ref(descs[1]["flag"])
        signals = torch.tensor([dflag.ptr], dtype=torch.int64, device=dev)
        src_ref = SliceRef.of(buf)
        stream = torch.cuda.current_stream()

        def table_for(cls: str, tile_kb: int, dma: str | None = None, dma_streams: int = 8) -> tuple[CopyTable, int]:
            t = CopyTable(dev, tile_bytes=tile_kb * 1024, dma_min_bytes=0 if dma else None, dma_mode=dma or "graph",
                          dma_streams=dma_streams)
            _add = t.add
            t.add = lambda *a, **k: _add(*a, dma_ok=bool(dma), **k)
            bf = torch.bfloat16
            if cls == "chunks28m":
                step = 28 << 20
                n = nbytes // step
                for k in range(n):
                    t.add((step // 2,), [SliceRef(src_ref.ptr + k * step, (1,), bf, src_ref.lo, src_ref.hi)],
                          [SliceRef(dst.ptr + k * step, (1,), bf, dst.lo, dst.hi)])
                return t.finalize(), n * step
            if cls == "contig":
                t.add((nbytes // 2,), [SliceRef(src_ref.ptr, (1,), bf, src_ref.lo, src_ref.hi)],
                      [SliceRef(dst.ptr, (1,), bf, dst.lo, dst.hi)])
                return t.finalize(), nbytes
            if cls in ("rows2k", "rows7k"):
                run = 1024 if cls == "rows2k" else 3584  # elements per run; the pitch is four runs
                rows = nbytes // 2 // (4 * run)
                # column block 1 of a [rows, 4*run] matrix -> contiguous [rows, run]
                t.add((rows, run), [SliceRef(src_ref.ptr + 2 * run, (4 * run, 1), bf, src_ref.lo, src_ref.hi)],
                      [SliceRef(dst.ptr, (run, 1), bf, dst.lo, dst.hi)])
                return t.finalize(), rows * run * 2
            if cls == "norm2k":
                n = min(4096, nbytes // 4096)
                for k in range(n):  # 2 KiB messages, sources and destinations 4 KiB apart
                    t.add((1024,), [SliceRef(src_ref.ptr + 4096 * k, (1,), bf, src_ref.lo, src_ref.hi)],
                          [SliceRef(dst.ptr + 4096 * k, (1,), bf, dst.lo, dst.hi)])
                return t.finalize(), n * 2048
            raise ValueError(cls)

        def timed(fn) -> float:
            for _ in range(args.warmup):
                fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ts.sort()
            return ts[len(ts) // 2]

        epoch = [0]
        for cls in args.classes.split(","):
            for eng in args.engines.split(","):
                if eng == "ce":
                    if cls != "contig":
                        continue
                    ms = timed(lambda: L.check(lib.etha_copy_engine_d2d(dst.ptr, src_ref.ptr, nbytes, stream.cuda_stream), "ce copy"))
                    moved = nbytes
                else:
                    parts = eng.split(":")
                    bulk = parts[0] == "bulk"
                    if parts[0] == "dma":
                        ctas, tile_kb = 2, 64
                        table, moved = table_for(cls, 64, dma=parts[1], dma_streams=int(parts[2]) if len(parts) > 2 else 8)
                    else:
                        ctas = int(parts[1]) if len(parts) > 1 else 2
                        tile_kb = int(parts[2]) if len(parts) > 2 else 64
                        table, moved = table_for(cls, tile_kb)

                    def go():
                        epoch[0] += 1
                        table.launch(stream, signals, epoch[0], ctas_per_sm=ctas, bulk=bulk)

                    ms = timed(go)
                    if table.error_word():
                        raise RuntimeError(f"{cls}/{eng}: kernel error word {table.error_word()}")
                gbs = moved / ms / 1e6
                results.append({"class": cls, "engine": eng, "MiB": round(moved / 2**20, 1), "ms_median": round(ms, 4),
                                "GBps": round(gbs, 1), "frac_of_900": round(gbs * 1e9 / LINK_NOMINAL, 3)})
                print(json.dumps(results[-1]), flush=True)
        # last of all, one more contiguous copy with the last copy-kernel engine, checked by the consumer below
        kernels = [e for e in args.engines.split(",") if e != "ce" and not e.startswith("dma")]
        if kernels:
            table, _ = table_for("contig", 64)
            epoch[0] += 1
            table.launch(stream, signals, epoch[0], bulk=kernels[-1].startswith("bulk"))
            torch.cuda.synchronize()
    dist.barrier()
    sums = [None, None]
    dist.all_gather_object(sums, int(buf.view(torch.int64).sum().item()))
    if rank == 0:
        ok = sums[0] == sums[1]
        print(json.dumps({"summary": "link_bench", "final_copy_checksum_equal": ok}), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump({"summary": "link_bench", "final_copy_checksum_equal": ok, "results": results}, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
