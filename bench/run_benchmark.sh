#!/usr/bin/env bash
# Runs the benchmark suite on one 8-GPU node (counterpart of the reference's Slurm launcher bench/run_benchmark.sh,
# which spans two nodes over InfiniBand; this framework's data path is one NVLink domain).
#   bash bench/run_benchmark.sh [GPUS]           # GPUS = 1, 2, 4 or 8 (default 8)
set -euo pipefail
cd "$(dirname "$0")/.."
N="${1:-8}"
PORT="${MASTER_PORT:-29540}"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node ${N} --master-addr 127.0.0.1"
if [ "${N}" = "1" ]; then RUN="python"; fi
launch() { if [ "${N}" = "1" ]; then python "$@"; else ${RUN} --master-port "${PORT}" "$@"; PORT=$((PORT + 1)); fi; }

launch bench.py --gpus "${N}" --impl reference
launch bench.py --gpus "${N}"
launch bench/transfer_benchmark.py --config single --max-mb 4096
if [ "${N}" -ge 2 ]; then
  launch bench/transfer_benchmark.py --config single --max-mb 4096 --impl reference   # chunk, 256 MiB buckets, gather-broadcast
  launch bench.py --gpus "${N}" --model mixtral-8x7b --impl reference
  launch bench.py --gpus "${N}" --model mixtral-8x7b
  launch bench.py --gpus "${N}" --source-dtype float32 --impl reference
  launch bench.py --gpus "${N}" --source-dtype float32
fi
if [ "${N}" -ge 4 ]; then
  launch bench/transfer_benchmark.py --config single --max-mb 1024 --layouts "S0->R" --nvls 1
  launch bench.py --gpus "${N}" --model qwen2-7b --layout partial2x2-tp
  launch bench.py --gpus "${N}" --model qwen2-7b --layout partial2x2-tp --nvls 1
fi
if [ "${N}" = "2" ]; then
  launch bench/link_bench.py --mb 1024 --iters 20
fi
python bench/kernel_bench.py --case all --mb 1024
python bench/kvstore_benchmark.py --iters 1000
