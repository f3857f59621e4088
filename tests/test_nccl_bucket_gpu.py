"""Bucket executor over NCCL on two (or four) GPUs, one child process per GPU."""

import os
import subprocess
import sys

import pytest

from conftest import free_port

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(600)
def test_bucket_comm_over_nccl():
    import torch

    # 1+1 GPUs, or 2+2 when four are present (adds Shard(0)->Shard(1), a BROADCAST to two replicas and a Partial source)
    n = 4 if torch.cuda.device_count() >= 4 else 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "nccl_bucket_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=400)
    out = proc.stdout + proc.stderr
    assert proc.returncode == 0, out[-4000:]
    assert out.count("RESULT PASS") == n, out[-4000:]
