"""NVLS multicast fan-out and fd-shared VMM arenas on two GPUs (child processes, one per GPU)."""

import os
import subprocess
import sys

import pytest

from conftest import free_port

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(600)
def test_multicast_fanout_two_gpus():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "nvls_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    out = proc.stdout + proc.stderr
    if "SKIP: multicast not supported" in out:
        pytest.skip("multicast not supported on this machine")
    assert proc.returncode == 0, out[-4000:]
    assert out.count("RESULT PASS") == 2, out[-4000:]
