"""The multi-process weight-sync example (agents + trainer workers + inference workers as separate processes),
the integration test the reference runs on 8 GPUs (tests/test_distributed_model_transfer.py): here on CPU/gloo
for every run, and on GPUs through CUDA IPC + the peer-to-peer kernels when at least two are present."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAUNCH = os.path.join(ROOT, "examples", "weight_sync", "launch.py")


def _run(*args, timeout=600):
    proc = subprocess.run([sys.executable, LAUNCH, *args], capture_output=True, text=True, timeout=timeout)
    out = proc.stdout + proc.stderr
    assert proc.returncode == 0, out[-4000:]
    assert "all inference ranks verified their shards" in out
    return out


@pytest.mark.timeout(900)
def test_example_cpu_two_plus_two():
    out = _run("--side-size", "2", "--model", "tiny", "--device", "cpu", "--syncs", "2")
    assert out.count('"golden_match": true') == 4


def _side_for_gpus() -> int:
    import torch

    n = torch.cuda.device_count()
    return 4 if n >= 8 else (2 if n >= 4 else 1)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(1800)
@pytest.mark.parametrize("source_dtype", ["float32", "bfloat16"])
def test_example_gpu_peer_to_peer(source_dtype):
    """The reference's integration test (Qwen3-0.6B shapes, 10 transfers, fp32 -> bf16 and same-dtype, one trainer
    group and one inference group behind agents; tests/test_distributed_model_transfer.py:59-157) at the largest
    scale the machine allows: 4+4 GPUs on eight, 2+2 on four, 1+1 (tiny model) on two."""
    side = _side_for_gpus()
    model, syncs = ("qwen3-0.6b", 10) if side >= 2 else ("tiny", 3)
    out = _run("--side-size", str(side), "--model", model, "--syncs", str(syncs), "--source-dtype", source_dtype, timeout=1500)
    assert out.count('"golden_match": true') == 2 * side


@pytest.mark.timeout(900)
def test_moe_example_cpu_hsdp_and_expert_meshes():
    """2-D HSDP trainer mesh + 3-D expert mesh -> 2-D TP / 1-D EP consumers, eight named pairs, fused qkv and gate-up
    tensors registered as views on both sides (guard rows checked), rounds gated on control keys."""
    out = _run("--scenario", "moe", "--trainer-mesh", "2x2", "--inference-mesh", "2x2", "--device", "cpu", "--syncs", "2")
    assert out.count('"golden_match": true') == 8 and out.count('"pairs": 8') == 8


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.timeout(1800)
def test_moe_example_gpu():
    import torch

    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip("the MoE example needs at least 2+2 GPUs")
    mesh = "2x2" if n >= 8 else "1x2"
    out = _run("--scenario", "moe", "--trainer-mesh", mesh, "--inference-mesh", mesh, "--syncs", "3", timeout=1500)
    assert out.count('"golden_match": true') == (8 if n >= 8 else 4)


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_example_two_agents_sharing_one_gpu():
    """Producer and consumer agents (and their workers) all on GPU 0: NCCL cannot run two ranks on one device, the
    peer-to-peer path can; completion then goes through the KV store, never through a device-side spin."""
    out = _run("--side-size", "1", "--model", "tiny", "--syncs", "3", "--share-gpu")
    assert out.count('"golden_match": true') == 2
