import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        n = 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(skip_multi)

    # Order: everything that needs at most one GPU first, then the multi-process multi-GPU integration tests, and the
    # allocation-free entry point last of all, so that a run that stops at the first failure (-x) has already been
    # through the kernels' numerics tests when it reaches the long integration runs.
    late = ["test_nccl_bucket_gpu", "test_nvls_gpu", "test_example_gpu_peer_to_peer", "test_moe_example_gpu", "test_y_bus_nvls_gpu"]

    def rank(item):
        if "test_zz_" in item.nodeid:
            return 100
        if "multigpu" not in item.keywords:
            return 0
        return 1 + next((i for i, name in enumerate(late) if name in item.nodeid), len(late))  # shortest runs first

    items.sort(key=rank)


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture
def master_env(monkeypatch):
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(free_port()))
    yield
