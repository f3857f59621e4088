"""In-tree builds of the native libraries (no JIT cache: the `.so` files sit next to this file).

* `libetha_b200_cuda.so` — sm_100a kernels, table packer, CUDA IPC / VMM helpers (nvcc).
* `libetha_b200_host.so` — POSIX semaphores and the shared-memory command queue / state store (g++),
  loadable on machines without a CUDA driver.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")

CUDA_SOURCES = ["m2n_kernels.cu", "m2n_bulk.cu", "m2n_typed.cu", "dma_graph.cu", "table_pack.cpp", "ipc.cu", "vmm_arena.cpp"]
HOST_SOURCES = ["psem.cpp", "shmq.cpp"]
CUDA_LIB = os.path.join(HERE, "libetha_b200_cuda.so")
HOST_LIB = os.path.join(HERE, "libetha_b200_host.so")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]


HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared"]


def _existing(names: list[str]) -> list[str]:
    return [os.path.join(CSRC, n) for n in names if os.path.exists(os.path.join(CSRC, n))]


def _fingerprint(sources: list[str], flags: list[str]) -> str:
    """Hash of everything that determines the binary: sources, headers and flags (file times do not survive copies)."""
    import hashlib

    h = hashlib.sha256(" ".join(flags).encode())
    deps = sorted(sources + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")])
    for path in deps:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target: str, sources: list[str], flags: list[str]) -> bool:
    stamp = target + ".stamp"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _fingerprint(sources, flags)


def _write_stamp(target: str, sources: list[str], flags: list[str]) -> None:
    tmp = target + f".stamp.tmp{os.getpid()}"
    with open(tmp, "w") as f:
        f.write(_fingerprint(sources, flags))
    os.replace(tmp, target + ".stamp")


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build_cuda_lib(force: bool = False, verbose: bool = False) -> str:
    sources = _existing(CUDA_SOURCES)
    if not force and not _stale(CUDA_LIB, sources, NVCC_FLAGS):
        return CUDA_LIB
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libetha_b200_cuda.so")
    tmp = CUDA_LIB + f".tmp{os.getpid()}"
    cmd = [nvcc, *NVCC_FLAGS, "-o", tmp, *sources, "-lrt", "-lpthread"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    _run(cmd)
    os.replace(tmp, CUDA_LIB)
    _write_stamp(CUDA_LIB, sources, NVCC_FLAGS)
    return CUDA_LIB


def build_host_lib(force: bool = False) -> str:
    sources = _existing(HOST_SOURCES)
    if not force and not _stale(HOST_LIB, sources, HOST_FLAGS):
        return HOST_LIB
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    tmp = HOST_LIB + f".tmp{os.getpid()}"
    _run([cxx, *HOST_FLAGS, "-o", tmp, *sources, "-lrt", "-lpthread"])
    os.replace(tmp, HOST_LIB)
    _write_stamp(HOST_LIB, sources, HOST_FLAGS)
    return HOST_LIB


def build_all(force: bool = False) -> None:
    build_host_lib(force)
    build_cuda_lib(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(CUDA_LIB)
    print(HOST_LIB)
