"""Profiling hooks: NVTX ranges, a torch.profiler harness and memory snapshots.

Counterpart of the reference's bench/utils.py:36-123 (`ProfilingSpec`, `maybe_enable_profiling`,
`dump_memory_snapshot`).  Ranges cost nothing unless a profiler is attached; NVTX goes through
`torch.cuda.nvtx` when a CUDA build is present and is a no-op otherwise.
"""

from __future__ import annotations

import contextlib
import os
import pickle
from dataclasses import dataclass

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range + torch.profiler record_function around a block (plan / launch / wait phases)."""
    pushed = False
    if torch.cuda.is_available():
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:
            pushed = False
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


@dataclass
class ProfilingSpec:
    enable_profiling: bool = False
    dump_folder: str = "./profiling"
    save_traces_folder: str = "traces"
    profile_freq: int = 10
    warmup_steps: int = 3
    active_steps: int = 1
    enable_memory_snapshot: bool = False


@contextlib.contextmanager
def maybe_enable_profiling(spec: ProfilingSpec, global_step: int = 0, rank: int = 0):
    """Yields a torch profiler (call `.step()` once per iteration) or None when profiling is off.
    One chrome trace per rank is written to `{dump_folder}/{save_traces_folder}/rank{rank}_step{N}.json`."""
    if not spec.enable_profiling:
        yield None
        return
    trace_dir = os.path.join(spec.dump_folder, spec.save_traces_folder)
    os.makedirs(trace_dir, exist_ok=True)
    wait = max(spec.profile_freq - spec.warmup_steps - spec.active_steps, 0)

    def on_ready(prof):
        prof.export_chrome_trace(os.path.join(trace_dir, f"rank{rank}_step{prof.step_num}.json"))

    activities = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        activities.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(
        activities=activities,
        schedule=torch.profiler.schedule(wait=wait, warmup=spec.warmup_steps, active=spec.active_steps),
        on_trace_ready=on_ready,
        record_shapes=True,
        with_stack=True,
        profile_memory=True,
    ) as prof:
        prof.step_num = global_step
        yield prof


def start_memory_history(max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def dump_memory_snapshot(folder: str, step: int, rank: int = 0) -> str | None:
    """Pickle of the CUDA caching-allocator snapshot (viewable with pytorch.org/memory_viz)."""
    if not torch.cuda.is_available():
        return None
    os.makedirs(folder, exist_ok=True)
    path = os.path.join(folder, f"rank{rank}_step{step}_memory_snapshot.pickle")
    with open(path, "wb") as f:
        pickle.dump(torch.cuda.memory._snapshot(), f)
    return path
