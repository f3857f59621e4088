"""The profiling hooks are live: ranges around plan / table build / launch show up in a chrome trace."""

import glob
import json
import os

import torch
from torch.distributed.tensor.placement_types import Shard

from etha_b200.comm.planner import plan_m2m
from etha_b200.utils.profiling import ProfilingSpec, maybe_enable_profiling, nvtx_range


def test_chrome_trace_contains_the_named_ranges(tmp_path):
    spec = ProfilingSpec(enable_profiling=True, dump_folder=str(tmp_path), save_traces_folder="traces/plan",
                         profile_freq=3, warmup_steps=1, active_steps=2)
    with maybe_enable_profiling(spec, rank=0) as prof:
        assert prof is not None
        for _ in range(3):
            with nvtx_range("etha.plan"):
                plan_m2m(torch.arange(4), (Shard(0),), torch.arange(4, 8), (Shard(1),))
            prof.step()
    files = glob.glob(os.path.join(str(tmp_path), "traces", "plan", "rank0_step*.json"))
    assert files, "no chrome trace was written"
    names = {e.get("name") for e in json.load(open(files[0]))["traceEvents"]}
    assert "etha.plan" in names


def test_profiling_off_yields_none(tmp_path):
    with maybe_enable_profiling(ProfilingSpec(enable_profiling=False, dump_folder=str(tmp_path))) as prof:
        assert prof is None
    assert not os.listdir(tmp_path)
