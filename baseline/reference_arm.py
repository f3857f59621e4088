"""`bench.py --impl reference`: the unmodified reference executor on the benchmark's configuration."""

from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def run_reference(args) -> dict:
    if not os.path.isdir(os.path.join(REF_DIR, "etha")):
        if int(os.environ.get("RANK", "0")) == 0:
            return {"impl": "reference", "unavailable": "baseline/_ref/etha is missing: the reference package was not installed"}
        return {}
    from .reference_run import run

    return run(args, REF_DIR)
