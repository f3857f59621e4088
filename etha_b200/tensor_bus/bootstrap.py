"""Worker bootstrap: find the agent of this rank and connect (reference: src/etha/tensor_bus/bootstrap.py:14-135).

Agent rank = `AGENT_RANK`, else `RANK + AGENT_RANK_OFFSET`; default files `/tmp/agent_rank{N}_command.lmdb` and
`/tmp/agent_rank{N}_state.lmdb` (names kept although the files are memory-mapped rings, not LMDB).
"""

from __future__ import annotations

import ctypes
import logging
import os
from collections.abc import Callable
from dataclasses import dataclass

from .client import TensorBusClient

logger = logging.getLogger(__name__)


def setup_ptrace() -> bool:
    """Allow any process of this user to attach (`prctl(PR_SET_PTRACER, ANY)`).

    Needed only when a worker shares expandable-segment (VMM) memory whose file descriptors the agent must
    duplicate; plain `cudaMalloc` allocations travel as IPC handles and need nothing.
    """
    PR_SET_PTRACER = 0x59616D61
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        return libc.prctl(PR_SET_PTRACER, ctypes.c_ulong(-1), 0, 0, 0) == 0
    except OSError:
        return False


@dataclass
class BootstrapInfo:
    agent_rank: int
    global_rank: int
    rank_offset: int | None
    command_queue_path: str
    state_path: str
    method: str  # "direct" (AGENT_RANK) or "offset" (RANK + AGENT_RANK_OFFSET)


def default_paths(agent_rank: int) -> tuple[str, str]:
    return f"/tmp/agent_rank{agent_rank}_command.lmdb", f"/tmp/agent_rank{agent_rank}_state.lmdb"


def bootstrap_client(
    path_naming_fn: Callable[[int], tuple[str, str]] | None = None,
    connection_timeout: float = 30.0,
) -> tuple[TensorBusClient, BootstrapInfo]:
    setup_ptrace()
    global_rank = int(os.environ["RANK"])
    if "AGENT_RANK" in os.environ:
        rank_offset, agent_rank, method = None, int(os.environ["AGENT_RANK"]), "direct"
    else:
        rank_offset = int(os.environ.get("AGENT_RANK_OFFSET", 0))
        agent_rank, method = global_rank + rank_offset, "offset"
    command_queue_path, state_path = (path_naming_fn or default_paths)(agent_rank)
    client = TensorBusClient(
        agent_rank=agent_rank,
        lmdb_command_queue_path=command_queue_path,
        agent_state_lmdb_path=state_path,
        connection_timeout=connection_timeout,
    )
    info = BootstrapInfo(agent_rank, global_rank, rank_offset, command_queue_path, state_path, method)
    logger.info("[Bootstrap] agent_rank=%s (%s)", agent_rank, method)
    return client, info
