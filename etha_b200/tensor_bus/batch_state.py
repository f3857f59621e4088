"""In-memory state of one registered batch on an agent (reference: src/etha/tensor_bus/batch_state.py:17-43)."""

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass(kw_only=True)
class BatchState:
    batch_id: str
    pair_names: list[str]
    local_leader: int | None = None
    local_ranks: list[int] = field(default_factory=list)
    remote_ranks: list[int] = field(default_factory=list)
    pair_tensors: dict[str, list[Any]] = field(default_factory=dict)  # local tensors (CPU) or descriptors (CUDA)
    pair_target_dtypes: dict[str, list[torch.dtype]] = field(default_factory=dict)
    bucket_size: int | None = None
    # executors, one per direction; which type depends on where the tensors live
    send_exec: Any = None
    recv_exec: Any = None
    send_buckets: list | None = None
    recv_buckets: list | None = None
    epoch: int = 0
    recv_done: int = 0  # epoch of the last receive this agent completed
    in_flight: bool = False  # a transfer has passed its start and not reached its end (stays set if it dies half-way)
    keepalive: list = field(default_factory=list)
    gen: int = 0  # how often this agent has registered this batch id; part of every key of the registration
    key: str = ""  # "batch:{id}/gen:{gen}"
    kind: str = ""  # "cuda" | "cpu"
    flags: Any = None  # CUDA: {"fwd": int32[ranks], "bwd": ...} completion flags other agents write into
    shared_gpu: bool = False  # another agent of the batch drives the same physical GPU: completion goes through the store
    any_shared_gpu: bool = False  # some GPU is driven by two agents of the batch: producers publish completion in the store
    wrote_done: bool = False
    node_barrier: Any = None  # semaphore rendezvous when every agent of the batch is on this machine
    # NVLS: this agent's arena in the batch's multicast team (the worker's replicated arena, or scratch), the team
    arena: Any = None
    scratch_arena: Any = None
    team: Any = None
    team_keys: list = field(default_factory=list)
    multicast_ops: int = 0  # ops of this agent's copy tables written with multimem.st
