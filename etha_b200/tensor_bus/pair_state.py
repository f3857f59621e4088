"""In-memory state of one registered pair on an agent (reference: src/etha/tensor_bus/pair_state.py:12-37)."""

from dataclasses import dataclass
import torch

from ..comm.ir import M2MMap


@dataclass(kw_only=True)
class PairState:
    pair_name: str
    local_name: str
    local_ranks: list[int]
    remote_name: str
    remote_ranks: list[int]
    pair_size: int
    local_is_first: bool
    # meshes of global agent ranks and placements of both sides (None when a side sent none)
    local_mesh: torch.Tensor | None = None
    local_placements: tuple | None = None
    remote_mesh: torch.Tensor | None = None
    remote_placements: tuple | None = None
    m2m_send: M2MMap | None = None  # local -> remote
    m2m_recv: M2MMap | None = None  # remote -> local
