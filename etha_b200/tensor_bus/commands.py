"""Worker -> agent commands (wire format of the reference: src/etha/tensor_bus/commands.py:8-74).

msgspec tagged union: the tag field is `"type"` with the class name as value; the fields of a command
come first, then the two keyword-only base fields, e.g.
`{"type":"Transfer","batch_id":"b","transfer_type":"send","timestamp":1.0,"semaphore_name":"/s"}`.
"""

from typing import Literal

import msgspec


class BaseCommand(msgspec.Struct, tag=True, kw_only=True):
    timestamp: float | None = None
    semaphore_name: str | None = None  # posted by the agent once the command has been handled


class Transfer(BaseCommand):
    """Run one direction of a registered batch."""

    batch_id: str
    transfer_type: Literal["send", "recv"]


class RegisterTensors(BaseCommand):
    """Register the tensors of one batch; `tensors` is `[(pair_name, payload)]` in registration order."""

    batch_id: str
    tensors: list[tuple[str, memoryview]]
    bucket_size: int | None = None


class InitPair(BaseCommand):
    """Declare this side of a named pair together with its mesh shape and placements (pickled)."""

    pair_name: str
    local_name: str
    expected_world_size: int
    remote_name: str
    mesh_shape_payload: memoryview | None = None
    placements_payload: memoryview | None = None


class QueryStatus(BaseCommand):
    batch_id: str
    state_name: str


class CleanupBatch(BaseCommand):
    batch_id: str


Message = Transfer | RegisterTensors | InitPair | QueryStatus | CleanupBatch
