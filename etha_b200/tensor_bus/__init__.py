"""Tensor bus: worker-side client, agent daemon, command queue (API of the reference's `etha.tensor_bus`)."""

from .batch_state import BatchState
from .command_queue import CommandQueue, QueueFullError
from .commands import CleanupBatch, InitPair, Message, QueryStatus, RegisterTensors, Transfer
from .pair_state import PairState

__all__ = [
    "Message", "Transfer", "InitPair", "RegisterTensors", "QueryStatus", "CleanupBatch", "PairState", "BatchState",
    "CommandQueue", "QueueFullError", "TensorBusAgent", "TensorBusClient", "BatchHandler", "bootstrap_client",
    "BootstrapInfo", "TensorBusError",
]


def __getattr__(name):
    if name in ("TensorBusClient", "BatchHandler", "TensorBusError"):
        from . import client

        return getattr(client, name)
    if name == "TensorBusAgent":
        from .agent import TensorBusAgent

        return TensorBusAgent
    if name in ("bootstrap_client", "BootstrapInfo", "setup_ptrace"):
        from . import bootstrap

        return getattr(bootstrap, name)
    raise AttributeError(name)
