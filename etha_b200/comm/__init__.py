"""Planner, chunk specializer and executors (API of the reference's `etha.comm`, src/etha/comm/__init__.py)."""

from .baselines import gather_broadcast_comm
from .bucket_exec import bucket_comm
from .buckets import chunk_to_bucket_ops
from .chunks import m2m_to_chunks
from .ir import Bucket, Chunk, Endpoint, M2MMap, PartialFamily, Route, Transport
from .planner import get_m2m_map, plan_m2m
from .shaped import plan_for_shape, shaped_to_chunks

__all__ = [
    "M2MMap",
    "Route",
    "Endpoint",
    "Transport",
    "Chunk",
    "Bucket",
    "PartialFamily",
    "get_m2m_map",
    "plan_m2m",
    "m2m_to_chunks",
    "chunk_to_bucket_ops",
    "bucket_comm",
    "gather_broadcast_comm",
    "plan_for_shape",
    "shaped_to_chunks",
    "P2PBatch",
    "PairLayout",
]


def __getattr__(name):
    # the peer-to-peer executor loads the CUDA library; import it only when asked for
    if name in ("P2PBatch", "PairLayout", "TransferTimeout", "link_local"):
        from . import p2p

        return getattr(p2p, name)
    raise AttributeError(name)
