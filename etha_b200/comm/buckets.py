"""Coalescing of chunks into wire messages (reference: src/etha/comm/get_buckets.py:12-43).

Chunks that share a `bucket_key` are packed greedily, in arrival order, until `bucket_size` bytes
(wire dtype) are reached; a chunk that is at least `bucket_size` travels alone, so `bucket_size=1`
disables coalescing.  Producer, contributors and consumers of a key all see the same chunk
sub-sequence, hence cut it at the same places.
"""

from __future__ import annotations

from .ir import Bucket, Chunk

__all__ = ["chunk_to_bucket_ops"]


def _device_of(chunk: Chunk):
    t = chunk.tensor
    return t.device if t is not None else None


def chunk_to_bucket_ops(chunks: list[Chunk], bucket_size: int) -> list[Bucket]:
    if bucket_size is None or bucket_size < 1:
        bucket_size = 1
    out: list[Bucket] = []
    open_groups: dict[tuple, list] = {}  # key -> [chunks, bytes]
    for c in chunks:
        n = c.nbytes
        if n >= bucket_size:
            out.append(Bucket(chunks=[c], device=_device_of(c)))
            continue
        group = open_groups.setdefault(c.bucket_key, [[], 0])
        group[0].append(c)
        group[1] += n
        if group[1] >= bucket_size:
            out.append(Bucket(chunks=group[0], device=_device_of(c)))
            del open_groups[c.bucket_key]
    for members, _ in open_groups.values():
        if members:
            out.append(Bucket(chunks=members, device=_device_of(members[0])))
    return out
