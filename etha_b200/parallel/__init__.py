"""Peer memory plumbing: exporting/mapping device allocations across processes, signal flags, VMM arenas."""

from .peer import PeerMemory, RegionDesc, TensorDesc

__all__ = ["PeerMemory", "RegionDesc", "TensorDesc"]
