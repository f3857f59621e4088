"""Bucket executor over `torch.distributed` point-to-point messages (gloo on CPU, NCCL on GPUs).

This is the portable path: the oracle on CPU, the fallback across nodes and the NCCL baseline the
peer-to-peer executor is measured against.  It plays the role of the reference's `bucket_comm`
(src/etha/comm/comm_methods.py:53-119) but is organised differently:

* the unit of ordering is the *directed pair channel* `(sender -> receiver)`.  Both ends enumerate
  the messages of a channel in the same canonical order, so matching needs no sub-groups; a
  BROADCAST bucket is packed once and sent on one channel per consumer;
* a `Partial` source is collapsed at the route's primary: the other family members send their
  pending values (source dtype), the primary accumulates in fp32 in family order, rounds once to the
  wire dtype and ships.  No all-reduce, no process-group creation;
* with gloo every receive is posted up front and messages carry their channel sequence number as
  tag (blocking waits cannot deadlock); with NCCL, which has no tags, channels are strictly ordered,
  at most `max_in_flight` messages are outstanding per channel and completion is polled.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .ir import Bucket, Chunk, reduce_family_values

__all__ = ["bucket_comm"]


def _align16(n: int) -> int:
    return (n + 15) & ~15


def _layout(chunks: list[Chunk], itemsize_of) -> tuple[list[int], int]:
    offs, cur = [], 0
    for c in chunks:
        cur = _align16(cur)
        offs.append(cur)
        cur += c.numel * itemsize_of(c)
    return offs, max(cur, 1)


def _views(buf: torch.Tensor, chunks: list[Chunk], offsets: list[int], dtype_of) -> list[torch.Tensor]:
    out = []
    for c, off in zip(chunks, offsets):
        dt = dtype_of(c)
        n = c.numel * dt.itemsize
        out.append(buf.narrow(0, off, n).view(dt).view(c.chunk_shape))
    return out


@dataclass
class _Message:
    bucket_id: int
    peer: int
    is_send: bool
    seq: int = 0  # position on its channel
    buffer: torch.Tensor | None = None
    work: dist.Work | None = None
    posted: bool = False
    done: bool = False
    inplace: bool = False  # the receive landed directly in the destination view


@dataclass
class _BucketState:
    bucket: Bucket
    role: str  # "primary" | "contributor" | "consumer"
    sends: list[_Message] = field(default_factory=list)
    contrib_recvs: list[_Message] = field(default_factory=list)
    data_recv: _Message | None = None
    wire: torch.Tensor | None = None
    wire_ready: bool = False


class _Engine:
    def __init__(self, buckets: list[Bucket], max_in_flight: int):
        self.rank = dist.get_rank()
        self.window = max(1, max_in_flight)
        self.states: list[_BucketState] = []
        self.out_ch: dict[int, deque[_Message]] = {}
        self.in_ch: dict[int, deque[_Message]] = {}
        seq_out: dict[int, int] = {}
        seq_in: dict[int, int] = {}

        def add(msg: _Message) -> _Message:
            table, seqs = (self.out_ch, seq_out) if msg.is_send else (self.in_ch, seq_in)
            msg.seq = seqs.get(msg.peer, 0)
            seqs[msg.peer] = msg.seq + 1
            table.setdefault(msg.peer, deque()).append(msg)
            return msg

        for i, b in enumerate(buckets):
            head = b.head
            if head.contributes_to is not None:
                st = _BucketState(bucket=b, role="contributor")
                st.sends.append(add(_Message(i, head.contributes_to, True)))
            elif head.is_source:
                st = _BucketState(bucket=b, role="primary")
                if head.family is not None:
                    for q in head.family.ranks:
                        if q != self.rank:
                            st.contrib_recvs.append(add(_Message(i, q, False)))
                for d in head.dst_ranks:
                    st.sends.append(add(_Message(i, d, True)))
            else:
                st = _BucketState(bucket=b, role="consumer")
                st.data_recv = add(_Message(i, head.src_rank, False))
            self.states.append(st)

        dev = next((b.device for b in buckets if b.device is not None), torch.device("cpu"))
        self.device = dev
        self.on_cpu = dev.type == "cpu"

    # ---- buffers -------------------------------------------------------------------------
    def _alloc(self, nbytes: int) -> torch.Tensor:
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device)

    def _recv_buffer(self, st: _BucketState, msg: _Message) -> torch.Tensor:
        b = st.bucket
        if st.role == "consumer":
            if len(b.chunks) == 1:
                c = b.head
                view = c.dst_view()
                if view.is_contiguous() and view.dtype == c.transfer_dtype and view.numel() > 0:
                    msg.inplace = True
                    return view
            return self._alloc(b.total_bytes)
        # contribution: same chunks, source dtype
        src_dtype = b.head.src_tensor.dtype
        _, total = _layout(b.chunks, lambda c: src_dtype.itemsize)
        return self._alloc(total)

    def _build_contribution(self, st: _BucketState) -> torch.Tensor:
        b = st.bucket
        src_dtype = b.head.src_tensor.dtype
        if len(b.chunks) == 1:
            v = b.head.src_view()
            if v.is_contiguous() and v.numel() > 0:
                return v
        offs, total = _layout(b.chunks, lambda c: src_dtype.itemsize)
        buf = self._alloc(total)
        for c, dst in zip(b.chunks, _views(buf, b.chunks, offs, lambda c: src_dtype)):
            dst.copy_(c.src_view())
        return buf

    def _build_wire(self, st: _BucketState) -> None:
        """Primary: gather (and reduce) the bucket into wire layout; serve the local consumer if any."""
        b = st.bucket
        fam = b.head.family
        single_inplace = False
        if fam is None and len(b.chunks) == 1:
            c = b.head
            v = c.src_view()
            if v.is_contiguous() and v.dtype == c.transfer_dtype and v.numel() > 0:
                st.wire = v
                single_inplace = True
        if not single_inplace:
            st.wire = self._alloc(b.total_bytes)
            wire_views = _views(st.wire, b.chunks, b.offsets, lambda c: c.transfer_dtype)
            if fam is None:
                for c, w in zip(b.chunks, wire_views):
                    w.copy_(c.src_view())
            else:
                src_dtype = b.head.src_tensor.dtype
                offs, _ = _layout(b.chunks, lambda c: src_dtype.itemsize)
                contrib_views = {
                    m.peer: _views(m.buffer.view(torch.uint8).reshape(-1), b.chunks, offs, lambda c: src_dtype)
                    for m in st.contrib_recvs
                }
                for k, (c, w) in enumerate(zip(b.chunks, wire_views)):
                    vals = [c.src_view() if q == self.rank else contrib_views[q][k] for q in fam.ranks]
                    # collapse in fp32, round once to the source dtype (what Partial -> Replicate yields),
                    # then convert to the wire dtype
                    w.copy_(reduce_family_values(vals, fam, src_dtype))
        # local consumers (a rank on both meshes may be one of the consumers of its own cells)
        if single_inplace:
            c = b.head
            if c.is_target:
                c.dst_view().copy_(st.wire.view(c.chunk_shape))
        else:
            for c, w in zip(b.chunks, _views(st.wire, b.chunks, b.offsets, lambda c: c.transfer_dtype)):
                if c.is_target:
                    c.dst_view().copy_(w)
        st.wire_ready = True

    def _scatter(self, st: _BucketState) -> None:
        b = st.bucket
        buf = st.data_recv.buffer
        if st.data_recv.inplace:
            return
        for c, w in zip(b.chunks, _views(buf, b.chunks, b.offsets, lambda c: c.transfer_dtype)):
            c.dst_view().copy_(w)

    # ---- wire ----------------------------------------------------------------------------
    @staticmethod
    def _flat(t: torch.Tensor) -> torch.Tensor:
        return t.reshape(-1) if t.is_contiguous() else t

    def _post(self, msg: _Message, use_tags: bool) -> None:
        tag = msg.seq if use_tags else 0
        buf = self._flat(msg.buffer)
        if msg.is_send:
            msg.work = dist.isend(buf, dst=msg.peer, tag=tag)
        else:
            msg.work = dist.irecv(buf, src=msg.peer, tag=tag)
        msg.posted = True

    # ---- gloo: post everything, tags decouple order -----------------------------------------
    def run_tagged(self) -> None:
        for st in self.states:
            for m in st.contrib_recvs:
                m.buffer = self._recv_buffer(st, m)
                self._post(m, True)
            if st.data_recv is not None:
                st.data_recv.buffer = self._recv_buffer(st, st.data_recv)
                self._post(st.data_recv, True)
        # dependency-free sends first
        for st in self.states:
            if st.role == "contributor":
                buf = self._build_contribution(st)
                for m in st.sends:
                    m.buffer = buf
                    self._post(m, True)
            elif st.role == "primary" and st.bucket.head.family is None:
                self._build_wire(st)
                for m in st.sends:
                    m.buffer = st.wire
                    self._post(m, True)
        for st in self.states:
            if st.role == "primary" and st.bucket.head.family is not None:
                for m in st.contrib_recvs:
                    m.work.wait()
                self._build_wire(st)
                for m in st.sends:
                    m.buffer = st.wire
                    self._post(m, True)
        for st in self.states:
            for m in st.sends:
                m.work.wait()
            if st.data_recv is not None:
                st.data_recv.work.wait()
                self._scatter(st)

    # ---- NCCL: ordered channels, bounded window, polling -------------------------------------
    def run_ordered(self) -> None:
        in_flight_out: dict[int, deque[_Message]] = {p: deque() for p in self.out_ch}
        in_flight_in: dict[int, deque[_Message]] = {p: deque() for p in self.in_ch}
        pending = sum(len(q) for q in self.out_ch.values()) + sum(len(q) for q in self.in_ch.values())
        # buckets with no wire message at all (pure local copies)
        for st in self.states:
            if st.role == "primary" and not st.sends and not st.contrib_recvs:
                self._build_wire(st)
                st.wire = None
        while pending:
            progressed = False
            # receives: never depend on anything
            for peer, q in self.in_ch.items():
                fl = in_flight_in[peer]
                while q and len(fl) < self.window:
                    m = q.popleft()
                    st = self.states[m.bucket_id]
                    m.buffer = self._recv_buffer(st, m)
                    self._post(m, False)
                    fl.append(m)
                    progressed = True
                while fl and fl[0].work.is_completed():
                    m = fl.popleft()
                    m.work.wait()
                    m.done = True
                    pending -= 1
                    progressed = True
                    st = self.states[m.bucket_id]
                    if st.role == "consumer":
                        self._scatter(st)
                        m.buffer = None
            # sends: the head of a channel may wait for contributions
            for peer, q in self.out_ch.items():
                fl = in_flight_out[peer]
                while q and len(fl) < self.window:
                    m = q[0]
                    st = self.states[m.bucket_id]
                    if st.role == "contributor":
                        if m.buffer is None:
                            m.buffer = self._build_contribution(st)
                    else:
                        if not st.wire_ready:
                            if not all(r.done for r in st.contrib_recvs):
                                break
                            self._build_wire(st)
                            for r in st.contrib_recvs:
                                r.buffer = None
                        m.buffer = st.wire
                    q.popleft()
                    self._post(m, False)
                    fl.append(m)
                    progressed = True
                while fl and fl[0].work.is_completed():
                    m = fl.popleft()
                    m.work.wait()
                    m.done = True
                    m.buffer = None
                    pending -= 1
                    progressed = True
                    st = self.states[m.bucket_id]
                    if all(s.done for s in st.sends):
                        st.wire = None
            # primaries whose only consumers are local still need their contributions
            for st in self.states:
                if st.role == "primary" and not st.sends and st.contrib_recvs and not st.wire_ready:
                    if all(r.done for r in st.contrib_recvs):
                        self._build_wire(st)
                        st.wire = None
                        progressed = True
            if not progressed and self.on_cpu:
                raise RuntimeError("ordered execution made no progress on a backend without completion polling")


def bucket_comm(buckets: list[Bucket], max_in_flight: int = 2) -> None:
    """Execute `buckets` (all of this rank's, both roles) and return when this rank's part is done.

    On CUDA the call ends with a device synchronize, like the reference's, so timing it with events
    around the call is meaningful.
    """
    if not buckets:
        return
    eng = _Engine(buckets, max_in_flight)
    if eng.on_cpu:
        eng.run_tagged()
        # local-only primaries with contributions are handled inside run_tagged via _build_wire
    else:
        eng.run_ordered()
        torch.cuda.synchronize()
