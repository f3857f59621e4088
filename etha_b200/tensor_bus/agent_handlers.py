"""Command handlers of the agent, written as generators that `yield` whenever they have to wait.

Key layout in the KV store (component `tensorbus` unless noted), same names as the reference where it has
them (src/etha/tensor_bus/agent.py:224-243, 450-455):

    pair:{p}/rank:{r}/{local_name}             "1"      this agent registered for side `local_name`
    pair:{p}/{local_name}/expected_world_size  int      ranks on that side
    pair:{p}/rank:{r}/mesh_shape | placements  pickles  layout of the side `r` belongs to
    batch:{b}/regs/rank:{r}                    int      how often agent `r` registered batch id `b`: the generation  (new)
    batch:{b}/gen:{g}/rank:{r}/meta            pickle   tensor descriptors + flag arrays of agent `r`   (new)
    batch:{b}/gen:{g}/go/...                   barrier  round k = every agent entered transfer k          (new)
    batch:{b}/gen:{g}/done/rank:{r}            int      last transfer whose copies producer `r` finished (host completion) (new)
    batch:{b}/gen:{g}/state:send_epoch         int      newest send, component `global`                   (new)
    batch:{b}/state:transfer_signal            "1"/"0"  component `global`

Every key that belongs to one registration carries its generation `g`: registering the same batch id again (after a
cleanup or a worker restart) never reads descriptors, barrier counts or epochs of the previous registration.  The
barrier and completion keys are reused by every transfer, and `CleanupBatch` deletes what this agent wrote.
"""

from __future__ import annotations

import logging
import os
import pickle
import time

import torch
from torch.distributed.tensor.placement_types import Partial

from ..comm import chunk_to_bucket_ops, m2m_to_chunks
from ..comm.bucket_exec import bucket_comm
from ..comm.ir import M2MMap
from ..comm.planner import plan_m2m
from .batch_state import BatchState
from .commands import CleanupBatch, InitPair, QueryStatus, RegisterTensors, Transfer
from .pair_state import PairState

logger = logging.getLogger(__name__)


def _hostname() -> str:
    import socket

    return socket.gethostname()


def _wire_dtype(src: torch.dtype, dst: torch.dtype) -> torch.dtype:
    """Smaller item size wins; on a tie the SOURCE dtype travels and the consumer converts (the reference lets each
    side pick its own dtype on a tie and reinterprets bytes, src/etha/tensor_bus/agent.py:635-640)."""
    return src if src.itemsize <= dst.itemsize else dst


class AgentHandlers:
    # ---- InitPair ---------------------------------------------------------------------------------
    def _init_pair_job(self, msg: InitPair):
        pair, local_name, remote_name = msg.pair_name, msg.local_name, msg.remote_name
        store = self.store
        store.set(f"pair:{pair}/rank:{self.rank}/{local_name}", "1")
        store.set(f"pair:{pair}/{local_name}/expected_world_size", str(msg.expected_world_size))
        if msg.mesh_shape_payload is not None and msg.placements_payload is not None:
            store.set_bytes(f"pair:{pair}/rank:{self.rank}/mesh_shape", bytes(msg.mesh_shape_payload))
            store.set_bytes(f"pair:{pair}/rank:{self.rank}/placements", bytes(msg.placements_payload))

        def side(name: str, expected: int):
            cands = [f"pair:{pair}/rank:{r}/{name}" for r in range(self.world_size)]
            while True:
                keys = store.poll_keys(f"pair:{pair}/rank:*/{name}", "1", cands)
                if len(keys) >= expected:
                    return sorted(self._extract_rank(k) for k in keys)[:expected]
                yield None

        local_ranks = yield from side(local_name, msg.expected_world_size)
        while True:
            raw = store.try_get(f"pair:{pair}/{remote_name}/expected_world_size")
            if raw:
                break
            yield
        expected_remote = int(raw.decode())
        remote_ranks = yield from side(remote_name, expected_remote)

        def layout(ranks):
            infos = []
            for r in ranks:
                ms = store.get_bytes(f"pair:{pair}/rank:{r}/mesh_shape")
                pl = store.get_bytes(f"pair:{pair}/rank:{r}/placements")
                if ms and pl:
                    mesh = pickle.loads(ms)
                    # newer clients send {"shape", "ids"} (the mesh's rank ids in mesh order); a bare shape tuple is
                    # the reference's payload and means "ascending ranks, row-major"
                    shape = tuple(mesh["shape"]) if isinstance(mesh, dict) else tuple(mesh)
                    ids = tuple(mesh["ids"]) if isinstance(mesh, dict) and mesh.get("ids") is not None else None
                    infos.append((shape, tuple(pickle.loads(pl)), ids))
            if not infos:
                return None
            for i, info in enumerate(infos):
                if info != infos[0]:
                    raise ValueError(f"pair '{pair}': rank {ranks[i]} declared {info}, rank {ranks[0]} declared {infos[0]}")
            shape, plc, ids = infos[0]
            n = 1
            for s in shape:
                n *= s
            if n != len(ranks):
                raise ValueError(f"pair '{pair}': mesh shape {shape} does not hold {len(ranks)} ranks")
            agents = sorted(ranks)
            if ids is None:
                # the registered ranks, ascending, fill the mesh row-major (the reference assumes a contiguous range)
                return torch.tensor(agents).view(shape), plc
            # the worker's mesh names its ranks in its own numbering: the k-th smallest id is the worker attached to
            # the k-th smallest agent rank of this side, and the mesh keeps the worker's order
            if len(set(ids)) != n:
                raise ValueError(f"pair '{pair}': the device mesh {ids} does not name {n} distinct ranks")
            order = {wid: k for k, wid in enumerate(sorted(ids))}
            return torch.tensor([agents[order[w]] for w in ids]).view(shape), plc

        local, remote = layout(local_ranks), layout(remote_ranks)
        st = PairState(
            pair_name=pair, local_name=local_name, local_ranks=local_ranks, remote_name=remote_name,
            remote_ranks=remote_ranks, pair_size=len(local_ranks) + len(remote_ranks), local_is_first=local_name < remote_name,
        )
        if local and remote:
            st.local_mesh, st.local_placements = local
            st.remote_mesh, st.remote_placements = remote
            def plan(smesh, splc, tmesh, tplc):
                from ..comm.planner import _check_placements, is_strided_shard
                from ..comm.shaped import BOX_PLAN_ONLY

                if any(is_strided_shard(p) for p in tuple(splc) + tuple(tplc)):
                    # no shape-independent plan exists for a strided shard: validate now, plan per tensor from boxes
                    _check_placements(tuple(splc), smesh, "source", allow_strided=True)
                    _check_placements(tuple(tplc), tmesh, "target", allow_strided=True)
                    return BOX_PLAN_ONLY
                return plan_m2m(smesh, splc, tmesh, tplc)

            if not any(isinstance(p, Partial) for p in st.remote_placements):
                st.m2m_send = plan(st.local_mesh, st.local_placements, st.remote_mesh, st.remote_placements)
            if not any(isinstance(p, Partial) for p in st.local_placements):
                st.m2m_recv = plan(st.remote_mesh, st.remote_placements, st.local_mesh, st.local_placements)
        self.pairs[pair] = st
        self.state.set_matched(pair)
        logger.info("Agent %s: pair '%s' matched: %s %s <-> %s %s", self.rank, pair, local_name, local_ranks, remote_name, remote_ranks)

    # ---- RegisterTensors --------------------------------------------------------------------------
    def _register_tensors_job(self, msg: RegisterTensors):
        from .agent import decode_tensor

        batch_id = msg.batch_id
        entries = []  # (pair_name, kind, tensor-or-desc)
        for pair_name, payload in msg.tensors:
            if pair_name not in self.pairs:
                raise ValueError(f"RegisterTensors for unknown pair: {pair_name}")
            kind, obj = decode_tensor(bytes(payload))
            entries.append((pair_name, kind, obj))
        pair_names = list(dict.fromkeys(p for p, _, _ in entries))
        first = self.pairs[pair_names[0]]
        for p in pair_names[1:]:
            ps = self.pairs[p]
            if set(ps.local_ranks) != set(first.local_ranks) or set(ps.remote_ranks) != set(first.remote_ranks):
                raise ValueError(f"Batch {batch_id}: pair '{p}' spans different ranks than pair '{pair_names[0]}'")
        kinds = {k for _, k, _ in entries}
        if len(kinds) != 1:
            raise ValueError(f"Batch {batch_id}: CPU and CUDA tensors cannot be mixed")
        kind = kinds.pop()
        batch = BatchState(batch_id=batch_id, pair_names=pair_names, bucket_size=msg.bucket_size,
                           local_leader=min(first.local_ranks), local_ranks=list(first.local_ranks),
                           remote_ranks=list(first.remote_ranks))
        for p, _, obj in entries:
            batch.pair_tensors.setdefault(p, []).append(obj)
        all_ranks = sorted(set(first.local_ranks) | set(first.remote_ranks))
        if batch_id in self.batches:
            self._drop_batch(self.batches.pop(batch_id))  # re-registration without a cleanup: release the old one first
        # generation of this registration: every agent of the batch registers it the same number of times, and the
        # count lives in the store, so it also survives an agent that was restarted in between
        batch.gen = self.store.counter_add(f"batch:{batch_id}/regs/rank:{self.rank}", 1)
        batch.key = f"batch:{batch_id}/gen:{batch.gen}"

        # publish what the other agents need, then wait for theirs
        import uuid

        meta = {"rank": self.rank, "kind": kind, "local_name": first.local_name, "gen": batch.gen, "host": _hostname(),
                "nonce": uuid.uuid4().hex[:12]}
        if kind == "cuda":
            from ..parallel.peer import PeerMemory

            if self._peer is None:
                self._peer = PeerMemory(self.device)
            flags = {d: torch.zeros(len(all_ranks), dtype=torch.int32, device=self.device) for d in ("fwd", "bwd")}
            batch.flags = flags
            meta["descs"] = [obj for _, _, obj in entries]
            meta["flags"] = {d: self._peer.describe(t) for d, t in flags.items()}
            # tensors the worker placed in its replicated (VMM) arena: fetch the arena once, tell the others its size
            tickets = {(d.arena["pid"], d.arena["va"]): d.arena for _, _, d in entries if getattr(d, "arena", None)}
            if len(tickets) > 1:
                raise ValueError(f"Batch {batch_id}: tensors of {len(tickets)} replicated arenas; a worker has one")
            if tickets:
                ticket = next(iter(tickets.values()))
                batch.arena = self._import_worker_arena(ticket)
                meta["arena"] = {"size": ticket["size"], "key": (ticket["pid"], ticket["device_index"], ticket["va"]),
                                 "socket": ticket["socket"]}
            meta["gpu"] = str(torch.cuda.get_device_properties(self.device).uuid)
            from ..ops import device_info

            meta["multicast"] = bool(device_info()["multicast"])
        else:
            meta["descs"] = [(tuple(t.shape), str(t.dtype).replace("torch.", "")) for _, _, t in entries]
        self.store.set_bytes(f"{batch.key}/rank:{self.rank}/meta", pickle.dumps(meta))
        metas = {}
        while len(metas) < len(all_ranks):
            for r in all_ranks:
                if r not in metas:
                    raw = self.store.get_bytes(f"{batch.key}/rank:{r}/meta")
                    if raw:
                        metas[r] = pickle.loads(raw)
            if len(metas) < len(all_ranks):
                yield
        for r, m in metas.items():
            if len(m["descs"]) != len(entries) or m["kind"] != kind:
                raise ValueError(f"Batch {batch_id}: rank {r} registered {len(m['descs'])} {m['kind']} tensors, "
                                 f"rank {self.rank} registered {len(entries)} {kind} tensors")
        batch.kind = kind
        try:
            self._build_executors(batch, entries, metas, all_ranks, kind, flags if kind == "cuda" else None)
        except Exception:
            self._drop_batch(batch)  # nothing of a registration that failed half-way stays behind (semaphores, keys, teams)
            raise
        self.batches[batch_id] = batch
        self.state.put(f"batch:{batch_id}/state:multicast_ops", str(batch.multicast_ops).encode())
        logger.info("Agent %s: batch %s registered (%d tensors, %s)", self.rank, batch_id, len(entries), kind)

    def _build_executors(self, batch: BatchState, entries, metas, all_ranks, kind: str, flags) -> None:
        """Everything a registration builds once every agent's descriptors are known."""
        batch_id = batch.batch_id
        if len({m.get("host") for m in metas.values()}) == 1 and len(all_ranks) > 1:
            # every agent of the batch runs on this machine: the per-transfer rendezvous uses semaphores, not the store
            from .node_barrier import NodeBarrier

            # the scope carries every agent's nonce of this registration: semaphores a crashed earlier run left under the
            # same namespace and batch id can never be picked up
            nonces = "".join(metas[r].get("nonce", "") for r in all_ranks)
            batch.node_barrier = NodeBarrier(f"{self.namespace}/{batch.key}/{nonces}", self.rank, all_ranks)
        if kind == "cuda" and len({m.get("host") for m in metas.values()}) == 1:
            if any(m.get("arena") for m in metas.values()):
                self._join_multicast_team(batch, metas, all_ranks)
            self._build_p2p(batch, entries, metas, all_ranks, flags)
        elif kind == "cuda":
            # the pair spans machines: peer pointers end at the NVLink domain, so fall back to the bucket executor
            # over NCCL on tensors rebuilt from the workers' descriptors
            local = [(p, k, self._peer.as_tensor(d)) for p, k, d in entries]
            for m in metas.values():
                m["descs"] = [(tuple(d.shape), d.dtype) for d in m["descs"]]
            self._build_buckets(batch, local, metas)
        else:
            self._build_buckets(batch, entries, metas)

    def _build_buckets(self, batch: BatchState, entries, metas) -> None:
        """CPU tensors: chunks and buckets for both directions (gloo bucket executor)."""
        import torch as _t

        remote0 = metas[batch.remote_ranks[0]]["descs"]
        send_chunks, recv_chunks = [], []
        fallback = True
        for k, (pair_name, _, t) in enumerate(entries):
            ps = self.pairs[pair_name]
            rdtype = getattr(_t, remote0[k][1])
            if ps.m2m_send is not None:
                fallback = False
                send_chunks += self._chunks_for(ps.m2m_send, ps.local_mesh, ps.local_placements, ps.remote_mesh,
                                                ps.remote_placements, {r: metas[r]["descs"][k][0] for r in ps.local_ranks},
                                                {r: metas[r]["descs"][k][0] for r in ps.remote_ranks}, source=t, wire=_wire_dtype(t.dtype, rdtype), k=k)
            if ps.m2m_recv is not None:
                fallback = False
                recv_chunks += self._chunks_for(ps.m2m_recv, ps.remote_mesh, ps.remote_placements, ps.local_mesh,
                                                ps.local_placements, {r: metas[r]["descs"][k][0] for r in ps.remote_ranks},
                                                {r: metas[r]["descs"][k][0] for r in ps.local_ranks}, target=t, wire=_wire_dtype(rdtype, t.dtype), k=k)
        if fallback:
            batch.send_exec = batch.recv_exec = "plain"
        else:
            size = batch.bucket_size or 1
            batch.send_buckets = chunk_to_bucket_ops(send_chunks, size)
            batch.recv_buckets = chunk_to_bucket_ops(recv_chunks, size)
            # a direction is usable only if every pair of the batch has a plan for it (a Partial side can only send)
            pairs = [self.pairs[p] for p in batch.pair_names]
            batch.send_exec = "bucket" if all(ps.m2m_send is not None for ps in pairs) else None
            batch.recv_exec = "bucket" if all(ps.m2m_recv is not None for ps in pairs) else None

    def _chunks_for(self, m2m, smesh, splc, tmesh, tplc, source_shapes, target_shapes, source=None, target=None,
                    wire=None, k=0):
        """Chunks of one tensor: the lcm plan when every shard of both sides divides evenly, explicit boxes otherwise
        (decided from all ranks' shapes, so both sides agree)."""
        from ..comm.chunks import plan_fits_shapes
        from ..comm.shaped import BOX_PLAN_ONLY

        if m2m is not BOX_PLAN_ONLY and plan_fits_shapes(m2m, source_shapes, target_shapes):
            return m2m_to_chunks(m2m, self.rank, source_tensor=source, target_tensor=target, transfer_dtype=wire,
                                 source_mesh=smesh, tensor_id=k)
        from ..comm.shaped import infer_global_shape, plan_for_shape, shaped_to_chunks

        plan = plan_for_shape(smesh, splc, tmesh, tplc, infer_global_shape(smesh, splc, source_shapes))
        return shaped_to_chunks(plan, self.rank, source, target, wire, source_mesh=smesh, tensor_id=k)

    def _build_p2p(self, batch: BatchState, entries, metas, all_ranks, flags) -> None:
        """CUDA tensors: one copy table per direction, built from every agent's descriptors."""
        from ..comm.p2p import P2PBatch, PairLayout

        first = self.pairs[batch.pair_names[0]]
        local_name = first.local_name
        # canonical direction names so that both sides pick the same flag array for a direction
        send_dir = "fwd" if first.local_is_first else "bwd"
        recv_dir = "bwd" if first.local_is_first else "fwd"

        def build(direction: str, sending: bool):
            layouts, ok = [], True
            for pair_name, _, _ in entries:
                ps = self.pairs[pair_name]
                m = ps.m2m_send if sending else ps.m2m_recv
                if m is None and ps.local_mesh is None and ps.remote_mesh is None:
                    # no layout was declared for this pair: tensor i goes whole to the same-index rank of the other
                    # side (reference fallback, src/etha/tensor_bus/agent.py:485-498), as one copy op per tensor
                    src_ranks = sorted(batch.local_ranks if sending else batch.remote_ranks)
                    dst_ranks = sorted(batch.remote_ranks if sending else batch.local_ranks)
                    if len(src_ranks) != len(dst_ranks):
                        raise ValueError(f"pair '{pair_name}' declared no layout and its sides have {len(src_ranks)} and "
                                         f"{len(dst_ranks)} ranks: whole tensors can only go rank to rank")
                    layouts.append(PairLayout(torch.tensor(src_ranks), None, torch.tensor(dst_ranks), None, plain=True))
                    continue
                if m is None:
                    ok = False
                    break
                lay = (PairLayout(ps.local_mesh, ps.local_placements, ps.remote_mesh, ps.remote_placements) if sending
                       else PairLayout(ps.remote_mesh, ps.remote_placements, ps.local_mesh, ps.local_placements))
                if isinstance(m, M2MMap):
                    lay._plan = m  # a layout without a shape-independent plan is planned from boxes by the batch itself
                layouts.append(lay)
            if not ok:
                return None
            src_side = set(batch.local_ranks if sending else batch.remote_ranks)
            by_rank = {}
            for r in all_ranks:
                descs = metas[r]["descs"]
                by_rank[r] = {
                    "rank": r,
                    "src": descs if r in src_side else [None] * len(descs),
                    "dst": descs if r not in src_side else [None] * len(descs),
                    "flags": metas[r]["flags"][direction],
                    "gpu": metas[r].get("gpu"),
                }
            b = P2PBatch(self.rank, all_ranks, self.device, peer=self._peer, use_ipc=True, nvls=batch.team)
            b.multicast_min_replicas = int(os.environ.get("ETHA_NVLS_MIN_REPLICAS", "2"))
            b.build_from(layouts, by_rank, flags[direction])
            batch.multicast_ops += b.multicast_ops
            return b

        batch.send_exec = build(send_dir, True)
        batch.recv_exec = build(recv_dir, False)
        # the device-side wait is used only when no other agent of the batch drives the same physical GPU:
        # two processes time-slicing one GPU must never have one kernel spin on a flag the other one sets
        mine = metas[self.rank]["gpu"]
        batch.shared_gpu = sum(1 for r in all_ranks if metas[r]["gpu"] == mine) > 1
        gpus = [metas[r]["gpu"] for r in all_ranks]
        batch.any_shared_gpu = len(set(gpus)) < len(gpus)  # some agent of the batch completes through the store

    # ---- NVLS: replicated arenas of the workers bound to one multicast object --------------------------------
    def _import_worker_arena(self, ticket: dict):
        """Map the worker's replicated arena in this process: the file descriptor comes over the Unix socket the
        worker's client serves (SCM_RIGHTS).  One import per arena; later batches reuse it."""
        import socket

        from ..parallel.arena import ImportedArena

        key = (ticket["pid"], ticket["va"])
        arena = self._worker_arenas.get(key)
        if arena is None:
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.settimeout(10.0)
                c.connect(ticket["socket"])
                _msg, fds, _flags, _addr = socket.recv_fds(c, 16, 4)
                c.send(b"k")
            if not fds:
                raise RuntimeError(f"the worker's arena socket {ticket['socket']} sent no file descriptor")
            arena = ImportedArena(fds[0], ticket["size"], self.device)
            self._worker_arenas[key] = arena
            # descriptors of views of the arena name the worker's address range: resolve them to this mapping
            self._peer.adopt_mapping((ticket["pid"], ticket["device_index"], ticket["va"]), arena.va)
        return arena

    def _kv_all_gather(self, batch: BatchState, ranks):
        """`all_gather(obj)` over the KV store for the ranks of one batch (blocking, bounded by the store timeout):
        what the multicast team construction uses as its exchange and barrier."""
        seq = [0]

        def all_gather(obj):
            seq[0] += 1
            prefix = f"{batch.key}/team/{seq[0]}"
            self.store.set_bytes(f"{prefix}/rank:{self.rank}", pickle.dumps(obj))
            batch.team_keys.append(f"{prefix}/rank:{self.rank}")
            deadline = time.monotonic() + min(self.store_timeout, 120.0)
            out = {}
            while len(out) < len(ranks):
                for r in ranks:
                    if r not in out:
                        raw = self.store.get_bytes(f"{prefix}/rank:{r}")
                        if raw:
                            out[r] = pickle.loads(raw)
                if len(out) < len(ranks):
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"multicast team of batch {batch.batch_id}: ranks {sorted(set(ranks) - set(out))} did not answer")
                    time.sleep(0.001)
            return [out[r] for r in ranks]

        return all_gather

    def _join_multicast_team(self, batch: BatchState, metas, all_ranks) -> None:
        """Every agent of the batch joins one NVLS team: consumers whose workers registered tensors of a replicated
        arena bind that arena, everybody else binds a scratch arena of the same size (every member device of a
        multicast object must have memory bound).  Any obstacle (no multicast support, arenas of different sizes)
        leaves `batch.team` unset and the fan-out falls back to one peer store per replica."""
        from ..ops import device_info
        from ..parallel.arena import NvlsTeam, TeamUnavailable, VmmArena

        sizes = {m["arena"]["size"] for m in metas.values() if m.get("arena")}
        supported = all(m.get("multicast", False) for m in metas.values())
        if len(sizes) != 1 or not supported or not device_info()["multicast"]:
            logger.warning("Agent %s: batch %s: no multicast team (arena sizes %s, multicast supported everywhere: %s)",
                           self.rank, batch.batch_id, sorted(sizes), supported)
            self._map_peer_arenas(batch, metas, all_ranks)
            return
        size = sizes.pop()
        mine = batch.arena
        if mine is None:
            mine = batch.scratch_arena = VmmArena(size, self.device, n_team=len(all_ranks))
            if mine.size != size:
                raise ValueError(f"Batch {batch.batch_id}: replicated arenas of {size} bytes are not a multiple of the "
                                 f"multicast granularity on this device ({mine.size} after rounding)")
        try:
            team = NvlsTeam(self.rank, all_ranks, mine, f"{self.namespace}_{batch.batch_id}_{batch.gen}".replace("/", "_"),
                            self._kv_all_gather(batch, all_ranks))
        except TeamUnavailable as e:
            # agreed on by every member: nobody is bound any more, the fan-out uses one peer store per replica.  A
            # producer still has to reach the consumers' arenas: it maps them like any other peer allocation.
            logger.warning("Agent %s: batch %s: no multicast team: %s", self.rank, batch.batch_id, e)
            if batch.scratch_arena is not None:
                batch.scratch_arena.close()
                batch.scratch_arena = None
            self._map_peer_arenas(batch, metas, all_ranks)
            return
        team.replicas = sorted(r for r in all_ranks if metas[r].get("arena"))
        for r in team.replicas:
            if r != self.rank:  # views of a consumer's arena resolve to the mapping the team made of it
                self._peer.adopt_mapping(tuple(metas[r]["arena"]["key"]), team.peer_va[r])
        batch.team = team

    def _map_peer_arenas(self, batch: BatchState, metas, all_ranks) -> None:
        """Without a team, views of another agent's worker arena still have to resolve to an address here: fetch the
        arena's file descriptor from that worker's socket and map it like the own worker's arena."""
        for r in all_ranks:
            info = metas[r].get("arena")
            if r == self.rank or not info:
                continue
            pid, device_index, va = info["key"]
            self._import_worker_arena({"pid": pid, "device_index": device_index, "va": va, "size": info["size"],
                                       "socket": info["socket"]})

    # ---- Transfer -----------------------------------------------------------------------------------
    def _store_barrier(self, key_prefix: str, ranks, round_no: int):
        """Round `round_no` of the barrier `key_prefix` over `ranks`; yields until everybody has arrived."""
        ranks = list(ranks)
        self.store.barrier_arrive(key_prefix, self.rank, round_no, len(ranks))
        while not self.store.barrier_wait(key_prefix, ranks, round_no):
            yield

    def _transfer_job(self, msg: Transfer):
        batch = self.batches.get(msg.batch_id)
        if batch is None:
            raise ValueError(f"Transfer for unknown batch: {msg.batch_id}")
        sending = msg.transfer_type == "send"
        signal_key = f"batch:{batch.batch_id}/state:transfer_signal"
        if (batch.send_exec if sending else batch.recv_exec) is None:
            partial_side = [p for p in batch.pair_names
                            if any(isinstance(x, Partial) for x in ((self.pairs[p].remote_placements if sending
                                                                      else self.pairs[p].local_placements) or ()))]
            why = (f"pair(s) {partial_side} would have a Partial target in that direction, which is not supported "
                   "(Partial is only valid as a source placement)" if partial_side else
                   "no executor could be built for that direction when the batch was registered")
            raise RuntimeError(f"Batch {batch.batch_id}: no {msg.transfer_type} plan: {why}.")
        if batch.in_flight:
            # an earlier transfer of this batch died between its rendezvous and its completion (a peer that never came,
            # a timeout): arrivals and epochs of the two sides no longer pair up, so a later rendezvous could let a
            # producer write before its consumer asked.  Only a fresh registration (a new generation) is safe.
            raise RuntimeError(f"Batch {batch.batch_id}: an earlier transfer did not complete; close the batch and "
                               "register it again")
        batch.in_flight = True
        batch.epoch += 1
        epoch = batch.epoch
        if sending and self.rank == batch.local_leader:
            # the epoch of the newest send is what receivers compare with the receives they have completed
            self.store.set(f"{batch.key}/state:send_epoch", str(epoch), component="global")
        all_ranks = sorted(set(batch.local_ranks) | set(batch.remote_ranks))
        # both sides meet here, like the reference's barrier on the batch group (agent.py:457)
        if batch.node_barrier is not None:
            batch.node_barrier.arrive()
            while not batch.node_barrier.passed():
                yield
        else:
            yield from self._store_barrier(f"{batch.key}/go", all_ranks, epoch)

        ex = batch.send_exec if sending else batch.recv_exec
        if sending and self.rank == batch.local_leader and ex in ("bucket", "plain"):
            self.store.set(signal_key, "1", component="global")  # the peer-to-peer path writes it while its copies run
        t0 = time.perf_counter()
        if ex == "bucket":
            bucket_comm(batch.send_buckets if sending else batch.recv_buckets)
        elif ex == "plain":
            yield from self._plain_transfer(batch, sending)
        else:
            yield from self._p2p_transfer(batch, ex, sending, epoch, signal_key)
        ms = (time.perf_counter() - t0) * 1e3
        self.state.put(f"batch:{batch.batch_id}/state:last_{msg.transfer_type}_ms", f"{ms:.3f}".encode())
        if not sending:
            batch.recv_done = epoch
            if self.rank == batch.local_leader:
                self.store.set(signal_key, "0", component="global")
        batch.in_flight = False
        logger.info("Agent %s: batch %s %s done in %.2f ms", self.rank, batch.batch_id, msg.transfer_type, ms)

    def _p2p_transfer(self, batch: BatchState, ex, sending: bool, epoch: int, signal_key: str | None = None):
        """Producers launch their copy table; every rank whose memory other ranks write (consumers) or read (Partial
        contributors) then waits until those ranks are done — on the device with the bounded flag wait, or through
        the KV store when another agent of the batch drives the same physical GPU."""
        from ..utils.profiling import nvtx_range

        shared_gpu = batch.shared_gpu
        stream = torch.cuda.current_stream(self.device)
        ex.epoch = epoch - 1
        ex.begin()
        done_prefix = f"{batch.key}/done"
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        with nvtx_range(f"etha.transfer.{'send' if sending else 'recv'}.launch"):
            if sending:
                ex.send(stream)
            waits_on_device = bool(ex._producers) and not shared_gpu
            if waits_on_device:
                ex.recv(stream, timeout_s=min(self.store_timeout, 60.0))
        e1.record(stream)
        if sending and signal_key and self.rank == batch.local_leader:
            # the reference's "1"/"0" key, kept for observers (`query_transfer_signal` reads the epoch instead, because a
            # late "0" of receive k can overwrite the "1" of send k+1); written while the copies run, off the critical path
            self.store.set(signal_key, "1", component="global")
            signal_key = None
        while not e1.query():
            yield
        ex.check()
        if sending:
            self.state.put(f"batch:{batch.batch_id}/state:last_send_device_ms", f"{e0.elapsed_time(e1):.3f}".encode())
            if batch.any_shared_gpu:
                # own copies are complete: published (as "done up to this transfer") before any wait, for the agents
                # that share a GPU with another one and therefore wait on the host
                self.store.mark_reached(done_prefix, self.rank, epoch)
                batch.wrote_done = True
        if ex._producers and shared_gpu:
            producers = list(ex._producers)
            while self.store.count_reached(done_prefix, producers, epoch) < len(producers):
                yield

    def _plain_transfer(self, batch: BatchState, sending: bool):
        """No layout was declared: tensor i goes whole to the same-index rank of the other side (reference
        fallback, src/etha/tensor_bus/agent.py:485-498)."""
        import torch.distributed as dist

        peer = batch.remote_ranks[sorted(batch.local_ranks).index(self.rank)]
        works = []
        for pair_name in batch.pair_names:
            for t in batch.pair_tensors[pair_name]:
                works.append(dist.isend(t, dst=peer) if sending else dist.irecv(t, src=peer))
        for w in works:
            w.wait()
        yield

    # ---- QueryStatus / CleanupBatch -----------------------------------------------------------------
    def _query_status_job(self, msg: QueryStatus):
        if msg.batch_id not in self.batches:
            raise ValueError(f"QueryStatus for unknown batch: {msg.batch_id}")
        if msg.state_name != "transfer_signal":
            raise ValueError(f"Invalid state name: {msg.state_name}")
        batch = self.batches[msg.batch_id]
        raw = self.store.try_get(f"{batch.key}/state:send_epoch", component="global")
        pending = int(raw.decode()) > batch.recv_done if raw else False
        self.state.set_signal(msg.batch_id, msg.state_name, pending)
        return
        yield

    def _cleanup_batch_job(self, msg: CleanupBatch):
        batch = self.batches.pop(msg.batch_id, None)
        if batch is None:
            logger.warning("Agent %s: cleanup for unknown batch %s", self.rank, msg.batch_id)
        else:
            self._drop_batch(batch)
        return
        yield

    def _drop_batch(self, batch: BatchState) -> None:
        """Release everything a registration holds: the executors' use of the peers' IPC mappings (a mapping no other
        batch uses is closed), the flag arrays, and the keys this agent wrote for this generation."""
        if self.device.type == "cuda" and (batch.send_exec is not None or batch.recv_exec is not None):
            torch.cuda.synchronize(self.device)  # nothing of this batch may still be in flight
        for ex in (batch.send_exec, batch.recv_exec):
            if hasattr(ex, "close"):
                ex.close()
        batch.send_exec = batch.recv_exec = None
        batch.send_buckets = batch.recv_buckets = None
        if batch.node_barrier is not None:
            batch.node_barrier.close()
            batch.node_barrier = None
        if batch.team is not None:  # leave the multicast team (unmap, unbind) before any arena goes away
            batch.team.close()
            batch.team = None
        if batch.scratch_arena is not None:
            batch.scratch_arena.close()
            batch.scratch_arena = None
        batch.arena = None  # an imported worker arena stays mapped for the next registration (closed with the agent)
        for k in batch.team_keys:
            self.store.delete(k)
        batch.team_keys.clear()
        if batch.flags and self._peer is not None:
            self._peer.forget(batch.flags.values())
        batch.flags = None
        batch.pair_tensors.clear()
        batch.keepalive.clear()
        if batch.key:
            self.store.delete(f"{batch.key}/rank:{self.rank}/meta")
            self.store.barrier_forget(f"{batch.key}/go", self.rank)
            if batch.wrote_done:
                self.store.delete(f"{batch.key}/done/rank:{self.rank}")
            if self.rank == batch.local_leader:
                self.store.delete(f"{batch.key}/state:send_epoch", component="global")
        self.state.delete(f"batch:{batch.batch_id}/state:transfer_signal")
        for d in ("send", "recv"):
            self.state.delete(f"batch:{batch.batch_id}/state:last_{d}_ms")
        self.state.delete(f"batch:{batch.batch_id}/state:last_send_device_ms")
        self.state.delete(f"batch:{batch.batch_id}/state:multicast_ops")
