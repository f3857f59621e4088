"""Device-resident copy table: built once per registered batch, launched once per transfer.

`CopyTable.add*` collect strided-box copies (optionally converting, fanning out to several
destinations or collapsing several Partial sources); `finalize()` packs them with the native packer,
splits them into the two kernel classes and uploads them; `launch()` issues at most two persistent
kernels on the given stream and, when asked, publishes an epoch to the consumers' flags from the
last CTA.  Nothing here allocates or touches the host during `launch()`.

The reference does this work per chunk and per transfer in Python (`Chunk.prepare`/`Bucket.prepare`/
`finalize`, src/etha/comm/ir.py:101-141,229-310).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from . import lib as L

_DT_CODE = {torch.float32: L.DT_F32, torch.bfloat16: L.DT_BF16, torch.float16: L.DT_F16}

DEFAULT_TILE_BYTES = 64 * 1024

# kernels launched by CopyTable.launch in this process (benchmarks report it)
LAUNCH_COUNT = [0]
# copy-engine copies enqueued by CopyTable.launch in this process (not kernels; reported separately)
DMA_COPY_COUNT = [0]


def dtype_code(dt: torch.dtype) -> int:
    return _DT_CODE.get(dt, L.DT_RAW)


@dataclass
class SliceRef:
    """A strided box in some GPU's memory: address of element [0,...,0], element strides, allocation bounds."""

    ptr: int
    strides: tuple[int, ...]
    dtype: torch.dtype
    lo: int = 0  # allocation [lo, hi) the box must stay inside (0, 0 = unchecked)
    hi: int = 0

    @staticmethod
    def of(view: torch.Tensor) -> "SliceRef":
        st = view.untyped_storage()
        base = st.data_ptr()
        return SliceRef(view.data_ptr(), tuple(view.stride()), view.dtype, base, base + st.nbytes())


class _KernelSet:
    """Device arrays of the kernel classes for one set of ops."""

    def __init__(self):
        self.ops_dev: list[torch.Tensor | None] = [None, None]
        self.tiles_dev: list[torch.Tensor | None] = [None, None]
        self.tiles_rest_dev: torch.Tensor | None = None  # prefix sums of the fast ops the TMA kernel cannot run
        self.n_ops, self.n_tiles = [0, 0], [0, 0]
        self.n_bulk_ops = self.n_bulk_tiles = 0
        # streaming instances of the typed class: key -> (ops, tile prefix sums, number of ops, tiles)
        self.typed: dict[int, tuple[torch.Tensor, torch.Tensor, int, int]] = {}


class CopyTable:
    """`dma_min_bytes`: when set, a bit copy of at least that many bytes whose box is one run or the rows of a matrix,
    and which the caller marks `dma_ok` (its destination is on another GPU), is a candidate for the DMA engines: at
    `finalize()` the largest candidates, up to `dma_fraction` of the bytes the table delivers, become memcpy nodes
    of a CUDA graph (`dma_mode="graph"`) or asynchronous copies on `dma_streams` side streams
    (`dma_mode="streams"`); everything else is packed for the kernels.  At launch the copies run next to the
    kernels: the DMA engines write larger NVLink packets than SM stores can, and the kernels fill the gaps
    between consecutive DMA copies."""

    def __init__(self, device: torch.device | int | str, tile_bytes: int = DEFAULT_TILE_BYTES,
                 dma_min_bytes: int | None = None, dma_mode: str = "graph", dma_streams: int = 8,
                 dma_fraction: float = 1.0):
        self.device = torch.device(device) if not isinstance(device, torch.device) else device
        self.tile_bytes = int(tile_bytes)
        self.dma_min_bytes = dma_min_bytes
        self.dma_mode, self.dma_streams, self.dma_fraction = dma_mode, dma_streams, dma_fraction
        self._dma: list[L.DmaCopy] = []
        self._dma_candidates: list[tuple[int, int, list, tuple]] = []  # (bytes, position, copies, packed entry)
        self._dma_plan = None
        self.dma_bytes = 0
        self._lib = L.cuda_lib()
        self._op_size = self._lib.etha_sizeof_op()
        self._packed: list[tuple[int, int, bytes, bool, int]] = []  # (class, tiles, op bytes, TMA-capable, stream key)
        self.stream_typed = True  # conversions / collapses over simple boxes use the streaming kernel instances
        self.payload_bytes = 0  # bytes delivered (destination side, all replicas)
        self.read_bytes = 0
        self._final = False
        self._keepalive: list = []
        self.n_ops = [0, 0]
        self.n_tiles = [0, 0]
        # fast-class ops are kept in two groups: those the TMA kernel can run (uploaded first) and the rest
        self.n_bulk_ops = 0
        self.n_bulk_tiles = 0

    # ---- building ---------------------------------------------------------------------------
    def add(
        self,
        shape: Sequence[int],
        srcs: Sequence[SliceRef],
        dsts: Sequence[SliceRef],
        reduce_sizes: Sequence[int] = (),
        reduce_ops: Sequence[str] = (),
        multimem: bool = False,
        dma_ok: bool = False,
    ) -> None:
        """One op: `srcs` (1, or a Partial family in family order) -> every slice of `dsts`."""
        if self._final:
            raise RuntimeError("table already finalized")
        if len(shape) > 8:
            raise ValueError("at most 8 dims")
        if len(srcs) > L.MAX_SRC:
            raise ValueError(f"at most {L.MAX_SRC} Partial contributors per cell are supported on the device")
        if len(reduce_sizes) > 2:
            raise ValueError("at most two Partial mesh dims are supported on the device")
        src0 = srcs[0]
        for s in srcs[1:]:
            if s.strides != src0.strides or s.dtype != src0.dtype:
                raise ValueError("Partial contributors must share strides and dtype")
        # group destinations by (strides, dtype): one op per group of at most MAX_DST
        groups: dict[tuple, list[SliceRef]] = {}
        for d in dsts:
            groups.setdefault((d.strides, d.dtype), []).append(d)
        numel = int(np.prod(shape)) if len(shape) else 1
        for (dstrides, ddtype), members in groups.items():
            for k in range(0, len(members), L.MAX_DST):
                part = members[k : k + L.MAX_DST]
                spec = L.OpSpec()
                spec.ndim = len(shape)
                for i, n in enumerate(shape):
                    spec.shape[i] = int(n)
                    spec.src_stride[i] = int(src0.strides[i])
                    spec.dst_stride[i] = int(dstrides[i])
                spec.src_itemsize, spec.dst_itemsize = src0.dtype.itemsize, ddtype.itemsize
                spec.src_dtype, spec.dst_dtype = dtype_code(src0.dtype), dtype_code(ddtype)
                if spec.src_dtype == L.DT_RAW and spec.dst_dtype == L.DT_RAW and src0.dtype != ddtype:
                    raise ValueError(f"no conversion from {src0.dtype} to {ddtype}")
                spec.nsrc, spec.ndst = len(srcs), len(part)
                for i, s in enumerate(srcs):
                    spec.src[i], spec.src_lo[i], spec.src_hi[i] = s.ptr, s.lo, s.hi
                for i, d in enumerate(part):
                    spec.dst[i], spec.dst_lo[i], spec.dst_hi[i] = d.ptr, d.lo, d.hi
                sizes = list(reduce_sizes) or [len(srcs)]
                ops = list(reduce_ops) or ["sum"]
                spec.red_size[0], spec.red_size[1] = sizes[0], (sizes[1] if len(sizes) > 1 else 1)
                spec.red_op[0] = L.RED_CODES[ops[0]]
                spec.red_op[1] = L.RED_CODES[ops[1]] if len(ops) > 1 else 0
                spec.flags = L.FLAG_MULTIMEM if multimem else 0
                spec.tile_bytes = self.tile_bytes
                buf = C.create_string_buffer(self._op_size)
                err = C.create_string_buffer(512)
                rc = self._lib.etha_pack_op(C.byref(spec), buf, err, 512)
                if rc != 0:
                    raise ValueError(f"cannot pack op ({rc}): {err.value.decode(errors='replace')}")
                tiles = self._lib.etha_op_tiles(buf)
                if tiles:
                    cls = self._lib.etha_op_class(buf)
                    tma = cls == 0 and bool(self._lib.etha_op_bulk_ok(buf))
                    skey = self._lib.etha_op_stream_key(buf) if (cls == 1 and self.stream_typed) else 0
                    entry = (cls, tiles, buf.raw, tma, skey)
                    self._packed.append(entry)
                    if dma_ok and self.dma_min_bytes is not None and numel * ddtype.itemsize >= self.dma_min_bytes:
                        out = (L.DmaCopy * L.MAX_DST)()
                        n = self._lib.etha_op_dma_copies(buf, out)
                        if n > 0:
                            copies = []
                            for j in range(n):
                                c = L.DmaCopy()
                                C.memmove(C.byref(c), C.byref(out[j]), C.sizeof(L.DmaCopy))
                                copies.append(c)
                            self._dma_candidates.append((numel * ddtype.itemsize * n, len(self._packed) - 1, copies, entry))
                self.payload_bytes += numel * ddtype.itemsize * len(part)
        self.read_bytes += numel * src0.dtype.itemsize * len(srcs)

    def add_copy(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """Local convenience: copy (and convert) `src` view into `dst` view of the same shape."""
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"shape mismatch {tuple(src.shape)} vs {tuple(dst.shape)}")
        self._keepalive += [src, dst]
        self.add(tuple(src.shape), [SliceRef.of(src)], [SliceRef.of(dst)])

    def add_reduce(self, srcs: Sequence[torch.Tensor], dst: torch.Tensor, sizes: Sequence[int], ops: Sequence[str]) -> None:
        self._keepalive += list(srcs) + [dst]
        self.add(tuple(dst.shape), [SliceRef.of(s) for s in srcs], [SliceRef.of(dst)], sizes, ops)

    # ---- upload -----------------------------------------------------------------------------
    def _upload(self, packed) -> "_KernelSet":
        """Device arrays of one set of packed ops, split into the kernel classes."""
        ks = _KernelSet()

        def prefix(tiles):
            starts = np.zeros(len(tiles) + 1, dtype=np.uint64)
            np.cumsum(tiles, out=starts[1:])
            if starts[-1] >= 2**32:
                raise ValueError("too many tiles in one table")
            return starts

        def to_dev(starts):
            return torch.from_numpy(starts.astype(np.uint32).view(np.int32).copy()).to(self.device)

        keys = list(dict.fromkeys(k for c, _, _, _, k in packed if c == 1 and k))
        for key in keys:
            members = [(t, raw) for c, t, raw, _, k in packed if c == 1 and k == key]
            starts = prefix([t for t, _ in members])
            blob = np.frombuffer(b"".join(raw for _, raw in members), dtype=np.uint8)
            ks.typed[key] = (torch.from_numpy(blob.copy()).to(self.device), to_dev(starts), len(members), int(starts[-1]))
        for cls in (0, 1):
            members = [(t, raw, tma) for c, t, raw, tma, k in packed if c == cls and not (c == 1 and k)]
            if cls == 0:  # stable split: TMA-capable ops first, relative order kept inside both groups
                members = [m for m in members if m[2]] + [m for m in members if not m[2]]
                ks.n_bulk_ops = sum(1 for m in members if m[2])
                ks.n_bulk_tiles = sum(m[0] for m in members if m[2])
            ks.n_ops[cls] = len(members)
            if not members:
                continue
            starts = prefix([t for t, _, _ in members])
            ks.n_tiles[cls] = int(starts[-1])
            blob = np.frombuffer(b"".join(raw for _, raw, _ in members), dtype=np.uint8)
            ks.ops_dev[cls] = torch.from_numpy(blob.copy()).to(self.device)
            ks.tiles_dev[cls] = to_dev(starts)
            if cls == 0 and 0 < ks.n_bulk_ops < len(members):
                ks.tiles_rest_dev = to_dev(prefix([t for t, _, _ in members[ks.n_bulk_ops:]]))
        return ks

    def _select_dma(self) -> set[int]:
        """Positions (in `_packed`) of the ops handed to the DMA engines: the largest candidates first, as long as the
        byte budget `dma_fraction x delivered bytes` is not exceeded (a candidate that does not fit is skipped, smaller
        ones may still fit).  Their copies are queued in table order, so the producers' rotation is kept."""
        budget = self.dma_fraction * self.payload_bytes
        taken: set[int] = set()
        for nbytes, pos, _copies, _ in sorted(self._dma_candidates, key=lambda c: (-c[0], c[1])):
            if self.dma_bytes + nbytes > budget:
                continue
            taken.add(pos)
            self.dma_bytes += nbytes
        for _nbytes, pos, copies, _ in self._dma_candidates:
            if pos in taken:
                self._dma += copies
        return taken

    def finalize(self, sm_count: int | None = None) -> "CopyTable":
        if self._final:
            return self
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sm_count = sm_count
        taken = self._select_dma()
        # two kernel sets share this table: every op (kernels only), and what is left next to the DMA copies
        self._all = self._upload(self._packed)
        self._rest = self._upload([e for i, e in enumerate(self._packed) if i not in taken]) if taken else self._all
        typed_ops = sum(v[2] for v in self._all.typed.values())
        typed_tiles = sum(v[3] for v in self._all.typed.values())
        # [fast class, typed + general]: the streaming instances count with the general class they were taken from
        self.n_ops = [self._all.n_ops[0], self._all.n_ops[1] + typed_ops]
        self.n_tiles = [self._all.n_tiles[0], self._all.n_tiles[1] + typed_tiles]
        self.n_typed_ops = typed_ops
        self.n_bulk_ops, self.n_bulk_tiles = self._all.n_bulk_ops, self._all.n_bulk_tiles
        self._dma_candidates = []
        self._sync = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._packed = []
        if self._dma:
            arr = (L.DmaCopy * len(self._dma))(*self._dma)
            plan = C.c_void_p()
            with torch.cuda.device(self.device):
                L.check(self._lib.etha_dma_plan_create(arr, len(self._dma), 1 if self.dma_mode == "graph" else 0,
                                                       self.dma_streams, C.byref(plan)), "dma plan")
            self._dma_plan = plan
        self._final = True
        return self

    def __del__(self):
        plan, self._dma_plan = getattr(self, "_dma_plan", None), None
        if plan:
            try:
                self._lib.etha_dma_plan_destroy(plan)
            except Exception:
                pass

    @property
    def n_dma_copies(self) -> int:
        return len(self._dma)

    @property
    def empty(self) -> bool:
        return self.n_tiles[0] + self.n_tiles[1] == 0

    def device_buffers(self) -> list[torch.Tensor]:
        """Every device array a launch reads (callers that drop the table right after a launch tie these to the stream)."""
        out = [self._sync]
        for ks in {id(self._all): self._all, id(self._rest): self._rest}.values():
            out += [b for b in (*ks.ops_dev, *ks.tiles_dev, ks.tiles_rest_dev) if b is not None]
            for ops_t, tiles_t, _, _ in ks.typed.values():
                out += [ops_t, tiles_t]
        return out

    # ---- launch -----------------------------------------------------------------------------
    def launch(
        self,
        stream: torch.cuda.Stream | None = None,
        signals: torch.Tensor | None = None,
        epoch: int = 0,
        ctas_per_sm: int = 2,
        bulk: bool = False,
        dma: bool | None = None,
    ) -> None:
        """Enqueue the table on `stream`. `signals`: int64 device tensor of flag addresses to publish `epoch` to.
        `bulk`: TMA ring kernel instead of the LD/ST kernel for the 16-byte bit copies; `dma=False`: every copy by
        the kernels even if the table holds a DMA plan."""
        if not self._final:
            self.finalize()
        s = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        n_sig = 0 if signals is None else signals.numel()
        sig_ptr = 0 if signals is None else signals.data_ptr()
        dma = self._dma_plan is not None and dma is not False
        ks = self._rest if dma else self._all
        # launches of this transfer: (kernel, ops, tile prefix sums, number of ops, tiles)
        plan = []
        if ks.n_tiles[0]:
            ops0, tiles0 = ks.ops_dev[0].data_ptr(), ks.tiles_dev[0].data_ptr()
            if bulk and ks.n_bulk_tiles:
                plan.append(("bulk", ops0, tiles0, ks.n_bulk_ops, ks.n_bulk_tiles))
                rest = ks.n_ops[0] - ks.n_bulk_ops
                if rest:
                    plan.append(("fast", ops0 + ks.n_bulk_ops * self._op_size, ks.tiles_rest_dev.data_ptr(), rest,
                                 ks.n_tiles[0] - ks.n_bulk_tiles))
            else:
                plan.append(("fast", ops0, tiles0, ks.n_ops[0], ks.n_tiles[0]))
        for key, (ops_t, tiles_t, n, tiles) in ks.typed.items():
            plan.append((key, ops_t.data_ptr(), tiles_t.data_ptr(), n, tiles))
        if ks.n_tiles[1]:
            plan.append(("general", ks.ops_dev[1].data_ptr(), ks.tiles_dev[1].data_ptr(), ks.n_ops[1], ks.n_tiles[1]))
        if not plan or dma:
            # with DMA copies in the transfer: the copies start on side streams, the kernels run next to them on
            # the caller's stream without a signal, the stream then waits for the copies and the flags go last
            if dma:
                L.check(self._lib.etha_dma_plan_launch(self._dma_plan, s), "dma launch")
                DMA_COPY_COUNT[0] += len(self._dma)
            for kernel, ops_ptr, tiles_ptr, n_ops, n_tiles in plan:
                self._launch_kernel(kernel, ops_ptr, tiles_ptr, n_ops, n_tiles, ctas_per_sm, (sig_ptr, 0, 0, 0), s)
            if dma:
                L.check(self._lib.etha_dma_plan_join(self._dma_plan, s), "dma join")
            if n_sig:
                L.check(self._lib.etha_set_flags(sig_ptr, n_sig, epoch & 0xFFFFFFFF, s), "set_flags")
                LAUNCH_COUNT[0] += 1
            return
        for i, (kernel, ops_ptr, tiles_ptr, n_ops, n_tiles) in enumerate(plan):
            last = i == len(plan) - 1
            sig = (sig_ptr, n_sig, epoch & 0xFFFFFFFF, 1) if (last and n_sig) else (sig_ptr, 0, epoch & 0xFFFFFFFF, 0)
            self._launch_kernel(kernel, ops_ptr, tiles_ptr, n_ops, n_tiles, ctas_per_sm, sig, s)

    def _launch_kernel(self, kernel, ops_ptr, tiles_ptr, n_ops, n_tiles, ctas_per_sm, sig, s) -> None:
        if kernel == "bulk":
            rc = self._lib.etha_m2n_bulk_launch(ops_ptr, tiles_ptr, n_ops, min(n_tiles, self.sm_count),
                                                self._sync.data_ptr(), *sig, s)
        elif isinstance(kernel, int):  # key of a streaming instance
            grid = min(n_tiles, self.sm_count * self._lib.etha_stream_ctas_per_sm())
            rc = self._lib.etha_m2n_typed_launch(ops_ptr, tiles_ptr, n_ops, kernel, grid, self._sync.data_ptr(), *sig, s)
        else:
            general = kernel == "general"
            # the fast kernel is compiled for two 512-thread CTAs per SM; the general one reports its own occupancy
            per_sm = max(ctas_per_sm, self._lib.etha_general_ctas_per_sm()) if general else ctas_per_sm
            rc = self._lib.etha_m2n_launch(ops_ptr, tiles_ptr, n_ops, int(general), min(n_tiles, self.sm_count * per_sm), 0,
                                           self._sync.data_ptr(), *sig, s)
        L.check(rc, "m2n launch")
        LAUNCH_COUNT[0] += 1

    def error_word(self) -> int:
        """Device-side error word of the last launches (synchronizes)."""
        return int(self._sync[1].item()) if (self.n_tiles[0] + self.n_tiles[1]) else 0
