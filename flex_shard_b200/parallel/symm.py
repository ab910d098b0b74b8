"""Symmetric memory over NVLink and the collectives built on it.

``SymmRegion`` is one symmetric allocation (same size on every rank of a group, every rank
maps every peer's copy) carved into a flag area and a payload area. ``SymmComm`` is a drop-in
``Comm`` whose all-gather and reduce-scatter are this library's own peer-memory kernels
(``csrc/comm.cu``): ranks publish epoch flags, consumers pull remote rows with plain loads.
The reduce-scatter sums the W rows in rank order, so its result is deterministic and equal
on every run (NCCL's order depends on the algorithm it picks).

The allocation and the exchange of mappings use ``torch.distributed._symmetric_memory``
(CUDA VMM handles over the process group's store); nothing else of it is used.

Parity: this is the native counterpart of the reference's symmetric-memory transport
(``custom_placements/owner_rows_transport.py:182-244``); on one NVSwitch domain every peer is
one hop away, so its host/relay planning reduces to direct peer access.
"""
from __future__ import annotations

import os
import weakref

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import count_launch
from .comm import Comm, ReducePlan

FLAG_BYTES = 64 * 1024          # 1024 slots x 16 ranks x 4 bytes
MAX_RANKS = 16
DEFAULT_MAX_POLLS = 20_000_000  # x >=200 ns back-off: several seconds before a wait gives up
_declared = False


def _ensure():
    global _declared
    if _declared:
        return
    c = ctypes
    vp, i32, i64, u32, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_uint, c.c_float
    _lib.declare("fsb_comm_signal", [vp, i32, i32, u32, vp])
    _lib.declare("fsb_comm_wait", [vp, i32, u32, u32, vp, vp])
    _lib.declare("fsb_comm_gather_pull", [vp, i32, i32, vp, i32, u32, u32, vp, vp])
    _lib.declare("fsb_comm_reduce_rows", [vp, i32, i64, f32, vp, vp, i32, vp, vp, f32, f32, f32, f32, f32, i32,
                                          vp, u32, u32, vp, vp])
    _lib.declare("fsb_comm_reduce_rows_mc", [c.c_ulonglong, i32, i64, f32, vp, vp, i32, vp, vp, f32, f32, f32, f32,
                                             f32, i32, vp, u32, u32, vp, vp])
    _lib.declare("fsb_comm_wait_many", [vp, vp, i32, i32, u32, vp, vp])
    _lib.declare("fsb_comm_copy_segments_dma", [vp, vp, vp, i32, vp])
    _declared = True


CANARY_BYTES, CANARY_VALUE = 256, 0xA5
_canary_regions: list = []


def _install_canary_hook() -> None:
    if check_canaries not in _lib._check_hooks:
        _lib._check_hooks.append(check_canaries)


def check_canaries() -> None:
    """Debug mode only: raise if the guard bytes behind any live symmetric region's payload were overwritten."""
    alive = []
    for ref in _canary_regions:
        reg = ref()
        if reg is None:
            continue
        alive.append(ref)
        if not reg.canary_intact():
            raise RuntimeError(f"guard bytes behind the payload of {reg.name} were overwritten: something wrote past "
                               f"the end of its {reg.payload_bytes} payload bytes")
    _canary_regions[:] = alive


_warned_lazy = False


def _warn_if_lazy_loading() -> None:
    """Peer waits and lazy kernel loading do not mix (see ``fsb_module_loading_mode``): say so once."""
    global _warned_lazy
    if _warned_lazy:
        return
    _warned_lazy = True
    try:
        fn = _lib.load().fsb_module_loading_mode
        fn.argtypes, fn.restype = [], ctypes.c_int
        mode = fn()
    except Exception:
        return
    if mode == 2:
        import warnings

        warnings.warn(
            "CUDA loads kernels lazily in this process (CUDA was initialised before flex_shard_b200 was imported, or "
            "CUDA_MODULE_LOADING=LAZY is set). The first launch of a kernel can then stall behind a kernel that "
            "waits for a peer, and two ranks can block each other until the device-side waits time out. Set "
            "CUDA_MODULE_LOADING=EAGER in the environment of every rank.", RuntimeWarning, stacklevel=3)


class SymmRegion:
    """A symmetric buffer: ``[flags (64 KB) | payload]`` on every rank, peers mapped."""

    _count = 0

    def __init__(self, group: dist.ProcessGroup, payload_bytes: int, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        _ensure()
        _warn_if_lazy_loading()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"symmetric regions support up to {MAX_RANKS} ranks")
        self.device = device
        self.payload_bytes = (payload_bytes + 255) // 256 * 256
        # debug mode (FSB200_CANARY=1): 256 bytes of a fixed pattern behind the payload; check_canaries() (called by
        # ops.check_status) raises if a kernel or a peer wrote past the end of the payload
        self.canary_bytes = CANARY_BYTES if os.environ.get("FSB200_CANARY", "0") == "1" else 0
        total = FLAG_BYTES + self.payload_bytes + self.canary_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[:FLAG_BYTES].zero_()
        if self.canary_bytes:
            self.buf[FLAG_BYTES + self.payload_bytes:].fill_(CANARY_VALUE)
            _canary_regions.append(weakref.ref(self))
            _install_canary_hook()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.peer_base = [int(p) for p in self.handle.buffer_ptrs]
        # address of the same buffer in the NVSwitch multicast mapping (0: not available or switched off);
        # multimem loads through it return the sum over all ranks' copies, added inside the switch
        self.mc_base = 0
        if os.environ.get("FSB200_MULTIMEM", "1") != "0":
            try:
                self.mc_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            except Exception:
                self.mc_base = 0
        self.epoch = 0   # gather epoch of a region that holds a bucket's resident storage
        # name shown when a wait on one of this region's flags runs out (users may set a better one: .name = ...)
        self._name = [f"symmetric region #{SymmRegion._count} ({self.payload_bytes} payload bytes)"]
        SymmRegion._count += 1
        box = self._name
        _lib.register_flag_range(self.peer_base[self.rank], FLAG_BYTES, lambda: box[0], MAX_RANKS * 4)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone signals
        self.max_polls = DEFAULT_MAX_POLLS

    @property
    def name(self) -> str:
        return self._name[0]

    @name.setter
    def name(self, value: str) -> None:
        self._name[0] = value

    # ---- addressing
    @property
    def payload(self) -> torch.Tensor:
        return self.buf[FLAG_BYTES:FLAG_BYTES + self.payload_bytes]

    def canary_intact(self) -> bool:
        if not self.canary_bytes:
            return True
        tail = self.buf[FLAG_BYTES + self.payload_bytes:]
        return bool((tail == CANARY_VALUE).all())

    def peer_payload_addr(self, r: int, offset: int = 0) -> int:
        return self.peer_base[r] + FLAG_BYTES + offset

    def mc_payload_addr(self, offset: int = 0) -> int:
        return self.mc_base + FLAG_BYTES + offset if self.mc_base else 0

    def flag_row_addr(self, r: int, slot: int) -> int:
        return self.peer_base[r] + slot * MAX_RANKS * 4

    # ---- flags
    def signal(self, slot: int, epoch: int) -> None:
        rows = (ctypes.c_ulonglong * self.world)(*[self.flag_row_addr(r, slot) for r in range(self.world)])
        rc = _lib.load().fsb_comm_signal(rows, self.rank, self.world, epoch & 0xFFFFFFFF,
                                         _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_signal")
        count_launch()

    def wait(self, slot: int, epoch: int) -> None:
        rc = _lib.load().fsb_comm_wait(self.flag_row_addr(self.rank, slot), self.world, epoch & 0xFFFFFFFF,
                                       self.max_polls, _lib.status_word(self.device).data_ptr(),
                                       _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_wait")
        count_launch()


_SEG = 32  # bytes per descriptor


def _pack_descs(segments, device) -> torch.Tensor:
    """(src_addr, dst_addr, nbytes) triples -> device tensor of SegDesc records."""
    import struct

    raw = bytearray()
    for src, dst, n in segments:
        raw += struct.pack("<QQqii", src, dst, n, 0, 0)
    host = torch.frombuffer(raw, dtype=torch.uint8).clone().pin_memory()
    return host.to(device, non_blocking=True)


class SymmComm(Comm):
    """``Comm`` whose all-gather / reduce-scatter run on peer memory instead of NCCL.

    Send data is staged into the symmetric payload (one local copy), published with an epoch
    flag, and pulled by every consumer. Separate staging areas and flag slots serve gathers and
    reductions, which run on different streams.
    """

    SLOT_AG_READY, SLOT_AG_DONE, SLOT_RS_READY, SLOT_RS_DONE = 0, 1, 2, 3

    def __init__(self, group, rank, world_size, device, ag_bytes: int = 0, rs_bytes: int = 0):
        super().__init__(group, rank, world_size, device)
        self._ag: SymmRegion | None = None
        self._rs: SymmRegion | None = None
        self._ag_epoch = 0
        self._rs_epoch = 0
        self._ag_hint, self._rs_hint = ag_bytes, rs_bytes
        self._desc_cache: dict = {}
        # weight gradients go straight into the owners' memory (FSB200_FUSED_REDUCE=0: gradients are
        # written locally in reduce-scatter layout and the owners pull and sum them)
        self.fused_reduce = os.environ.get("FSB200_FUSED_REDUCE", "1") != "0"
        self._grad_ring: SymmGradRing | None = None
        # buckets whose byte storage lives in symmetric memory: payload address -> region. Their gathers
        # read the peers' storage in place (no staging copy, no shared staging region to serialise on).
        self._resident: dict[int, SymmRegion] = {}
        self._unfenced: set[int] = set()
        self.resident_storage = os.environ.get("FSB200_RESIDENT", "1") != "0"
        self.stats = {"resident_gathers": 0, "staged_gathers": 0, "dma_gathers": 0, "multimem_reduces": 0,
                      "peer_reduces": 0}
        # in-switch gradient sum (multimem.ld_reduce): "1" switches it on. Off by default: measured on 2 and 4
        # ranks the rank-order peer loads are faster (0.79 / 1.05 ms against 1.38 / 1.31 ms for a Llama layer
        # bucket; the switch delivers reduced rows at about 670 GB/s whatever the rank count) and their sum has a
        # fixed, documented order
        self.multimem_reduce = os.environ.get("FSB200_MULTIMEM_REDUCE", "0") == "1"
        # "dma": segment gathers are issued as copy-engine copies (no SM time); "sm": the pull kernel
        self.gather_engine = os.environ.get("FSB200_GATHER", "dma")

    @classmethod
    def from_mesh(cls, mesh, **kw) -> "SymmComm":
        from .comm import mesh_group

        g, rank, ws, dev = mesh_group(mesh)
        return cls(g, rank, ws, dev, **kw)

    def new_like(self) -> "SymmComm":
        return SymmComm(self.group, self.rank, self.world_size, self.device, self._ag_hint, self._rs_hint)

    def _region(self, which: str, nbytes: int) -> SymmRegion:
        cur = self._ag if which == "ag" else self._rs
        if cur is None or cur.payload_bytes < nbytes:
            hint = self._ag_hint if which == "ag" else self._rs_hint
            size = max(nbytes, hint)
            if cur is not None:
                # the peers may still be reading the old region (their pull of the last epoch): wait for
                # every rank's "done" flag of that epoch before the memory goes away
                last = self._ag_epoch if which == "ag" else self._rs_epoch
                if last > 0:
                    cur.wait(self.SLOT_AG_DONE if which == "ag" else self.SLOT_RS_DONE, last)
                torch.cuda.synchronize(self.device)
                _lib.check_status(self.device)   # a peer that never signalled "done" may still read the old region: raise
                size = max(size, 2 * cur.payload_bytes)
            cur = SymmRegion(self.group, size, self.device)
            cur.name = ("all-gather staging region (slots: 0 ready, 1 done)" if which == "ag" else
                        "reduce-scatter staging region (slots: 2 ready, 3 done)") + f", {size} bytes"
            if which == "ag":
                self._ag, self._ag_epoch = cur, 0
            else:
                self._rs, self._rs_epoch = cur, 0
            self._desc_cache.clear()
        return cur

    # ------------------------------------------------------------------ resident bucket storage
    def alloc_storage(self, nbytes: int) -> torch.Tensor | None:
        """Byte storage for one bucket inside a symmetric region of its own (a collective call: every rank
        of the group allocates the same size in the same order). Returns None when switched off."""
        if not self.resident_storage or self.world_size == 1 or nbytes <= 0:
            return None
        reg = SymmRegion(self.group, nbytes, self.device)
        reg.name = f"resident bucket storage #{len(self._resident)} ({nbytes} bytes; slots: 0 gather ready, 1 gather done)"
        buf = reg.payload[:nbytes]
        self._resident[buf.data_ptr()] = reg
        return buf

    def release_storage(self, buf: torch.Tensor) -> None:
        """Forget a resident storage (its bucket was laid out anew). The peers may have read it last in a
        backward that has ended on every rank before anyone re-lays out, so no wait is needed here; the
        memory goes back once the last tensor viewing it is gone."""
        ptr = buf.data_ptr()
        self._resident.pop(ptr, None)
        self._unfenced.discard(ptr)
        # cached descriptor tables are keyed by the region object's identity, which a later region may reuse
        self._desc_cache.clear()

    def _resident_region(self, inp: torch.Tensor):
        reg = self._resident.get(inp.data_ptr())
        if reg is not None and inp.numel() * inp.element_size() <= reg.payload_bytes:
            return reg
        return None

    def wait_readers_done(self, buf: torch.Tensor) -> None:
        """Enqueue a wait until every peer has finished its latest gather out of the resident buffer ``buf``
        (for buffers that are rewritten between gathers, such as a quantised payload row)."""
        reg = self._resident.get(buf.data_ptr())
        if reg is not None and reg.epoch > 0:
            reg.wait(self.SLOT_AG_DONE, reg.epoch)
            self._unfenced.discard(buf.data_ptr())

    def fence_resident(self) -> None:
        """Enqueue, on the current stream, a wait until every peer has finished reading this rank's
        resident storages (their pulls of the latest gather epoch). Work queued afterwards, such as an
        optimizer step, may then overwrite the shards. One launch for all buckets."""
        regs = [self._resident[k] for k in self._unfenced if k in self._resident]
        self._unfenced.clear()
        regs = [r for r in regs if r.epoch > 0]
        if not regs:
            return
        rows = (ctypes.c_ulonglong * len(regs))(*[r.flag_row_addr(self.rank, self.SLOT_AG_DONE) for r in regs])
        eps = (ctypes.c_uint * len(regs))(*[r.epoch & 0xFFFFFFFF for r in regs])
        rc = _lib.load().fsb_comm_wait_many(rows, eps, len(regs), self.world_size, regs[0].max_polls,
                                            _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_wait_many")
        count_launch()

    def grad_ring(self, entry_bytes: int) -> SymmGradRing:
        if self._grad_ring is None or self._grad_ring.entry_bytes < entry_bytes:
            if self._grad_ring is not None:
                torch.cuda.synchronize(self.device)
            self._grad_ring = SymmGradRing(self.group, self.device, entry_bytes)
        return self._grad_ring

    def scatter_to_peers(self, segments) -> None:
        """Copy (local src addr, peer dst addr, nbytes) segments with one kernel launch."""
        if not segments:
            return
        descs = _pack_descs(segments, self.device)
        n = max(s[2] for s in segments)
        rc = _lib.load().fsb_comm_gather_pull(descs.data_ptr(), len(segments), max(1, min(32, n // (64 * 1024))),
                                              None, self.world_size, 0, 0,
                                              _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_gather_pull")
        count_launch()

    def reduce_incoming(self, bucket: "PeerBucket", scale: float, out: torch.Tensor | None, adam: dict | None):
        """Owner side of the fused reduce-scatter: wait for every source's ``written`` flag, sum the W
        incoming rows in rank order (+ AdamW on the shard when ``adam`` is given), then release the entry."""
        ring, k, u, row = bucket.ring, bucket.k, bucket.use, bucket.row
        reg = ring.region
        W = self.world_size
        reg.signal(ring.SLOT_WRITTEN0 + k, u)
        a = adam or {}
        p = a.get("p")
        tail = (out.data_ptr() if out is not None else None,
                p.data_ptr() if p is not None else None, int(p is not None and p.dtype == torch.float32),
                a["m"].data_ptr() if adam else None, a["v"].data_ptr() if adam else None,
                a.get("lr", 0.0), a.get("beta1", 0.0), a.get("beta2", 0.0), a.get("eps", 0.0),
                a.get("weight_decay", 0.0), a.get("step", 1),
                reg.flag_row_addr(self.rank, ring.SLOT_WRITTEN0 + k), u, reg.max_polls,
                _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        mc_row = ring.mc_read_addr(self.rank, k, row) if (self.multimem_reduce and row % 4 == 0) else 0
        if mc_row:
            # pull layout: every rank wrote its contribution for this rank at the same offset of its own
            # entry, so one multimem load per 16 bytes returns the W-way sum (added in the switch)
            rc = _lib.load().fsb_comm_reduce_rows_mc(mc_row, W, row, scale, *tail)
            self.stats["multimem_reduces"] += 1
        else:
            self.stats["peer_reduces"] += 1
            rows = (ctypes.c_ulonglong * W)(*[ring.read_addr(self.rank, s, k, row) for s in range(W)])
            rc = _lib.load().fsb_comm_reduce_rows(rows, W, row, scale, *tail)
        _lib.check(rc, "fsb_comm_reduce_rows")
        count_launch()
        reg.signal(ring.SLOT_CONSUMED0 + k, u)

    # ------------------------------------------------------------------ all-gather
    def _publish(self, inp: torch.Tensor, nbytes: int, alloc_bytes: int):
        """Make this rank's send data readable by the peers and announce it; returns (region, epoch).
        Resident storage is read in place: the announcement alone orders the peers' pulls after whatever
        this stream did to the shard. Anything else is copied into the shared staging region first, once
        the peers are done with the region's previous payload."""
        reg = self._resident_region(inp) if nbytes else None
        if reg is not None:
            reg.epoch += 1
            e = reg.epoch
            self._unfenced.add(inp.data_ptr())
            self.stats["resident_gathers"] += 1
        else:
            self.stats["staged_gathers"] += 1
            reg = self._region("ag", alloc_bytes)  # same size on every rank
            self._ag_epoch += 1
            e = self._ag_epoch
            if e > 1:
                reg.wait(self.SLOT_AG_DONE, e - 1)      # peers finished reading the previous payload
            if nbytes:
                reg.payload[:nbytes].copy_(inp.view(torch.uint8).view(-1))
        reg.signal(self.SLOT_AG_READY, e)
        return reg, e

    def all_gather_into_tensor(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        if self.world_size == 1:
            return super().all_gather_into_tensor(out, inp)
        W = self.world_size
        nbytes = inp.numel() * inp.element_size()
        assert out.numel() * out.element_size() == W * nbytes and out.is_contiguous() and inp.is_contiguous()
        # one segment per rank: the same path (copy engines or pull kernel, resident or staged source) as a
        # gather into per-parameter buffers
        self.all_gather_segments(inp, [(r, 0, out.data_ptr() + r * nbytes, nbytes) for r in range(W)], alloc_bytes=nbytes)
        return None

    def all_gather_segments(self, inp: torch.Tensor, segments, alloc_bytes: int = 0) -> None:
        """All-gather whose destination is a list of segments: ``segments`` = (rank, source byte offset
        inside that rank's ``inp``, destination address, nbytes). One pull kernel moves every piece to
        its final place (e.g. straight into per-parameter buffers), so no gather buffer and no
        copy-out pass exist."""
        W = self.world_size
        nbytes = inp.numel() * inp.element_size()
        reg, e = self._publish(inp, nbytes, max(nbytes, alloc_bytes))
        key = ("seg", id(reg), tuple((r, o, d, n) for r, o, d, n in segments))
        if self.gather_engine == "dma":
            arrs = self._desc_cache.get(("dma",) + key)
            if arrs is None:
                # rank me reads peer me+1 first, then me+2, ...: the ranks do not all pull from the same peer at
                # once (the sort is stable, so the caller's order is kept within a peer)
                ordered = sorted((s for s in segments if s[3] > 0), key=lambda s: (s[0] - self.rank - 1) % W)
                live = [(reg.peer_payload_addr(r, o), d, n) for r, o, d, n in ordered]
                k = len(live)
                arrs = ((ctypes.c_ulonglong * k)(*[a for a, _, _ in live]), (ctypes.c_ulonglong * k)(*[d for _, d, _ in live]),
                        (ctypes.c_longlong * k)(*[n for _, _, n in live]), k)
                if len(self._desc_cache) < 4096:
                    self._desc_cache[("dma",) + key] = arrs
            reg.wait(self.SLOT_AG_READY, e)               # every peer has published this epoch
            rc = _lib.load().fsb_comm_copy_segments_dma(arrs[0], arrs[1], arrs[2], arrs[3], _lib.stream_ptr(self.device))
            _lib.check(rc, "fsb_comm_copy_segments_dma")
            self.stats["dma_gathers"] += 1
            reg.signal(self.SLOT_AG_DONE, e)
            return
        descs = self._desc_cache.get(key)
        if descs is None:
            descs = _pack_descs([(reg.peer_payload_addr(r, o), d, n) for r, o, d, n in segments], self.device)
            if len(self._desc_cache) < 4096:
                self._desc_cache[key] = descs
        biggest = max(n for _, _, _, n in segments)
        blocks = max(1, min(48, biggest // (128 * 1024)))
        rc = _lib.load().fsb_comm_gather_pull(descs.data_ptr(), len(segments), blocks,
                                              reg.flag_row_addr(self.rank, self.SLOT_AG_READY), W, e, reg.max_polls,
                                              _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_gather_pull")
        count_launch()
        reg.signal(self.SLOT_AG_DONE, e)

    def all_to_all_pull(self, recv: torch.Tensor, send: torch.Tensor, table_bytes) -> bool:
        """Uneven all-to-all as peer pulls. ``table_bytes[src][dst]``: bytes rank ``src`` sends to rank
        ``dst``, laid out in ``src``'s ``send`` in order of ``dst``; this rank's pieces land in ``recv`` in
        order of ``src``. Every rank passes the same table (it is what sizes the symmetric region).
        Returns False (nothing done) when a piece is not a multiple of 16 bytes: use NCCL then."""
        W, me = self.world_size, self.rank
        if any(n % 16 for row in table_bytes for n in row):
            return False
        segs, dst = [], 0
        for r in range(W):
            n = table_bytes[r][me]
            if n:
                segs.append((r, sum(table_bytes[r][:me]), recv.data_ptr() + dst, n))
            dst += n
        if not segs:
            # nothing to receive: still publish (the peers pull from this rank) with one empty descriptor.
            # Its address is never dereferenced; it must not come from the region, whose creation is a
            # collective step that has to happen once, inside all_gather_segments, at the agreed size.
            segs = [(me, 0, recv.data_ptr() if recv.numel() else 0, 0)]
        self.all_gather_segments(send, segs, alloc_bytes=max(max(sum(row) for row in table_bytes), 16))
        return True

    # ------------------------------------------------------------------ reduce-scatter
    def reduce_scatter_tensor(self, out: torch.Tensor, inp: torch.Tensor, plan: ReducePlan, async_op: bool = False):
        if self.world_size == 1 or inp.dtype != torch.float32 or out.numel() % 4 != 0:
            return super().reduce_scatter_tensor(out, inp, plan, async_op)
        W = self.world_size
        self._apply_plan_pre(inp, plan)
        n = out.numel()
        nbytes = inp.numel() * 4
        assert inp.numel() == W * n and out.dtype == torch.float32 and out.is_contiguous()
        reg = self._region("rs", nbytes)
        self._rs_epoch += 1
        e = self._rs_epoch
        if e > 1:
            reg.wait(self.SLOT_RS_DONE, e - 1)
        reg.payload[:nbytes].copy_(inp.view(torch.uint8).view(-1))
        reg.signal(self.SLOT_RS_READY, e)
        if plan.op == "avg":
            scale = 1.0 / W
        elif plan.op == "premul_sum":
            scale = float(plan.premul)
        else:
            scale = 1.0
        if plan.post_divide is not None:
            scale /= plan.post_divide
        rows = (ctypes.c_ulonglong * W)(*[reg.peer_payload_addr(r, self.rank * n * 4) for r in range(W)])
        rc = _lib.load().fsb_comm_reduce_rows(rows, W, n, scale, out.data_ptr(), None, 0, None, None,
                                              0.0, 0.0, 0.0, 0.0, 0.0, 1,
                                              reg.flag_row_addr(self.rank, self.SLOT_RS_READY), e, reg.max_polls,
                                              _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_reduce_rows")
        count_launch()
        reg.signal(self.SLOT_RS_DONE, e)
        return None


def _symm_reduce_scatter_list(self, out: torch.Tensor, inps, plan: ReducePlan):
    """Reduce rows of different lengths into their owners (``inps[r]`` is this rank's contribution to rank
    r's row, ``out`` this rank's reduced row): every rank lays its contributions back to back in the
    symmetric staging region (same offsets everywhere, since every rank knows every row length) and each
    owner sums its row out of all peers' regions in rank order, one kernel, no padding to a common length.
    The reverse direction of the owner-rows gather; the reference reduces such rows with one grouped NCCL
    reduce per rank (``custom_placements/utils.py:175-190``) or through its chunk transport
    (``custom_placements/owner_rows_transport.py:544-585``)."""
    W = self.world_size
    lens = [t.numel() for t in inps]
    if (W == 1 or out.dtype != torch.float32 or any(t.dtype != torch.float32 for t in inps)
            or any(n % 4 for n in lens)):
        return Comm.reduce_scatter_list(self, out, inps, plan)
    for t in inps:
        self._apply_plan_pre(t, plan)
    offs = [4 * sum(lens[:r]) for r in range(W)]
    total = 4 * sum(lens)
    reg = self._region("rs", max(total, 16))
    self._rs_epoch += 1
    e = self._rs_epoch
    if e > 1:
        reg.wait(self.SLOT_RS_DONE, e - 1)
    from ..ops.segments import run_segment_ops

    run_segment_ops([(reg.payload[o:o + 4 * t.numel()].view(torch.float32), t.reshape(-1))
                     for t, o in zip(inps, offs) if t.numel()])
    reg.signal(self.SLOT_RS_READY, e)
    scale = {"avg": 1.0 / W, "premul_sum": float(plan.premul or 1.0)}.get(plan.op, 1.0)
    if plan.post_divide is not None:
        scale /= plan.post_divide
    n = lens[self.rank]
    if n:
        rows = (ctypes.c_ulonglong * W)(*[reg.peer_payload_addr(r, offs[self.rank]) for r in range(W)])
        rc = _lib.load().fsb_comm_reduce_rows(rows, W, n, scale, out.data_ptr(), None, 0, None, None,
                                              0.0, 0.0, 0.0, 0.0, 0.0, 1,
                                              reg.flag_row_addr(self.rank, self.SLOT_RS_READY), e, reg.max_polls,
                                              _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_comm_reduce_rows")
        count_launch()
    else:
        reg.wait(self.SLOT_RS_READY, e)
    reg.signal(self.SLOT_RS_DONE, e)
    self.stats["owner_row_reduces"] = self.stats.get("owner_row_reduces", 0) + 1
    return None


SymmComm.reduce_scatter_list = _symm_reduce_scatter_list


class SymmGradRing:
    """Symmetric *incoming gradient* regions for the fused weight-gradient -> reduce-scatter path.

    Entry ``k`` on rank ``r`` holds ``[W source ranks][row]`` fp32: source ``s`` writes its
    contribution to ``r``'s shard of the bucket into row ``s`` (the weight-gradient GEMM's epilogue
    stores there directly over NVLink). ``written[k]`` flags say a source has finished a bucket,
    ``consumed[k]`` flags say the owner has reduced it and the entry may be overwritten.
    """

    SLOT_WRITTEN0, SLOT_CONSUMED0 = 16, 32

    def __init__(self, group, device, entry_bytes: int, entries: int | None = None):
        # Entries in flight: a bucket's backward may not start writing entry k before every peer has
        # reduced the bucket that used it `entries` buckets earlier. Two is the minimum for overlap; more
        # keep the compute stream from stalling on a peer whose reduction lags (W x 4 bytes/param each).
        entries = entries or int(os.environ.get("FSB200_RING_ENTRIES", "3"))
        self.entry_bytes = (entry_bytes + 255) // 256 * 256
        self.entries = entries
        self.region = SymmRegion(group, entries * self.entry_bytes, device)
        self.region.name = (f"gradient ring ({entries} entries of {self.entry_bytes} bytes; slots: "
                            f"{self.SLOT_WRITTEN0}+k written, {self.SLOT_CONSUMED0}+k consumed)")
        self.uses = [0] * entries
        self.count = 0
        self.pull = os.environ.get("FSB200_REDUCE_MODE", "pull") != "push"

    def acquire(self) -> tuple[int, int]:
        """Next entry and its use index; enqueues (on the current stream) the wait for every peer to
        have consumed the entry's previous use."""
        k = self.count % self.entries
        self.count += 1
        self.uses[k] += 1
        u = self.uses[k]
        if u > 1:
            self.region.wait(self.SLOT_CONSUMED0 + k, u - 1)
        return k, u

    def incoming_addr(self, owner: int, k: int, src: int, row_elems: int, elem_off: int = 0) -> int:
        return self.region.peer_payload_addr(owner, k * self.entry_bytes + (src * row_elems + elem_off) * 4)

    # Two ways to use an entry. "push": rank ``me`` stores its contribution for owner ``dst`` straight
    # into ``dst``'s entry (slot ``me``) over NVLink, the owner sums its own entry. "pull" (default): ``me``
    # writes all W contributions into its own entry (slot ``dst``), the owner reads slot ``dst`` of every
    # rank's entry over NVLink while it sums. Same memory, same flags; pull keeps the GEMM epilogue's
    # stores local (remote stores from the epilogue slowed the weight-gradient GEMMs by 20-50 %).
    def write_addr(self, me: int, dst: int, k: int, row_elems: int, elem_off: int = 0) -> int:
        if self.pull:
            return self.incoming_addr(me, k, dst, row_elems, elem_off)
        return self.incoming_addr(dst, k, me, row_elems, elem_off)

    def mc_read_addr(self, me: int, k: int, row_elems: int) -> int:
        """Multicast address of the row every rank wrote for ``me`` (pull layout only), or 0."""
        if not self.pull or not self.region.mc_base:
            return 0
        return self.region.mc_payload_addr(k * self.entry_bytes + me * row_elems * 4)

    def read_addr(self, me: int, src: int, k: int, row_elems: int) -> int:
        if self.pull:
            return self.incoming_addr(src, k, me, row_elems)
        return self.incoming_addr(me, k, src, row_elems)


class PeerBucket:
    """Bookkeeping of one bucket's gradients living in the peers' incoming regions."""

    kind = "peer"

    def __init__(self, ring: SymmGradRing, k: int, use: int, row: int):
        self.ring, self.k, self.use, self.row = ring, k, use, row


def symm_comm_for(mesh, **kw) -> SymmComm:
    return SymmComm.from_mesh(mesh, **kw)
