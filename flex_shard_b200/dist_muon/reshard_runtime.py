"""Pipelined execution of DistMuon's redistributed buckets.

For every bucket of parameters whose storage layout differs from the compute layout the optimizer step is
three stages: **A** momentum update on the stored rows, pack the Nesterov direction as bf16 and exchange it
storage -> compute; **B** Newton-Schulz on the owners' whole matrices; **C** exchange the orthogonalised
rows compute -> storage and apply the update to the stored rows.  A and C run on a *transfer stream*, B on
the caller's stream, with two buffer slots, so while bucket *i* is in B the exchange of bucket *i+1* (A) and
the return of bucket *i-1* (C) are in flight: the transfer stream sees ``A0 A1 C0 A2 C1 A3 C2 ...``.
Buffers for both slots are reserved once, sized for the largest bucket.  Buckets that need no exchange run
A, B, C back to back on the caller's stream without touching a buffer.

The payload is bf16 in both directions.  Newton-Schulz starts by rounding its input to bf16 and ends with a
bf16 matrix, so nothing is lost against exchanging fp32, and the NVLink bytes halve.

Parity: ``dist_muon/_optimizer_reshard_runtime.py`` of the reference (two slots, one transfer stream,
three events per slot ``:234-282``; rolling prefetch ``:420-557``; pre-reserved buffers ``:325-418``; local
buckets bypass communication ``:644-661``).  CPU groups (gloo) run the same schedule without streams.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist

from .reshard_plan import PackedSchedule, RedistributionPlan, pack, unpack


@dataclass
class LocalBucket:
    """A bucket whose parameters are computed where they are stored."""

    items: tuple
    name: str = ""


@dataclass
class RedistributedBucket:
    """A bucket with at least one parameter that travels: plans and both packed schedules."""

    items: tuple                      # parameters that travel, in plan order
    plans: tuple[RedistributionPlan, ...]
    to_compute: PackedSchedule
    to_storage: PackedSchedule
    local_items: tuple = ()           # members of the bucket that need no exchange
    name: str = ""
    digest: int = 0


@dataclass
class _Slot:
    send: torch.Tensor | None = None
    recv: torch.Tensor | None = None
    back_send: torch.Tensor | None = None
    back_recv: torch.Tensor | None = None
    input_ready: Any = None
    compute_done: Any = None
    returned: Any = None
    keep: list = field(default_factory=list)


class RedistributionRuntime:
    SLOTS = 2

    def __init__(self, device: torch.device, group=None, payload_dtype: torch.dtype = torch.bfloat16,
                 exchange: Callable | None = None):
        self.device = device
        self.group = group
        self.payload_dtype = payload_dtype
        self.cuda = device.type == "cuda"
        self.transfer_stream = torch.cuda.Stream(device=device) if self.cuda else None
        self.slots = [_Slot() for _ in range(self.SLOTS)]
        self._reserved = (0, 0)
        self._exchange_fn = exchange or self._all_to_all
        self.exchanges = 0            # exchanges issued (two per redistributed bucket per step)
        self.trace: list[str] = []    # order in which stages were issued (tests assert the pipeline shape)
        self.record_trace = False

    # ------------------------------------------------------------------ buffers
    def reserve(self, buckets: Sequence) -> None:
        """Allocate both slots' buffers for the largest bucket (idempotent while sizes do not grow)."""
        fwd = max((max(b.to_compute.send_numel, b.to_compute.recv_numel) for b in buckets
                   if isinstance(b, RedistributedBucket)), default=0)
        back = max((max(b.to_storage.send_numel, b.to_storage.recv_numel) for b in buckets
                    if isinstance(b, RedistributedBucket)), default=0)
        if fwd <= self._reserved[0] and back <= self._reserved[1]:
            return
        fwd, back = max(fwd, self._reserved[0]), max(back, self._reserved[1])
        for s in self.slots:
            s.send = torch.empty(fwd, dtype=self.payload_dtype, device=self.device)
            s.recv = torch.empty(fwd, dtype=self.payload_dtype, device=self.device)
            s.back_send = torch.empty(back, dtype=self.payload_dtype, device=self.device)
            s.back_recv = torch.empty(back, dtype=self.payload_dtype, device=self.device)
        self._reserved = (fwd, back)

    # ------------------------------------------------------------------ transport
    def _all_to_all(self, recv, send, sched: PackedSchedule) -> None:
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_to_all_single(recv, send, list(sched.recv_splits), list(sched.send_splits), group=self.group)
        else:
            recv.copy_(send)

    def _exchange(self, recv, send, sched: PackedSchedule) -> None:
        self.exchanges += 1
        self._exchange_fn(recv[: sched.recv_numel], send[: sched.send_numel], sched)

    def _note(self, what: str) -> None:
        if self.record_trace:
            self.trace.append(what)

    # ------------------------------------------------------------------ the three stages
    def _stage_a(self, i, b: RedistributedBucket, slot: _Slot, prepare) -> None:
        """Transfer stream: momentum + direction on stored rows, pack, exchange to the owners."""
        self._note(f"A{i}")
        inputs = [prepare(item) for item in b.items]            # storage-layout directions
        pack(slot.send, inputs, b.to_compute.send_spans)
        self._exchange(slot.recv, slot.send, b.to_compute)
        slot.keep = inputs

    def _stage_b(self, i, b: RedistributedBucket, slot: _Slot, compute) -> None:
        """Caller's stream: unpack into whole matrices, orthogonalise, pack the results."""
        self._note(f"B{i}")
        rank = b.to_compute.rank
        full = [torch.empty(p.compute[rank].tensor_shape, dtype=self.payload_dtype, device=self.device)
                for p in b.plans]
        unpack(slot.recv, full, b.to_compute.recv_spans)
        outs = [compute(item, plan, t) for item, plan, t in zip(b.items, b.plans, full)]
        pack(slot.back_send, outs, b.to_storage.send_spans)

    def _stage_c(self, i, b: RedistributedBucket, slot: _Slot, finalize) -> None:
        """Transfer stream: exchange back to the storing ranks, unpack, apply the update."""
        self._note(f"C{i}")
        rank = b.to_storage.rank
        self._exchange(slot.back_recv, slot.back_send, b.to_storage)
        upd = [torch.empty(p.storage[rank].tensor_shape, dtype=self.payload_dtype, device=self.device)
               for p in b.plans]
        unpack(slot.back_recv, upd, b.to_storage.recv_spans)
        for item, u in zip(b.items, upd):
            finalize(item, u)
        slot.keep = []

    # ------------------------------------------------------------------ driver
    def run(self, buckets: Sequence, prepare: Callable, compute: Callable, finalize: Callable,
            local_step: Callable) -> None:
        """Run one optimizer step over ``buckets`` (in order).

        ``prepare(item) -> tensor``  the direction *u* in the storage layout (updates the momentum);
        ``compute(item, plan, full) -> tensor``  Newton-Schulz over the owner's stacked matrices;
        ``finalize(item, update)``  applies the returned rows to the stored parameter;
        ``local_step(item)``  the whole update for an item that needs no exchange."""
        self.reserve(buckets)
        red = [(i, b) for i, b in enumerate(buckets) if isinstance(b, RedistributedBucket)]
        ts = self.transfer_stream
        cur = torch.cuda.current_stream(self.device) if self.cuda else None

        def on_transfer(fn, *a):
            if ts is None:
                fn(*a)
                return None
            with torch.cuda.stream(ts):
                fn(*a)
                return ts.record_event()

        if ts is not None and red:
            ts.wait_event(cur.record_event())      # gradients and parameters are ready on the caller's stream
        nxt = 0                                     # index into `red` of the next bucket whose stage A is due
        if red:
            i0, b0 = red[0]
            self.slots[0].input_ready = on_transfer(self._stage_a, i0, b0, self.slots[0], prepare)
            nxt = 1
        k = 0                                       # position in `red` of the bucket whose stage B is next
        for i, b in enumerate(buckets):
            if isinstance(b, LocalBucket):
                self._note(f"L{i}")
                for item in b.items:
                    local_step(item)
                continue
            slot = self.slots[k % self.SLOTS]
            # prefetch: the next redistributed bucket's exchange goes out before this bucket's Newton-Schulz
            if nxt < len(red) and nxt == k + 1:
                j, bj = red[nxt]
                sj = self.slots[nxt % self.SLOTS]
                sj.input_ready = on_transfer(self._stage_a, j, bj, sj, prepare)
                nxt += 1
            if slot.input_ready is not None:
                cur.wait_event(slot.input_ready)
            self._stage_b(i, b, slot, compute)
            for item in b.local_items:
                local_step(item)
            if ts is not None:
                slot.compute_done = cur.record_event()
                ts.wait_event(slot.compute_done)
            slot.returned = on_transfer(self._stage_c, i, b, slot, finalize)
            k += 1
        if ts is not None:
            for s in self.slots:
                if s.returned is not None:
                    cur.wait_event(s.returned)      # later work on the caller's stream sees the updated rows
                s.input_ready = s.compute_done = s.returned = None
