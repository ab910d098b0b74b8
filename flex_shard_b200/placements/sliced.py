"""Shared gather/reduce engine for placements whose local shard is a slice of the parameter.

``BlockShard`` (whole blocks along a dim), ``BucketedOwned`` (whole parameters or dim-0
slabs on an owner) and ``Shard`` members of a mixed bucket all store, on rank ``r``, one
contiguous range ``[start, start+length)`` of one dim of the parameter (possibly empty).
One row per rank is laid out as::

    [ owner-exclusive region | regular slots ]

* a *regular* parameter gets a slot of ``max_r(piece bytes)`` at the same offset in every row
  (zero padded);
* *owner-style* parameters (non-empty on one rank only) are packed back to back inside the
  owner region of their owner's row, whose size is the largest owner's total, so an owned
  matrix costs its own size once instead of once per rank.

The gather is one all-gather of byte rows (mixed dtypes allowed) and the reduction one
reduce-scatter of rows in the reduce dtype. When a bucket holds only owner-style
parameters the rows are exchanged at their own lengths with the list-form collectives
(no padding at all).

Parity: row planning of ``custom_placements/mixed_bucket.py:1603-1657`` and the owner-rows
path ``:781-976`` of the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import torch

from ..parallel.comm import plan_reduction
from ..placement_contract import (
    GradientReduction,
    Placement,
    PlacementPreparedReduceGrad,
    PlacementPreparedUnshard,
    PlacementReduceGradResult,
    PlacementUnshardResult,
)
from ..ops.segments import run_segment_ops
from ..utils.profiling import record

ALIGN = 16  # bytes; every slot starts on a 16-byte boundary


def _up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def contig_stride(shape):
    stride, acc = [], 1
    for s in reversed(shape):
        stride.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(stride))


@dataclass(frozen=True)
class Piece:
    dim: int
    start: int
    length: int

    def shape(self, global_shape: Sequence[int]) -> tuple[int, ...]:
        s = list(global_shape)
        s[self.dim] = self.length
        return tuple(s)

    def numel(self, global_shape: Sequence[int]) -> int:
        return math.prod(self.shape(global_shape)) if self.length > 0 else 0


class SlicedPlacement(Placement):
    """Base of placements described by ``pieces(global_shape, rank, world) -> [Piece]``.

    A rank may hold several pieces of one parameter only when they are adjacent slabs of dim 0
    (they are then stored back to back and treated as one local tensor).
    """

    owner_style: bool = False      # non-empty on few ranks: packed in the owner region
    allows_mixed_dtypes = True
    align_slots = True

    # ---- to implement
    def pieces(self, global_shape, rank, world_size) -> list[Piece]:
        raise NotImplementedError

    # ---- geometry from pieces
    def bucket_compatibility_key(self):
        return "sliced"

    def _dim(self, global_shape, world_size) -> int:
        for r in range(world_size):
            ps = self.pieces(global_shape, r, world_size)
            if ps:
                return ps[0].dim
        return 0

    def compute_local_shape(self, global_shape, rank, world_size):
        ps = self.pieces(global_shape, rank, world_size)
        d = ps[0].dim if ps else self._dim(global_shape, world_size)
        s = list(global_shape)
        s[d] = sum(p.length for p in ps)
        return tuple(s)

    def extract_local_shard(self, full, rank, world_size):
        ps = self.pieces(tuple(full.shape), rank, world_size)
        if not ps:
            return full.narrow(self._dim(tuple(full.shape), world_size), 0, 0)
        if len(ps) == 1:
            return full.narrow(ps[0].dim, ps[0].start, ps[0].length)
        return torch.cat([full.narrow(p.dim, p.start, p.length) for p in ps], dim=ps[0].dim)

    def local_storage_layout(self, global_shape, rank, world_size):
        from ..placement_contract import LocalStorageLayout

        ls = self.compute_local_shape(global_shape, rank, world_size)
        return LocalStorageLayout(ls, contig_stride(ls), math.prod(ls))

    def global_layout(self, global_shape, rank, world_size):
        from ..placement_contract import GlobalLayout

        g, l, s = [], [], []
        pos = 0
        nd = len(global_shape)
        for p in self.pieces(global_shape, rank, world_size):
            if p.length == 0:
                continue
            g.append(tuple(p.start if d == p.dim else 0 for d in range(nd)))
            l.append(tuple(pos if d == p.dim else 0 for d in range(nd)))
            s.append(p.shape(global_shape))
            pos += p.length
        return GlobalLayout(tuple(global_shape), tuple(g), tuple(l), tuple(s))

    # ---- bucket lifecycle through the shared engine
    def prepare_unshard_bucket(self, infos, byte_storage, comm, persistent):
        return prepare_unshard(infos, byte_storage, comm, persistent)

    def run_prepared_unshard(self, prepared, comm, async_op=False):
        run_unshard(prepared, comm, async_op)

    def finish_prepared_unshard(self, prepared, comm, persistent):
        return finish_unshard(prepared, comm, persistent)

    def prepare_reduce_grad(self, infos, grads, comm, reduce_dtype):
        return prepare_reduce(infos, grads, comm, reduce_dtype)

    def reduce_prepared_grad(self, prepared, comm, reduction):
        return reduce_prepared(prepared, comm, reduction)

    refills_persistent_buffers_in_finish = True


# --------------------------------------------------------------------------- row planning
@dataclass
class RowPlan:
    """Offsets (in ``unit`` bytes or elements) of every (param, rank) piece inside a rank row."""

    offsets: list[list[int | None]]   # [param][rank] -> offset of the local shard in rank's row
    sizes: list[list[int]]            # [param][rank] -> size of the local shard (same unit)
    row: int                          # row length when rows are padded to a common size
    row_by_rank: list[int]            # exact length of each rank's row (owner-only buckets)
    owner_only: bool


def plan_rows(infos, world_size: int, itemsize_of, align: int | None = None) -> RowPlan:
    """``itemsize_of(info)`` = bytes per element (gather rows) or 1 (reduce rows counted in elements).
    Every slot starts on a multiple of ``align`` units (default: 16 bytes for gather rows, 4 elements for
    reduce rows, so that packing and reduction kernels can use 16-byte accesses; ``align=1`` gives the
    reference's unpadded rows, ``custom_placements/mixed_bucket.py:1603-1657``)."""
    n = len(infos)
    sizes = [[0] * world_size for _ in range(n)]
    for i, info in enumerate(infos):
        for r in range(world_size):
            numel = sum(p.numel(info.global_shape) for p in info.placement.pieces(info.global_shape, r, world_size))
            sizes[i][r] = numel * itemsize_of(info)
    unit_align = align if align is not None else (ALIGN if any(itemsize_of(i) > 1 for i in infos) else 4)
    owner_idx = [i for i, info in enumerate(infos) if getattr(info.placement, "owner_style", False)]
    regular_idx = [i for i in range(n) if i not in owner_idx]
    offsets: list[list[int | None]] = [[None] * world_size for _ in range(n)]
    owner_tot = [0] * world_size
    for i in owner_idx:
        for r in range(world_size):
            if sizes[i][r] > 0:
                offsets[i][r] = owner_tot[r]
                owner_tot[r] = _up(owner_tot[r] + sizes[i][r], unit_align)
    region = max(owner_tot) if owner_idx else 0
    off = region
    for i in regular_idx:
        slot = _up(max(sizes[i]), unit_align)
        for r in range(world_size):
            offsets[i][r] = off
        off += slot
    owner_only = not regular_idx
    return RowPlan(offsets, sizes, off, owner_tot if owner_only else [off] * world_size, owner_only)


# --------------------------------------------------------------------------- gather
def _copy_or_loop(copies) -> None:
    """One segment launch when every pair is a supported (same dtype, fp32<->bf16) copy, else plain copies."""
    ok = all(d.dtype == s.dtype or {d.dtype, s.dtype} == {torch.float32, torch.bfloat16} for d, s in copies)
    if ok:
        run_segment_ops(copies)
    else:
        for d, s in copies:
            d.copy_(s)


def _local_flat(info, byte_storage):
    return info.placement.make_local_storage_view(info, byte_storage).reshape(-1)


def prepare_unshard(infos, byte_storage, comm, persistent) -> PlacementPreparedUnshard:
    W, rank = comm.world_size, comm.rank
    plan = plan_rows(infos, W, lambda i: i.param_dtype.itemsize)
    prep = PlacementPreparedUnshard(infos=infos, persistent=persistent)
    prep.extra["plan"] = plan
    prep.extra["storage"] = byte_storage
    if W == 1:
        prep.local_copy_out = True
        return prep
    dev = byte_storage.device
    with record("FlexShard::copy_in"):
        if plan.owner_only and len(set(plan.row_by_rank)) > 1:
            # uneven owner rows: exchanged at their own lengths
            rows = [torch.empty(n, dtype=torch.uint8, device=dev) for n in plan.row_by_rank]
            prep.extra["rows"] = rows
            send = rows[rank]
        else:
            prep.recv = torch.empty(W * plan.row, dtype=torch.uint8, device=dev)
            send = prep.recv[rank * plan.row:(rank + 1) * plan.row]
        if send.numel():
            needs_zero = True
            if needs_zero:
                send.zero_()
        copies = []
        for i, info in enumerate(infos):
            n = plan.sizes[i][rank]
            if n == 0:
                continue
            o = plan.offsets[i][rank]
            copies.append((send[o:o + n].view(info.param_dtype), _local_flat(info, byte_storage)))
        _copy_or_loop(copies)       # one launch for the whole bucket (casting where the compute dtype differs)
        prep.send = send
    return prep


def run_unshard(prepared, comm, async_op=False) -> None:
    if comm.world_size == 1:
        return
    rows = prepared.extra.get("rows")
    if rows is not None:
        with record("FlexShard::owner_rows_gather"):
            from .owner_rows_transport import gather_owner_rows

            gather_owner_rows(comm, prepared.send, [r.numel() for r in rows], rows)
    else:
        with record("FlexShard::mixed_all_gather"):
            prepared.work = comm.all_gather_into_tensor(prepared.recv, prepared.send, async_op=async_op)


def finish_unshard(prepared, comm, persistent) -> PlacementUnshardResult:
    W = comm.world_size
    infos = prepared.infos
    plan: RowPlan = prepared.extra["plan"]
    if prepared.work is not None:
        prepared.work.wait()
        prepared.work = None
    outs = []
    copies = []
    with record("FlexShard::copy_out"):
        for i, (info, buf) in enumerate(zip(infos, persistent)):
            full = buf[: info.global_numel].view(info.global_shape)
            for r in range(W):
                n = plan.sizes[i][r]
                if n == 0:
                    continue
                if W == 1:
                    src = _local_flat(info, prepared.extra["storage"])
                else:
                    o = plan.offsets[i][r]
                    rows = prepared.extra.get("rows")
                    row = rows[r] if rows is not None else prepared.recv[r * plan.row:(r + 1) * plan.row]
                    src = row[o:o + n].view(info.param_dtype)
                pos = 0
                for p in info.placement.pieces(info.global_shape, r, W):
                    if p.length == 0:
                        continue
                    m = p.numel(info.global_shape)
                    copies.append((full.narrow(p.dim, p.start, p.length), src[pos:pos + m].view(p.shape(info.global_shape))))
                    pos += m
            outs.append(full)
        _copy_or_loop(copies)       # every rank's piece of every parameter in one launch
    keep = [prepared.recv] if prepared.recv is not None else list(prepared.extra.get("rows") or [])
    return PlacementUnshardResult(outs, keepalive=keep)


# --------------------------------------------------------------------------- reduce
def prepare_reduce(infos, grads, comm, reduce_dtype) -> PlacementPreparedReduceGrad:
    W = comm.world_size
    plan = plan_rows(infos, W, lambda i: 1)
    dev = grads[0].device
    with record("FlexShard::reduce_scatter_copy_in"):
        uneven = plan.owner_only and len(set(plan.row_by_rank)) > 1
        if uneven:
            rows = [torch.zeros(n, dtype=reduce_dtype, device=dev) for n in plan.row_by_rank]
        else:
            flat = torch.zeros(W * plan.row, dtype=reduce_dtype, device=dev)
            rows = [flat[r * plan.row:(r + 1) * plan.row] for r in range(W)]
        copies = []
        for i, (info, g) in enumerate(zip(infos, grads)):
            for r in range(W):
                n = plan.sizes[i][r]
                if n == 0:
                    continue
                o = plan.offsets[i][r]
                pos = 0
                for p in info.placement.pieces(info.global_shape, r, W):
                    if p.length == 0:
                        continue
                    m = p.numel(info.global_shape)
                    copies.append((rows[r][o + pos:o + pos + m].view(p.shape(info.global_shape)),
                                   g.narrow(p.dim, p.start, p.length)))
                    pos += m
        _copy_or_loop(copies)
    prep = PlacementPreparedReduceGrad(infos=infos, send=None if uneven else flat, reduce_dtype=reduce_dtype)
    prep.extra["plan"] = plan
    prep.extra["rows"] = rows
    prep.extra["uneven"] = uneven
    return prep


def reduce_prepared(prepared, comm, reduction: GradientReduction) -> PlacementReduceGradResult:
    W, rank = comm.world_size, comm.rank
    plan: RowPlan = prepared.extra["plan"]
    rplan = plan_reduction(reduction, W, prepared.reduce_dtype)
    rows = prepared.extra["rows"]
    with record("FlexShard::mixed_reduce_scatter"):
        if W == 1:
            out = rows[0]
            if rplan.post_divide is not None:
                out.div_(rplan.post_divide)
        elif prepared.extra["uneven"]:
            out = torch.empty(plan.row_by_rank[rank], dtype=prepared.reduce_dtype, device=rows[0].device)
            comm.reduce_scatter_list(out, rows, rplan)
        else:
            out = torch.empty(plan.row, dtype=prepared.reduce_dtype, device=rows[0].device)
            comm.reduce_scatter_tensor(out, prepared.send, rplan)
    grads = []
    for i, info in enumerate(prepared.infos):
        n = plan.sizes[i][rank]
        o = plan.offsets[i][rank]
        if n == 0 or o is None:
            grads.append(torch.zeros(info.local_shape, dtype=prepared.reduce_dtype, device=out.device)
                         if math.prod(info.local_shape) == 0 else None)
        else:
            grads.append(out[o:o + n].view(info.local_shape))
    return PlacementReduceGradResult(grads=grads, output=out)
