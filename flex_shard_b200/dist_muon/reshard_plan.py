"""Plans for moving Muon's inputs from where parameters are *stored* to where they are *orthogonalised*.

A parameter stored as ``Shard(0)`` rows cannot be orthogonalised in place: Newton-Schulz needs whole
matrices.  For every such parameter a ``RedistributionPlan`` says, as rectangular regions, which part of
the logical tensor each rank stores, which part each rank computes on, and which *routes* carry one into
the other.  A plan is validated once when it is built: the storage regions and the compute regions each
tile the logical tensor exactly, every route has equal element counts at both ends, the routes tile the
logical tensor exactly, and per rank the routes' source regions tile its storage tensor and the
destination regions tile its compute tensor.  A bucket's plans are then flattened, per direction, into a
``PackedSchedule``: split sizes of one uneven all-to-all and, per parameter, the spans of the packed send
and receive buffers.  ``plan_digest`` / ``check_plans_across_ranks`` make sure every rank built the same
plans before the first exchange.

Parity: the role of ``dist_muon/_optimizer_reshard_schedule.py`` of the reference (regions, routes and
validated plans ``:105-318``, packed all-to-all schedules ``:705-890``, the cross-rank hash ``:1214-1251``).
Here parameters are plain local tensors, so plans are built from row intervals instead of DTensor specs,
and the same schedule drives either ``all_to_all_single`` or one peer-pull kernel over NVLink.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, field
from typing import Sequence

import torch
import torch.distributed as dist


class PlanError(RuntimeError):
    def __init__(self, message: str):
        super().__init__(f"invalid redistribution plan: {message}")


# --------------------------------------------------------------------------- geometry
@dataclass(frozen=True)
class Region:
    """A rectangular block of a tensor: ``offsets`` and ``shape`` per dimension."""

    offsets: tuple[int, ...]
    shape: tuple[int, ...]

    def __post_init__(self):
        object.__setattr__(self, "offsets", tuple(int(o) for o in self.offsets))
        object.__setattr__(self, "shape", tuple(int(s) for s in self.shape))

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    def inside(self, bounds: Sequence[int]) -> bool:
        return (len(self.offsets) == len(bounds) == len(self.shape)
                and all(o >= 0 and s >= 0 and o + s <= b for o, s, b in zip(self.offsets, self.shape, bounds)))

    def overlaps(self, other: "Region") -> bool:
        if self.numel == 0 or other.numel == 0:
            return False
        return all(a < bo + bs and bo < a + s
                   for a, s, bo, bs in zip(self.offsets, self.shape, other.offsets, other.shape))

    def view_of(self, t: torch.Tensor) -> torch.Tensor:
        for d, (o, s) in enumerate(zip(self.offsets, self.shape)):
            t = t.narrow(d, o, s)
        return t


def rows_region(lo: int, hi: int, shape: Sequence[int]) -> Region:
    """Rows ``[lo, hi)`` of a tensor of ``shape`` (all of every other dimension)."""
    return Region((lo, *([0] * (len(shape) - 1))), (hi - lo, *shape[1:]))


@dataclass(frozen=True)
class Partition:
    """What one rank holds: the shape of its local tensor and the logical regions in it, in local order
    (region *i* starts where region *i-1* ended along dim 0)."""

    rank: int
    tensor_shape: tuple[int, ...]
    logical_regions: tuple[Region, ...]


@dataclass(frozen=True)
class Route:
    """One logical region travelling from ``src_rank``'s storage tensor to ``dst_rank``'s compute tensor."""

    logical: Region
    src_rank: int
    src_region: Region
    dst_rank: int
    dst_region: Region

    def inverse(self) -> "Route":
        return Route(self.logical, self.dst_rank, self.dst_region, self.src_rank, self.src_region)


def _tiles_exactly(regions: Sequence[Region], bounds: Sequence[int], what: str) -> None:
    for r in regions:
        if not r.inside(bounds):
            raise PlanError(f"{what}: region {r.offsets}+{r.shape} leaves the bounds {tuple(bounds)}")
    live = [r for r in regions if r.numel]
    if sum(r.numel for r in live) != math.prod(bounds):
        raise PlanError(f"{what}: regions cover {sum(r.numel for r in live)} of {math.prod(bounds)} elements")
    live.sort(key=lambda r: r.offsets)
    for i, a in enumerate(live):
        for b in live[i + 1:]:
            if b.offsets[0] >= a.offsets[0] + a.shape[0]:
                break
            if a.overlaps(b):
                raise PlanError(f"{what}: regions {a.offsets}+{a.shape} and {b.offsets}+{b.shape} overlap")


@dataclass(frozen=True)
class RedistributionPlan:
    """Storage partition, compute partition and routes of one parameter over ``world`` ranks."""

    world: int
    logical_shape: tuple[int, ...]
    storage: tuple[Partition, ...]
    compute: tuple[Partition, ...]
    routes: tuple[Route, ...]
    matrices: tuple[tuple[int, int, int], ...] = ()   # (row start, row end, owner) of every Newton-Schulz matrix
    back_routes: tuple[Route, ...] = field(init=False)

    def __post_init__(self):
        object.__setattr__(self, "logical_shape", tuple(self.logical_shape))
        object.__setattr__(self, "back_routes", tuple(r.inverse() for r in self.routes))
        self.validate()

    def validate(self) -> None:
        W, shape = self.world, self.logical_shape
        for name, parts in (("storage", self.storage), ("compute", self.compute)):
            if [p.rank for p in parts] != list(range(W)):
                raise PlanError(f"{name} partitions must list ranks 0..{W - 1} in order")
            _tiles_exactly([r for p in parts for r in p.logical_regions], shape, f"{name} partition")
            for p in parts:
                if sum(r.numel for r in p.logical_regions) != math.prod(p.tensor_shape):
                    raise PlanError(f"{name} tensor of rank {p.rank} has {math.prod(p.tensor_shape)} elements "
                                    f"for {sum(r.numel for r in p.logical_regions)} logical ones")
        for rt in self.routes:
            if not (0 <= rt.src_rank < W and 0 <= rt.dst_rank < W):
                raise PlanError("a route names a rank outside the group")
            if not (rt.logical.numel == rt.src_region.numel == rt.dst_region.numel):
                raise PlanError("a route's logical, source and destination regions differ in size")
        _tiles_exactly([rt.logical for rt in self.routes], shape, "routes")
        for r in range(W):
            _tiles_exactly([rt.src_region for rt in self.routes if rt.src_rank == r],
                           self.storage[r].tensor_shape, f"sources on rank {r}")
            _tiles_exactly([rt.dst_region for rt in self.routes if rt.dst_rank == r],
                           self.compute[r].tensor_shape, f"destinations on rank {r}")

    @property
    def is_local(self) -> bool:
        """True when no element changes rank (storage already is the compute layout)."""
        return all(rt.src_rank == rt.dst_rank for rt in self.routes)

    def key(self) -> tuple:
        return (self.world, self.logical_shape,
                tuple((p.rank, p.tensor_shape, tuple((r.offsets, r.shape) for r in p.logical_regions))
                      for p in self.storage + self.compute),
                tuple((rt.logical.offsets, rt.logical.shape, rt.src_rank, rt.src_region.offsets, rt.dst_rank,
                       rt.dst_region.offsets) for rt in self.routes), self.matrices)


def plan_rows(logical_shape: Sequence[int], storage_rows: Sequence[tuple[int, int]],
              matrices: Sequence[tuple[int, int, int]]) -> RedistributionPlan:
    """Plan for a tensor stored in dim-0 intervals and computed on in dim-0 blocks.

    ``storage_rows[r]`` = rows ``[lo, hi)`` rank r stores (``Shard(0)`` geometry; empty ranks give
    ``lo == hi``).  ``matrices`` = ``(lo, hi, owner)`` per Newton-Schulz matrix: a whole 2-D parameter is one
    entry, a parameter cut into heads has one per head, a native ``[n, R, C]`` batch one per slice.  Each
    owner's compute tensor is its matrices stacked along dim 0 in order of ``lo``."""
    shape = tuple(int(s) for s in logical_shape)
    W = len(storage_rows)
    storage = tuple(Partition(r, (hi - lo, *shape[1:]), (rows_region(lo, hi, shape),) if hi > lo else ())
                    for r, (lo, hi) in enumerate(storage_rows))
    mats = sorted((int(lo), int(hi), int(o)) for lo, hi, o in matrices)
    base, owned = {}, {r: [] for r in range(W)}
    for lo, hi, o in mats:
        if not 0 <= o < W:
            raise PlanError(f"matrix rows [{lo}, {hi}) are assigned to rank {o} outside the group of {W}")
        base[(lo, hi)] = sum(h - l for l, h in owned[o])
        owned[o].append((lo, hi))
    compute = tuple(Partition(r, (sum(h - l for l, h in owned[r]), *shape[1:]),
                              tuple(rows_region(l, h, shape) for l, h in owned[r])) for r in range(W))
    routes = []
    for lo, hi, o in mats:
        for r, (slo, shi) in enumerate(storage_rows):
            a, b = max(lo, slo), min(hi, shi)
            if b <= a:
                continue
            routes.append(Route(rows_region(a, b, shape), r, rows_region(a - slo, b - slo, shape),
                                o, rows_region(base[(lo, hi)] + a - lo, base[(lo, hi)] + b - lo, shape)))
    return RedistributionPlan(W, shape, storage, compute, tuple(routes), tuple(mats))


# --------------------------------------------------------------------------- packed schedules
@dataclass(frozen=True)
class Span:
    """Where one endpoint region sits in a packed buffer (offset in elements)."""

    region: Region
    offset: int


@dataclass(frozen=True)
class PackedSchedule:
    """One rank's view of an uneven all-to-all over a bucket of parameters.

    ``send_splits[d]`` / ``recv_splits[s]`` are element counts per peer; ``table[s][d]`` is the whole
    traffic matrix (every rank computes it, which sizes symmetric buffers for the peer-pull transport);
    ``send_spans[i]`` / ``recv_spans[i]`` place parameter *i*'s regions in the packed buffers.  Pieces for
    one peer are ordered by parameter, then by route."""

    rank: int
    send_splits: tuple[int, ...]
    recv_splits: tuple[int, ...]
    table: tuple[tuple[int, ...], ...]
    send_spans: tuple[tuple[Span, ...], ...]
    recv_spans: tuple[tuple[Span, ...], ...]

    @property
    def send_numel(self) -> int:
        return sum(self.send_splits)

    @property
    def recv_numel(self) -> int:
        return sum(self.recv_splits)

    @property
    def has_remote(self) -> bool:
        return any(n for s, row in enumerate(self.table) for d, n in enumerate(row) if s != d)


def packed_schedule(plans: Sequence[RedistributionPlan], rank: int, to_compute: bool) -> PackedSchedule:
    """Flatten a bucket's plans into this rank's all-to-all schedule for one direction."""
    if not plans:
        raise PlanError("a bucket schedule needs at least one plan")
    W = plans[0].world
    if any(p.world != W for p in plans):
        raise PlanError("plans of one bucket must span the same ranks")
    routes = [p.routes if to_compute else p.back_routes for p in plans]
    table = [[0] * W for _ in range(W)]
    for rs in routes:
        for rt in rs:
            table[rt.src_rank][rt.dst_rank] += rt.logical.numel
    send_spans: list[list[Span]] = [[] for _ in plans]
    recv_spans: list[list[Span]] = [[] for _ in plans]
    cur = 0
    for d in range(W):
        for i, rs in enumerate(routes):
            for rt in rs:
                if rt.src_rank == rank and rt.dst_rank == d:
                    send_spans[i].append(Span(rt.src_region, cur))
                    cur += rt.logical.numel
    cur = 0
    for s in range(W):
        for i, rs in enumerate(routes):
            for rt in rs:
                if rt.src_rank == s and rt.dst_rank == rank:
                    recv_spans[i].append(Span(rt.dst_region, cur))
                    cur += rt.logical.numel
    return PackedSchedule(rank, tuple(table[rank]), tuple(table[s][rank] for s in range(W)),
                          tuple(tuple(r) for r in table), tuple(tuple(s) for s in send_spans),
                          tuple(tuple(s) for s in recv_spans))


def pack(buffer: torch.Tensor, tensors: Sequence[torch.Tensor], spans: Sequence[Sequence[Span]]) -> None:
    """Copy every span's region of its tensor into the packed buffer (casting to the buffer's dtype)."""
    for t, sp in zip(tensors, spans):
        for s in sp:
            if s.region.numel:
                buffer[s.offset:s.offset + s.region.numel].view(s.region.shape).copy_(s.region.view_of(t))


def unpack(buffer: torch.Tensor, tensors: Sequence[torch.Tensor], spans: Sequence[Sequence[Span]]) -> None:
    for t, sp in zip(tensors, spans):
        for s in sp:
            if s.region.numel:
                s.region.view_of(t).copy_(buffer[s.offset:s.offset + s.region.numel].view(s.region.shape))


# --------------------------------------------------------------------------- agreement between ranks
def plan_digest(plans: Sequence[RedistributionPlan], extra: Sequence = ()) -> int:
    """A 56-bit digest of a bucket's plans (and anything else every rank must agree on: names, dtypes)."""
    desc = repr((tuple(p.key() for p in plans), tuple(extra)))
    return int.from_bytes(hashlib.sha256(desc.encode()).digest()[:7], "little")


def check_plans_across_ranks(digest: int, group=None, device: torch.device | None = None) -> None:
    """Collectively compare ``digest``; raises on every rank that sees a different value anywhere.
    Without an initialised process group (one process) there is nothing to compare."""
    if not dist.is_initialized():
        return
    W = dist.get_world_size(group)
    if W == 1:
        return
    dev = device if device is not None and dist.get_backend(group) == "nccl" else torch.device("cpu")
    mine = torch.tensor([digest], dtype=torch.int64, device=dev)
    seen = [torch.empty_like(mine) for _ in range(W)]
    dist.all_gather(seen, mine, group=group)
    if any(int(t.item()) != digest for t in seen):
        raise RuntimeError("optimizer bucket plans differ across ranks")
