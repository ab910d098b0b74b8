"""``BucketedOwned``: whole parameters (or whole dim-0 slabs) live on owner ranks.

The storage scheme that lets Muon orthogonalise a matrix without communication: the owner holds
the full matrix, every other rank holds nothing. In a gather each owner contributes the rows it
owns (no padding: owner rows are exchanged at their own lengths, or packed in the owner region of
a mixed bucket); gradients are reduced into the owner's rows.

Parity: ``custom_placements/owned.py:54-583`` of the reference (``segments_by_fqn`` with
``view_kind`` ``full_param`` / ``expert_block``, LPT owner assignment hosts-first with carried
loads ``:393-495``, expert-block segments ``:505-583``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Mapping, Sequence

from ..utils.validation import assign_to_hosts_then_ranks, mesh_rank_hosts
from .sliced import Piece, SlicedPlacement


@dataclass(frozen=True)
class BucketedOwnedSegmentSpec:
    """A flat slice of one parameter and the rank that owns it: the bucket-level description of ownership
    (``{fqn: [specs]}``) that ``BucketedOwned`` also accepts.  ``param_offset`` and ``numel`` count elements of the
    row-major parameter and must cover whole dim-0 rows; ``storage_order`` orders the owners' storage.
    Parity: ``custom_placements/owned.py:39-48`` of the reference."""

    name: str
    fqn: str
    param_offset: int
    numel: int
    owner_rank: int
    storage_order: int = 0


class BucketedOwned(SlicedPlacement):
    """One parameter's ownership: ``segments`` = ((rank, start, length), ...) over dim 0.

    Also takes the bucket-level form ``{fqn: [BucketedOwnedSegmentSpec, ...]}``: one object for every parameter of
    the bucket, from which ``flex_shard`` takes each parameter's own placement (``for_param``).

    ``view_kind == "full_param"``: a single segment covering the parameter on its owner.
    ``view_kind == "expert_block"``: dim-0 slabs (e.g. experts of a stacked weight) with
    possibly different owners.
    """

    owner_style = True

    def __init__(self, segments, view_kind: str = "full_param"):
        if view_kind not in ("full_param", "expert_block"):
            raise ValueError(f"unknown view_kind {view_kind!r}")
        self.view_kind = view_kind
        self.segments_by_fqn = None
        if isinstance(segments, Mapping):
            for fqn, specs in segments.items():
                if not specs or any(not isinstance(sp, BucketedOwnedSegmentSpec) or sp.fqn != fqn for sp in specs):
                    raise ValueError(f"segments of {fqn!r} must be a non-empty list of BucketedOwnedSegmentSpec "
                                     "naming that parameter")
            self.segments_by_fqn = {f: tuple(specs) for f, specs in segments.items()}
            self.segments, self._extent = (), 0
            return
        self.segments = tuple((int(r), int(s), int(l)) for r, s, l in segments)
        pos = 0
        for _, s, l in sorted(self.segments, key=lambda t: t[1]):
            if s != pos or l <= 0:
                raise ValueError(f"segments must tile dim 0 exactly, got {self.segments}")
            pos += l
        self._extent = pos

    def for_param(self, fqn: str, shape: Sequence[int]) -> "BucketedOwned":
        """The placement of one parameter: this object itself, or, for the bucket-level form, the dim-0 row
        segments that the parameter's flat slices amount to."""
        if self.segments_by_fqn is None:
            return self
        specs = self.segments_by_fqn.get(fqn)
        if specs is None:
            raise ValueError(f"BucketedOwned has no segments for {fqn!r} (it describes {sorted(self.segments_by_fqn)})")
        row = math.prod(shape[1:]) if len(shape) > 1 else 1
        rows = []
        for sp in sorted(specs, key=lambda sp: sp.param_offset):
            if sp.param_offset % row or sp.numel % row or sp.numel <= 0:
                raise ValueError(f"segment {sp.name!r} of {fqn!r} (offset {sp.param_offset}, {sp.numel} elements) does "
                                 f"not cover whole dim-0 rows of {row} elements")
            rows.append((sp.owner_rank, sp.param_offset // row, sp.numel // row))
        return BucketedOwned(rows, self.view_kind)

    def __eq__(self, other):
        return isinstance(other, BucketedOwned) and (other.segments, other.view_kind, other.segments_by_fqn) == (
            self.segments, self.view_kind, self.segments_by_fqn)

    def __hash__(self):
        by_fqn = None if self.segments_by_fqn is None else tuple(sorted(self.segments_by_fqn.items()))
        return hash(("BucketedOwned", self.segments, self.view_kind, by_fqn))

    def __repr__(self):
        return f"BucketedOwned(segments={self.segments}, view_kind={self.view_kind!r})"

    @property
    def owners(self) -> tuple[int, ...]:
        return tuple(sorted({r for r, _, _ in self.segments}))

    def pieces(self, global_shape, rank, world_size):
        if self.segments_by_fqn is not None:
            raise ValueError("a bucket-level BucketedOwned describes several parameters: use for_param(fqn, shape)")
        if global_shape[0] != self._extent:
            raise ValueError(f"segments cover {self._extent} rows, the parameter has {global_shape[0]}")
        mine = sorted((s, l) for r, s, l in self.segments if r == rank)
        # adjacent slabs merge into one piece
        out: list[Piece] = []
        for s, l in mine:
            if out and out[-1].start + out[-1].length == s:
                out[-1] = Piece(0, out[-1].start, out[-1].length + l)
            else:
                out.append(Piece(0, s, l))
        return out

    def reduces_grads_in_param_layout(self, infos) -> bool:
        """Grads can be handed over as views of one mirror bucket when no cast separates the
        gradient dtype from the reduce dtype."""
        return all(i.param_dtype == (i.bucket_reduce_dtype or i.reduce_dtype) for i in infos)


def newton_schulz_cost(shape: Sequence[int], ns_steps: int = 5) -> float:
    """FLOP-proportional cost of orthogonalising one matrix: ``steps * s^2 (2 l + s)`` with
    s = min dim, l = max dim (batched leading dims multiply)."""
    if len(shape) < 2:
        return float(math.prod(shape))
    s, l = sorted(shape[-2:])
    return float(ns_steps * s * s * (2 * l + s) * math.prod(shape[:-2]))


def _global_ranks(mesh, group, world_size: int):
    """The mesh's global ranks in mesh order when they can be known (a sub-mesh need not start at rank 0 nor be
    contiguous, and hosts follow the global ranks), else the mesh size."""
    ranks = getattr(mesh, "mesh", None)
    if ranks is not None and hasattr(ranks, "flatten"):
        return [int(r) for r in ranks.flatten().tolist()]
    if group is not None and world_size > 1:
        import torch.distributed as dist

        return list(dist.get_process_group_ranks(group))
    return world_size


def make_bucketed_owned_full_param_placement_fn(carry_loads: bool = False, cost_fn=None,
                                                owner_by_fqn: Mapping[str, int] | None = None,
                                                ranks_per_host: int | None = None):
    """LPT assignment of whole parameters to owners (hosts first, then ranks). With
    ``carry_loads`` the per-rank loads persist across calls (buckets), which spreads many
    identical buckets over the whole mesh instead of reusing the same few owners."""
    cost_fn = cost_fn or (lambda fqn, p: newton_schulz_cost(tuple(p.shape)))
    carried: list[float] = []       # lives with this function (not in a registry keyed by an address that a later function could reuse)

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        group, _, W, _ = mesh_group(mesh)
        hosts = mesh_rank_hosts(_global_ranks(mesh, group, W), ranks_per_host)
        if carry_loads:
            if len(carried) != W:
                carried[:] = [0.0] * W
            loads = carried
        else:
            loads = [0.0] * W
        fixed = {f: owner_by_fqn[f] for f, _ in named_params if owner_by_fqn and f in owner_by_fqn}
        for f, p in named_params:
            if f in fixed:
                loads[fixed[f]] += cost_fn(f, p)
        free = [(f, p) for f, p in named_params if f not in fixed]
        owners = assign_to_hosts_then_ranks([cost_fn(f, p) for f, p in free], hosts, loads)
        out = {}
        for (f, p), r in zip(free, owners):
            out[f] = BucketedOwned(((r, 0, p.shape[0]),), "full_param")
        for f, p in named_params:
            if f in fixed:
                out[f] = BucketedOwned(((fixed[f], 0, p.shape[0]),), "full_param")
        return out

    fn.reset_loads = carried.clear
    return fn


def make_bucketed_owned_full_param_segments(named_params, world_size: int, *, hosts: Sequence[int] | None = None,
                                            carried_loads: Sequence[float] | None = None
                                            ) -> dict[str, list[BucketedOwnedSegmentSpec]]:
    """One whole-parameter segment per parameter; owners by longest-processing-time on the element count.  Without
    ``hosts``: the largest parameter first onto the rank that carries least, ``carried_loads`` (each rank's elements
    from earlier buckets) counted in.  With ``hosts`` (each rank's host, ``mesh_rank_hosts``): hosts first, then the
    ranks of the host, the bucket balanced by itself and ``carried_loads`` breaking ties.  ``carried_loads`` is not
    changed: the caller adds what this bucket placed.  Parity: ``custom_placements/owned.py:393-462`` of the
    reference."""
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}")
    if hosts is not None and len(hosts) != world_size:
        raise ValueError(f"hosts must give each of the {world_size} ranks a host")
    if carried_loads is not None and len(carried_loads) != world_size:
        raise ValueError(f"carried_loads must give each of the {world_size} ranks a load")
    named_params = list(named_params)
    sizes = [float(p.numel()) for _, p in named_params]
    if hosts is not None:
        owners = assign_to_hosts_then_ranks(sizes, list(hosts), carried_loads=list(carried_loads or [0.0] * world_size))
    else:
        load = list(carried_loads or [0.0] * world_size)
        owners = [0] * len(sizes)
        for i in sorted(range(len(sizes)), key=lambda i: -sizes[i]):
            r = min(range(world_size), key=lambda r: load[r])        # the first of equals: the lowest rank
            owners[i] = r
            load[r] += sizes[i]
    return {f: [BucketedOwnedSegmentSpec(f"{f}#full", f, 0, p.numel(), r, order)]
            for order, ((f, p), r) in enumerate(zip(named_params, owners))}


def make_bucketed_owned_expert_block_segments(named_params, world_size: int, *,
                                              suffix_order: tuple[str, ...] = (".w1", ".w3", ".w2")
                                              ) -> dict[str, list[BucketedOwnedSegmentSpec]]:
    """One segment per expert of stacked expert weights ``[E, ...]``; experts go to the ranks in contiguous runs, as
    evenly as possible, the same run for every weight; ``suffix_order`` orders the weights of one expert in the
    owner's storage.  Parity: ``custom_placements/owned.py:505-583`` of the reference."""
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}")
    if not suffix_order:
        raise ValueError("suffix_order must contain at least one suffix")
    named_params = list(named_params)
    bad = [(f, tuple(p.shape)) for f, p in named_params if p.dim() < 3 or not f.endswith(tuple(suffix_order))]
    if bad:
        raise ValueError(f"expert-block segments need stacked weights of at least 3 dims whose names end in one of "
                         f"{suffix_order}: {bad}")
    if not named_params:
        return {}
    E = named_params[0][1].shape[0]
    if any(p.shape[0] != E for _, p in named_params):
        raise ValueError("stacked expert weights of one bucket must hold the same number of experts")
    per = [E // world_size + (1 if r < E % world_size else 0) for r in range(world_size)]
    owner_of = [r for r, n in enumerate(per) for _ in range(n)]
    rank_of_suffix = {sfx: i for i, sfx in enumerate(suffix_order)}
    out: dict[str, list[BucketedOwnedSegmentSpec]] = {}
    for f, p in named_params:
        slab = p.numel() // E
        which = next(rank_of_suffix[sfx] for sfx in suffix_order if f.endswith(sfx))
        out[f] = [BucketedOwnedSegmentSpec(f"{f}#expert{e}", f, e * slab, slab, owner_of[e],
                                           e * len(suffix_order) + which) for e in range(E)]
    return out


def make_bucketed_owned_expert_block_placement_fn(experts_per_rank: Sequence[int] | None = None):
    """Stacked expert weights ``[E, ...]``: contiguous runs of experts per rank."""

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        out = {}
        for f, p in named_params:
            E = p.shape[0]
            per = list(experts_per_rank) if experts_per_rank else [E // W + (1 if r < E % W else 0) for r in range(W)]
            segs, pos = [], 0
            for r, n in enumerate(per):
                if n > 0:
                    segs.append((r, pos, n))
                    pos += n
            out[f] = BucketedOwned(tuple(segs), "expert_block")
        return out

    return fn
