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
from typing import Mapping, Sequence

from ..utils.validation import assign_to_hosts_then_ranks, mesh_rank_hosts
from .sliced import Piece, SlicedPlacement


class BucketedOwned(SlicedPlacement):
    """One parameter's ownership: ``segments`` = ((rank, start, length), ...) over dim 0.

    ``view_kind == "full_param"``: a single segment covering the parameter on its owner.
    ``view_kind == "expert_block"``: dim-0 slabs (e.g. experts of a stacked weight) with
    possibly different owners.
    """

    owner_style = True

    def __init__(self, segments: Sequence[tuple[int, int, int]], view_kind: str = "full_param"):
        if view_kind not in ("full_param", "expert_block"):
            raise ValueError(f"unknown view_kind {view_kind!r}")
        self.segments = tuple((int(r), int(s), int(l)) for r, s, l in segments)
        self.view_kind = view_kind
        pos = 0
        for _, s, l in sorted(self.segments, key=lambda t: t[1]):
            if s != pos or l <= 0:
                raise ValueError(f"segments must tile dim 0 exactly, got {self.segments}")
            pos += l
        self._extent = pos

    def __eq__(self, other):
        return isinstance(other, BucketedOwned) and (other.segments, other.view_kind) == (self.segments, self.view_kind)

    def __hash__(self):
        return hash(("BucketedOwned", self.segments, self.view_kind))

    def __repr__(self):
        return f"BucketedOwned(segments={self.segments}, view_kind={self.view_kind!r})"

    @property
    def owners(self) -> tuple[int, ...]:
        return tuple(sorted({r for r, _, _ in self.segments}))

    def pieces(self, global_shape, rank, world_size):
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

        _, _, W, _ = mesh_group(mesh)
        hosts = mesh_rank_hosts(W, ranks_per_host)
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
