"""``MixedBucketPlacement``: one all-gather and one reduce-scatter for a bucket that mixes
``Shard(0)``-style, ``BlockShard`` and ``BucketedOwned`` members (and dtypes).

Every member is a slice placement, so the shared row engine (``placements/sliced.py``) plans one
row per rank ``[owner-exclusive region | regular slots]``, gathers rows as bytes and reduces rows in
the bucket's reduce dtype. This class only adapts a member placement to that engine.

Parity: ``custom_placements/mixed_bucket.py:173-365`` (member wrappers) and ``:663-684``
(one collective per bucket) of the reference.
"""
from __future__ import annotations

from .shard import Shard
from .sliced import Piece, SlicedPlacement


class ShardSlice(SlicedPlacement):
    """``Shard(dim)`` geometry expressed as a slice placement (member of a mixed bucket)."""

    def __init__(self, dim: int = 0):
        self.dim = int(dim)
        self._shard = Shard(dim)

    def __eq__(self, other):
        return isinstance(other, ShardSlice) and other.dim == self.dim

    def __hash__(self):
        return hash(("ShardSlice", self.dim))

    def __repr__(self):
        return f"ShardSlice({self.dim})"

    def pieces(self, global_shape, rank, world_size):
        self._shard._check(global_shape, world_size)
        lo, hi = self._shard._range(global_shape[self.dim], rank, world_size)
        return [Piece(self.dim, lo, hi - lo)] if hi > lo else []


class MixedBucketPlacement(SlicedPlacement):
    """Wraps one member placement of a mixed bucket.

    ``MixedBucketPlacement({fqn: [BucketedOwnedSegmentSpec]})``, the reference's form
    (``custom_placements/mixed_bucket.py`` there), describes the bucket's owned parameters instead and hands out the
    members: ``.shard0``, ``.block_shard(blocks_per_rank, dim=0)`` and ``.bucketed_owned`` (narrowed to each
    parameter's own segments when ``flex_shard`` applies it)."""

    def __init__(self, member):
        from collections.abc import Mapping

        self._segments_by_fqn = None
        if isinstance(member, Mapping):
            from .owned import BucketedOwned

            self._segments_by_fqn = dict(member)
            member = BucketedOwned(self._segments_by_fqn) if self._segments_by_fqn else ShardSlice(0)
        if isinstance(member, Shard):
            member = ShardSlice(member.dim)
        if not isinstance(member, SlicedPlacement):
            raise TypeError(f"{member!r} cannot be a member of a mixed bucket")
        self.member = member
        self.owner_style = getattr(member, "owner_style", False)

    # ---- the reference's way of building the members of one bucket
    @property
    def shard0(self) -> "MixedBucketPlacement":
        return MixedBucketPlacement(Shard(0))

    def block_shard(self, blocks_per_rank, dim: int = 0) -> "MixedBucketPlacement":
        from .block_shard import BlockShard

        return MixedBucketPlacement(BlockShard(tuple(blocks_per_rank), dim))

    @property
    def bucketed_owned(self) -> "MixedBucketPlacement":
        from .owned import BucketedOwned

        if not self._segments_by_fqn:
            raise ValueError("this MixedBucketPlacement was built without owner segments")
        return MixedBucketPlacement(BucketedOwned(self._segments_by_fqn))

    def for_param(self, fqn: str, shape) -> "MixedBucketPlacement":
        narrow = getattr(self.member, "for_param", None)
        if narrow is None:
            return self
        member = narrow(fqn, shape)
        return self if member is self.member else MixedBucketPlacement(member)

    def __eq__(self, other):
        return isinstance(other, MixedBucketPlacement) and other.member == self.member

    def __hash__(self):
        return hash(("Mixed", self.member))

    def __repr__(self):
        return f"MixedBucketPlacement({self.member!r})"

    def pieces(self, global_shape, rank, world_size):
        return self.member.pieces(global_shape, rank, world_size)

    def reduces_grads_in_param_layout(self, infos) -> bool:
        """When every member of the bucket is whole on one owner and nothing casts between the gradient and the
        reduce dtype, the gradients may be views of one buffer in parameter order that autograd accumulates
        into (parity: ``custom_placements/mixed_bucket.py:1262-1282`` of the reference: all members one-hot
        owned, one dtype for gathered parameters, gradient accumulation and reduction)."""
        dtypes = {i.param_dtype for i in infos}
        return (len(dtypes) == 1 and all(
            getattr(getattr(i.placement, "member", None), "owner_style", False)
            and i.param_dtype == (i.bucket_reduce_dtype or i.reduce_dtype) for i in infos))


def make_mixed_placement_fn(member_fn, blocks_per_rank_by_fqn=None):
    """Wrap the placements returned by ``member_fn`` so that they may share one bucket.

    Also takes the reference's form ``make_mixed_placement_fn(owned_rank_by_fqn, blocks_per_rank_by_fqn)``
    (``dist_muon/placement.py:164-199`` there): the named parameters are whole on their owner rank, or stored in
    whole dim-0 blocks with the given blocks per rank; every other parameter of the bucket is ``Shard(0)``."""
    from collections.abc import Mapping

    if isinstance(member_fn, Mapping):
        owned, blocks = dict(member_fn), dict(blocks_per_rank_by_fqn or {})

        def by_name(named_params, mesh):
            from .block_shard import BlockShard
            from .owned import BucketedOwned

            out = {}
            for f, p in named_params:
                if f in blocks:
                    out[f] = MixedBucketPlacement(BlockShard(tuple(blocks[f]), 0))
                elif f in owned:
                    out[f] = MixedBucketPlacement(BucketedOwned(((int(owned[f]), 0, p.shape[0]),)))
                else:
                    out[f] = MixedBucketPlacement(Shard(0))
            return out

        return by_name

    def fn(named_params, mesh):
        return {f: MixedBucketPlacement(pl) for f, pl in member_fn(named_params, mesh).items()}

    return fn
