"""``BlockShard``: whole blocks of a parameter along one dim (e.g. attention heads) per rank.

Parity: ``custom_placements/block_shard.py:89-534`` of the reference: ``blocks_per_rank`` blocks
of equal size along ``dim``; rank r stores blocks ``[sum(b[:r]), sum(b[:r+1]))`` compactly (the
parameter keeps its rank); gathers pad every rank's slot to ``max(blocks_per_rank)`` blocks.
"""
from __future__ import annotations

from typing import Sequence

from .sliced import Piece, SlicedPlacement


class BlockShard(SlicedPlacement):
    def __init__(self, blocks_per_rank: Sequence[int], dim: int = 0):
        self.blocks_per_rank = tuple(int(b) for b in blocks_per_rank)
        if any(b < 0 for b in self.blocks_per_rank) or sum(self.blocks_per_rank) <= 0:
            raise ValueError(f"blocks_per_rank must be non-negative with a positive sum, got {blocks_per_rank}")
        self.dim = int(dim)
        # a parameter that lives whole on one rank is packed in the owner region of mixed rows
        self.owner_style = sum(1 for b in self.blocks_per_rank if b > 0) == 1

    def __eq__(self, other):
        return isinstance(other, BlockShard) and (other.blocks_per_rank, other.dim) == (self.blocks_per_rank, self.dim)

    def __hash__(self):
        return hash(("BlockShard", self.blocks_per_rank, self.dim))

    def __repr__(self):
        return f"BlockShard(blocks_per_rank={self.blocks_per_rank}, dim={self.dim})"

    def block_size(self, global_shape) -> int:
        total = sum(self.blocks_per_rank)
        n = global_shape[self.dim]
        if n % total != 0:
            raise ValueError(f"dim {self.dim} of size {n} does not split into {total} equal blocks")
        return n // total

    def pieces(self, global_shape, rank, world_size):
        if len(self.blocks_per_rank) != world_size:
            raise ValueError(f"BlockShard has {len(self.blocks_per_rank)} ranks, the mesh has {world_size}")
        if self.dim >= len(global_shape):
            raise ValueError(f"BlockShard(dim={self.dim}) does not apply to shape {tuple(global_shape)}")
        b = self.block_size(global_shape)
        start = sum(self.blocks_per_rank[:rank]) * b
        length = self.blocks_per_rank[rank] * b
        return [Piece(self.dim, start, length)] if length > 0 else []


def make_block_shard_placement_fn(dim: int = 0, num_blocks_of=None):
    """Evenly spread ``num_blocks_of(fqn, param)`` blocks (default: size of ``dim``) over the mesh."""

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        out = {}
        for fqn, p in named_params:
            nb = num_blocks_of(fqn, p) if num_blocks_of else p.shape[dim]
            base, rem = divmod(nb, W)
            out[fqn] = BlockShard(tuple(base + (1 if r < rem else 0) for r in range(W)), dim)
        return out

    return fn
