"""Placement helpers for DistMuon recipes. Parity: ``dist_muon/placement.py:26-222`` of the reference."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

from ..placements.block_shard import BlockShard
from ..placements.mixed_bucket import make_mixed_placement_fn
from ..placements.shard import shard_placement_fn


@dataclass(frozen=True)
class BlockShardPlan:
    blocks_per_rank: tuple[int, ...]
    block_rows: int

    def rows_of(self, rank: int) -> int:
        return self.blocks_per_rank[rank] * self.block_rows


def get_mesh_rank_groups(world_size: int, group_size: int) -> list[list[int]]:
    return [list(range(i, i + group_size)) for i in range(0, world_size, group_size)]


def get_dim0_block_partitions(num_blocks: int, world_size: int) -> tuple[int, ...]:
    base, rem = divmod(num_blocks, world_size)
    return tuple(base + (1 if r < rem else 0) for r in range(world_size))


def make_bucketed_block_placement_fn(num_blocks_of):
    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        return {n: BlockShard(get_dim0_block_partitions(num_blocks_of(n, p), W), 0) for n, p in named_params}

    return fn


shard0_placement_fn = shard_placement_fn(0)
__all__ = ["BlockShardPlan", "get_mesh_rank_groups", "get_dim0_block_partitions", "make_mixed_placement_fn",
           "shard0_placement_fn", "make_bucketed_block_placement_fn"]
