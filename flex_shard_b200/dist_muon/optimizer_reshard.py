"""Public configuration records of DistMuon.

Parity: ``dist_muon/optimizer_reshard.py:35-312`` of the reference (``Owned``, ``BlockShard``,
``ComputeLayout``, ``BucketConfig``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Sequence


@dataclass(frozen=True)
class Owned:
    """Whole matrices on owner ranks. ``block_sizes``: sizes of the dim-0 blocks that are
    orthogonalised separately (``None``: the parameter is one matrix)."""

    block_sizes: tuple[int, ...] | None = None

    def to_dict(self):
        return {"kind": "owned", "block_sizes": self.block_sizes}


@dataclass(frozen=True)
class BlockShard:
    """Blocks of ``dim`` spread over the mesh axis; ``block_sizes`` repeats to cover the dim."""

    dim: int = 0
    block_sizes: tuple[int, ...] = ()

    def num_blocks(self, extent: int) -> int:
        period = sum(self.block_sizes)
        if period <= 0 or extent % period != 0:
            raise ValueError(f"block_sizes {self.block_sizes} do not tile an extent of {extent}")
        return extent // period * len(self.block_sizes)

    def block_start(self, index: int) -> int:
        period, n = sum(self.block_sizes), len(self.block_sizes)
        return index // n * period + sum(self.block_sizes[: index % n])

    def to_dict(self):
        return {"kind": "block_shard", "dim": self.dim, "block_sizes": self.block_sizes}


@dataclass(frozen=True)
class ComputeLayout:
    """How a parameter is laid out while Muon computes on it: one sharding per mesh axis name."""

    shardings_by_mesh_axis: Mapping[str, Owned | BlockShard] = field(default_factory=dict)
    shard_order_by_tensor_dim: Mapping[int, Sequence[str]] | None = None

    def to_dict(self):
        return {"shardings_by_mesh_axis": {k: v.to_dict() for k, v in self.shardings_by_mesh_axis.items()},
                "shard_order_by_tensor_dim": dict(self.shard_order_by_tensor_dim or {})}


@dataclass(frozen=True)
class BucketConfig:
    """Parameters (fnmatch patterns) that are redistributed and computed together."""

    patterns: tuple[str, ...]
    name: str | None = None

    def __post_init__(self):
        object.__setattr__(self, "patterns", tuple(self.patterns))
