"""Bridge from FlexShard storage placements to DistMuon's local compute layouts.

Parity: ``dist_muon/storage_layout.py:57-165`` of the reference
(``capture_flex_shard_muon_canonical_shards``, ``get_flex_shard_muon_compute_layouts``,
``LocalMuonComputeLayout`` kinds owned / row_blocks / matrix_batch / row_shard).
"""
from __future__ import annotations

from typing import Mapping

import torch.nn as nn

from ..placements.block_shard import BlockShard
from ..placements.mixed_bucket import MixedBucketPlacement, ShardSlice
from ..placements.owned import BucketedOwned
from ..placements.shard import Shard
from .optimizer import LocalMuonComputeLayout


def capture_flex_shard_muon_canonical_shards(module: nn.Module) -> dict[str, tuple[int, ...]]:
    """Shapes of the parameters before ``flex_shard`` (their canonical, outer coordinates)."""
    return {n: tuple(p.shape) for n, p in module.named_parameters()}


def _unwrap(pl):
    return pl.member if isinstance(pl, MixedBucketPlacement) else pl


def get_flex_shard_muon_compute_layouts(module: nn.Module,
                                        block_rows_by_fqn: Mapping[str, int] | None = None
                                        ) -> dict[str, LocalMuonComputeLayout]:
    """One ``LocalMuonComputeLayout`` per managed parameter, from its storage placement.

    ``block_rows_by_fqn``: rows of one orthogonalisation block for ``BlockShard(dim=0)`` storage
    (default: the placement's block size, i.e. each stored block is one matrix).
    """
    out: dict[str, LocalMuonComputeLayout] = {}
    for st in module.sharded_bucket_storages:
        W, rank = st.comm.world_size, st.comm.rank
        for info in st.infos:
            pl = _unwrap(info.placement)
            gshape = tuple(info.global_shape)
            if W == 1:
                # a one-rank mesh stores every parameter whole, whatever the placement
                out[info.fqn] = LocalMuonComputeLayout("matrix_batch" if len(gshape) == 3 else "owned",
                                                       global_shape=gshape)
            elif isinstance(pl, BucketedOwned):
                if pl.view_kind == "expert_block" and len(gshape) == 3:
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                else:
                    out[info.fqn] = LocalMuonComputeLayout("owned", global_shape=gshape)
            elif isinstance(pl, BlockShard) and pl.dim == 0:
                if len(gshape) == 3:
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                else:
                    rows = (block_rows_by_fqn or {}).get(info.fqn, pl.block_size(gshape))
                    n_local = info.local_shape[0] // rows if rows else 0
                    out[info.fqn] = LocalMuonComputeLayout("row_blocks", block_rows=(rows,) * n_local,
                                                           global_shape=gshape)
            elif isinstance(pl, (Shard, ShardSlice)) and pl.dim == 0:
                if W == 1:
                    out[info.fqn] = LocalMuonComputeLayout("owned", global_shape=gshape)
                else:
                    lo, hi = Shard(0)._range(gshape[0], rank, W)
                    out[info.fqn] = LocalMuonComputeLayout("row_shard", global_shape=gshape, row_range=(lo, hi))
            else:
                raise ValueError(f"DistMuon has no compute layout for {info.fqn!r} stored as {pl!r}")
    return out
