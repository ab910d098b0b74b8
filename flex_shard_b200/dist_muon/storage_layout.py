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


def _block_rows(table: Mapping[str, int] | None, fqn: str) -> int | None:
    """Rows of one orthogonalisation block for ``fqn``: keys are full names, fnmatch patterns, or the last
    component of the name (``"wq_b"`` matches ``"layers.3.attn.wq_b"``)."""
    import fnmatch

    for key, rows in (table or {}).items():
        if fqn == key or fqn.endswith("." + key) or fnmatch.fnmatchcase(fqn, key):
            return int(rows)
    return None


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
            head_rows = _block_rows(block_rows_by_fqn, info.fqn) if len(gshape) == 2 else None
            if head_rows is not None and gshape[0] % head_rows != 0:
                raise ValueError(f"{info.fqn!r}: {gshape[0]} rows are not whole blocks of {head_rows}")
            if W == 1 or isinstance(pl, BucketedOwned):
                # whole on this rank (a one-rank mesh stores every parameter whole, whatever the placement;
                # an owner holds all rows, everyone else none)
                if len(gshape) == 3 and (W == 1 or pl.view_kind == "expert_block"):
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                elif head_rows is not None:      # per-head orthogonalisation of a matrix stored whole
                    out[info.fqn] = LocalMuonComputeLayout(
                        "row_blocks", block_rows=(head_rows,) * (info.local_shape[0] // head_rows), global_shape=gshape)
                else:
                    out[info.fqn] = LocalMuonComputeLayout("owned", global_shape=gshape)
            elif isinstance(pl, BlockShard) and pl.dim == 0:
                if len(gshape) == 3:
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                else:
                    rows = head_rows or pl.block_size(gshape)
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
