"""Bridge from FlexShard storage placements to DistMuon's local compute layouts.

Parity: ``dist_muon/storage_layout.py:57-165`` of the reference
(``capture_flex_shard_muon_canonical_shards``, ``get_flex_shard_muon_compute_layouts``,
``LocalMuonComputeLayout`` kinds owned / row_blocks / matrix_batch / row_shard).
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch.nn as nn

from ..placements.block_shard import BlockShard
from ..placements.bucketed_block_shard import BucketedBlockShard
from ..placements.mixed_bucket import MixedBucketPlacement, ShardSlice
from ..placements.owned import BucketedOwned
from ..placements.shard import Shard
from .optimizer import LocalMuonComputeLayout


def capture_flex_shard_muon_canonical_shards(module: nn.Module) -> dict[str, tuple[int, ...]]:
    """Shapes of the parameters before ``flex_shard`` (their canonical, outer coordinates)."""
    return {n: tuple(p.shape) for n, p in module.named_parameters()}


def _unwrap(pl):
    return pl.member if isinstance(pl, MixedBucketPlacement) else pl


def _block_rows(table: Mapping[str, int | Sequence[int]] | None, fqn: str) -> tuple[int, ...] | None:
    """Rows of the orthogonalisation blocks of ``fqn`` as one period of a repeating pattern: ``16`` -> ``(16,)``
    (every 16 rows one matrix), ``(16, 8)`` -> a 16-row matrix, an 8-row matrix, and so on down the rows (a head's
    no-position and rotary parts as separate matrices).  Keys are full names, fnmatch patterns, or the last
    component of the name (``"wq_b"`` matches ``"layers.3.attn.wq_b"``)."""
    import fnmatch

    for key, rows in (table or {}).items():
        if fqn == key or fqn.endswith("." + key) or fnmatch.fnmatchcase(fqn, key):
            pattern = (int(rows),) if isinstance(rows, int) else tuple(int(r) for r in rows)
            if not pattern or any(r <= 0 for r in pattern):
                raise ValueError(f"{fqn!r}: block rows must be positive integers, got {rows!r}")
            return pattern
    return None


def _repeat(fqn: str, pattern: tuple[int, ...], local_rows: int) -> tuple[int, ...]:
    period = sum(pattern)
    if local_rows % period != 0:
        raise ValueError(f"{fqn!r}: the {local_rows} rows stored on this rank are not whole repetitions of the "
                         f"blocks {pattern} (period {period}); store whole periods per rank")
    return pattern * (local_rows // period)


def get_flex_shard_muon_compute_layouts(module: nn.Module,
                                        block_rows_by_fqn: Mapping[str, int | Sequence[int]] | None = None
                                        ) -> dict[str, LocalMuonComputeLayout]:
    """One ``LocalMuonComputeLayout`` per managed parameter, from its storage placement.

    ``block_rows_by_fqn``: rows of one orthogonalisation block of a 2-D parameter stored whole or as
    ``BlockShard(dim=0)`` (default: the placement's block size, i.e. each stored block is one matrix), or a tuple
    of rows that repeats down the parameter (``(nope, rope)``: two matrices per attention head; parity:
    ``BlockShard(dim=0, block_sizes=(16, 8))`` of the reference's ``examples/deepseek_v3/muon.py:29-48``).
    """
    out: dict[str, LocalMuonComputeLayout] = {}
    for st in module.sharded_bucket_storages:
        W, rank = st.comm.world_size, st.comm.rank
        for info in st.infos:
            pl = _unwrap(info.placement)
            gshape = tuple(info.global_shape)
            head_rows = _block_rows(block_rows_by_fqn, info.fqn) if len(gshape) == 2 else None
            if head_rows is not None and gshape[0] % sum(head_rows) != 0:
                raise ValueError(f"{info.fqn!r}: {gshape[0]} rows are not whole blocks of "
                                 f"{head_rows[0] if len(head_rows) == 1 else head_rows}")
            if W == 1 or isinstance(pl, BucketedOwned):
                # whole on this rank (a one-rank mesh stores every parameter whole, whatever the placement;
                # an owner holds all rows, everyone else none)
                if len(gshape) == 3 and (W == 1 or pl.view_kind == "expert_block"):
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                elif head_rows is not None:      # per-head orthogonalisation of a matrix stored whole
                    out[info.fqn] = LocalMuonComputeLayout(
                        "row_blocks", block_rows=_repeat(info.fqn, head_rows, info.local_shape[0]), global_shape=gshape)
                else:
                    out[info.fqn] = LocalMuonComputeLayout("owned", global_shape=gshape)
            elif isinstance(pl, BlockShard) and pl.dim == 0:
                if len(gshape) == 3:
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                else:
                    pattern = head_rows or ((pl.block_size(gshape),) if pl.block_size(gshape) else None)
                    blocks = _repeat(info.fqn, pattern, info.local_shape[0]) if pattern else ()
                    out[info.fqn] = LocalMuonComputeLayout("row_blocks", block_rows=blocks, global_shape=gshape)
            elif isinstance(pl, BucketedBlockShard):
                # a flat block bucket cuts every parameter on whole dim-0 entries: whole matrices of a stacked
                # weight (experts), whole rows of a 2-D one
                if len(gshape) >= 3:
                    out[info.fqn] = LocalMuonComputeLayout("matrix_batch", global_shape=gshape)
                elif head_rows is not None:
                    out[info.fqn] = LocalMuonComputeLayout(
                        "row_blocks", block_rows=_repeat(info.fqn, head_rows, info.local_shape[0]), global_shape=gshape)
                else:
                    raise ValueError(f"{info.fqn!r} is stored in a flat block bucket, which cuts a 2-D parameter between "
                                     "any two rows: give its block rows (block_rows_by_fqn) or store it another way")
            elif isinstance(pl, (Shard, ShardSlice)) and pl.dim == 0:
                if W == 1:
                    out[info.fqn] = LocalMuonComputeLayout("owned", global_shape=gshape)
                else:
                    lo, hi = Shard(0)._range(gshape[0], rank, W)
                    out[info.fqn] = LocalMuonComputeLayout("row_shard", global_shape=gshape, row_range=(lo, hi))
            else:
                raise ValueError(f"DistMuon has no compute layout for {info.fqn!r} stored as {pl!r}")
    return out
