"""``build_local_dist_muon``: DistMuon over each rank's own storage, no process group involved.

The reference wraps local shards as replicated DTensors on a one-rank gloo mesh so its
DTensor-based optimizer can run without NCCL groups (``dist_muon/comm_free_adapter.py:134-256``);
this implementation's optimizer takes plain local tensors, so the adapter only selects the
matrix parameters, derives their compute layouts from the storage placements and checks that
none of them needs redistribution.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch.nn as nn

from .optimizer import DistMuon
from .storage_layout import get_flex_shard_muon_compute_layouts


def build_local_dist_muon(module: nn.Module, *, is_muon_param: Callable[[str, nn.Parameter], bool] | None = None,
                          block_rows_by_fqn: Mapping[str, int] | None = None, **muon_kwargs) -> DistMuon:
    """DistMuon over the local shards of ``module``'s matrix parameters; raises if any of them is
    stored in a layout that would need communication (``Shard(0)`` on more than one rank)."""
    is_muon_param = is_muon_param or (lambda n, p: len(getattr(p, "_fsb_global_shape", p.shape)) >= 2)
    layouts = get_flex_shard_muon_compute_layouts(module, block_rows_by_fqn)
    names, params = [], []
    for n, p in module.named_parameters():
        if is_muon_param(n, p):
            lay = layouts.get(n)
            if lay is None:
                raise ValueError(f"{n!r} is not managed by flex_shard")
            if lay.kind == "row_shard":
                raise ValueError(
                    f"{n!r} is stored as Shard(0) on several ranks; store it with BucketedOwned/BlockShard "
                    "(relayout_bucket) for a communication-free Muon step, or use DistMuon with a group")
            names.append(n)
            params.append(p)
    return DistMuon(params, param_names=names, compute_layouts={n: layouts[n] for n in names}, **muon_kwargs)
