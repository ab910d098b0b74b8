"""Adapter: parameters that are DTensors of an outer (TP/EP) sharding become plain local tensors
that declare where they sit in the full parameter, ready for ``flex_shard``.

Parity: ``layout_adapters/dtensor.py:24-64`` of the reference.
"""
from __future__ import annotations

import torch.nn as nn

from ..placement_contract import GlobalLayout, set_global_layout


def dtensor_layout(dt) -> GlobalLayout:
    """``GlobalLayout`` of a DTensor's local shard (``Shard`` / ``Replicate`` placements, even or
    uneven chunks as ``torch.chunk`` cuts them)."""
    from torch.distributed.tensor import Replicate, Shard

    shape = tuple(dt.shape)
    off = [0] * len(shape)
    size = list(shape)
    mesh = dt.device_mesh
    coord = mesh.get_coordinate()
    for mdim, pl in enumerate(dt.placements):
        if isinstance(pl, Replicate):
            continue
        if not isinstance(pl, Shard):
            raise ValueError(f"unsupported DTensor placement {pl!r} for an outer layout")
        n = mesh.size(mdim)
        r = coord[mdim]
        chunk = -(-size[pl.dim] // n)
        lo = min(size[pl.dim], r * chunk)
        hi = min(size[pl.dim], (r + 1) * chunk)
        off[pl.dim] += lo
        size[pl.dim] = hi - lo
    return GlobalLayout(shape, (tuple(off),), ((0,) * len(shape),), (tuple(size),))


def dtensor_to_global_layout(module: nn.Module) -> nn.Module:
    """Replace every DTensor parameter by its local tensor (same storage) tagged with its layout."""
    from torch.distributed.tensor import DTensor

    for mod in module.modules():
        for name, p in list(mod._parameters.items()):
            if isinstance(p, DTensor):
                local = nn.Parameter(p.to_local(), requires_grad=p.requires_grad)
                set_global_layout(local, dtensor_layout(p))
                mod._parameters[name] = local
            elif p is not None and isinstance(getattr(p, "data", None), DTensor):
                local = nn.Parameter(p.data.to_local(), requires_grad=p.requires_grad)
                set_global_layout(local, dtensor_layout(p.data))
                mod._parameters[name] = local
    return module
