"""Adapter: parameters that are DTensors of an outer (TP/EP) sharding become plain local tensors
that declare where they sit in the full parameter, ready for ``flex_shard``.

Parity: ``layout_adapters/dtensor.py:24-64`` of the reference.
"""
from __future__ import annotations

import torch.nn as nn

from ..placement_contract import GlobalLayout, set_global_layout


def dtensor_layout(dt) -> GlobalLayout:
    """``GlobalLayout`` of a DTensor's local shard (``Shard`` / ``Replicate`` placements, even or
    uneven chunks as ``torch.chunk`` cuts them; a rank without rows gets a layout without boxes).  Any other
    placement (``Partial``, strided shards) raises ``NotImplementedError`` naming it."""
    from torch.distributed.tensor import Replicate, Shard

    try:
        from torch.distributed.tensor.placement_types import _StridedShard
    except ImportError:                       # older layouts of the module
        _StridedShard = ()
    shape = tuple(dt.shape)
    off = [0] * len(shape)
    size = list(shape)
    mesh = dt.device_mesh
    coord = mesh.get_coordinate()
    for mdim, pl in enumerate(dt.placements):
        if isinstance(pl, Replicate):
            continue
        if (_StridedShard and isinstance(pl, _StridedShard)) or not isinstance(pl, Shard):
            raise NotImplementedError(f"a DTensor parameter with placements {dt.placements!r} cannot be declared as an "
                                      "outer layout (Shard and Replicate only)")
        n = mesh.size(mdim)
        r = coord[mdim]
        chunk = -(-size[pl.dim] // n)
        lo = min(size[pl.dim], r * chunk)
        hi = min(size[pl.dim], (r + 1) * chunk)
        off[pl.dim] += lo
        size[pl.dim] = hi - lo
    if any(n == 0 for n in size):
        return GlobalLayout(shape, (), (), ())
    return GlobalLayout(shape, (tuple(off),), ((0,) * len(shape),), (tuple(size),))


def dtensor_to_global_layout(module: nn.Module) -> nn.Module:
    """Replace every DTensor parameter by its local tensor tagged with its layout: call it before ``flex_shard`` on
    a model whose parameters are already DTensors (after tensor or expert parallelism).  A parameter's explicit
    ``grad_dtype`` is kept, and a parameter used under several names stays one parameter."""
    from torch.distributed.tensor import DTensor

    done: dict[int, nn.Parameter] = {}
    for mod in module.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            dt = p if isinstance(p, DTensor) else getattr(p, "data", None)
            if not isinstance(dt, DTensor):
                continue
            local = done.get(id(p))
            if local is None:
                local = nn.Parameter(dt.to_local().detach().contiguous(), requires_grad=p.requires_grad)
                grad_dtype = getattr(p, "grad_dtype", None)
                if grad_dtype is not None and grad_dtype != local.dtype:
                    local.grad_dtype = grad_dtype
                set_global_layout(local, dtensor_layout(dt))
                done[id(p)] = local
            mod._parameters[name] = local
    return module
