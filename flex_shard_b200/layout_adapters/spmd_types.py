"""Adapter for SPMD-typed parameters: any object that carries per-mesh-axis sharding annotations
(``param.spmd_sharding = {axis_name: ("shard", dim) | ("replicate",) | ("partial",)}`` together
with ``param.spmd_mesh = {axis_name: (rank, size)}``) is turned into a ``GlobalLayout`` and, for
partial axes, a partial-gradient group.

Parity: ``layout_adapters/spmd_types.py:20-127`` of the reference (there the annotations come from
the external ``spmd_types`` package; the contract kept here is the same: sharded axes compose into a
global layout, ``Partial`` gradients are summed over their group before the reduce-scatter).
"""
from __future__ import annotations

from typing import Mapping

import torch.nn as nn

from ..placement_contract import GlobalLayout, set_global_layout, set_partial_grad_group


def spmd_layout(local_shape, sharding: Mapping[str, tuple], mesh: Mapping[str, tuple[int, int]],
                shard_order: Mapping[int, tuple[str, ...]] | None = None) -> GlobalLayout:
    """Even shards only: axis ``a`` with ``("shard", d)`` multiplies dim ``d`` by the axis size; the
    order of several axes on one dim follows ``shard_order[d]`` (outermost first)."""
    gshape = list(local_shape)
    off = [0] * len(gshape)
    by_dim: dict[int, list[str]] = {}
    for axis, spec in sharding.items():
        if spec[0] == "shard":
            by_dim.setdefault(spec[1], []).append(axis)
    for d, axes in by_dim.items():
        order = list((shard_order or {}).get(d, axes))
        stride = local_shape[d]
        for axis in reversed(order):
            rank, size = mesh[axis]
            off[d] += rank * stride
            stride *= size
        gshape[d] = stride
    nd = len(gshape)
    return GlobalLayout(tuple(gshape), (tuple(off),), ((0,) * nd,), (tuple(local_shape),))


def spmd_types_to_global_layout(module: nn.Module, groups: Mapping[str, object] | None = None) -> nn.Module:
    for p in module.parameters():
        sharding = getattr(p, "spmd_sharding", None)
        if not sharding:
            continue
        mesh = p.spmd_mesh
        set_global_layout(p, spmd_layout(tuple(p.shape), sharding, mesh, getattr(p, "spmd_shard_order", None)))
        for axis, spec in sharding.items():
            if spec[0] == "partial":
                if not groups or axis not in groups:
                    raise ValueError(f"parameter has a partial gradient over axis {axis!r} but no group was given")
                set_partial_grad_group(p, groups[axis])
    return module
