"""Hidden sharding metadata carried by the local ``nn.Parameter`` views.

Parity: ``flex_shard/sharded_param.py:20-70`` of the reference (the five hidden
attributes and their getters).
"""
from __future__ import annotations

import torch

_ATTRS = ("_fsb_placements", "_fsb_global_shape", "_fsb_global_stride", "_fsb_mesh", "_fsb_outer_layout")


def set_sharding_info(param: torch.Tensor, placements=None, global_shape=None, global_stride=None, mesh=None,
                      outer_layout=None, *, placement=None) -> None:
    """Record how ``param`` is sharded.  ``placements``: the reference's one-element tuple (one entry per dimension of
    a 1-D mesh); ``placement=``: the bare placement."""
    if (placements is None) == (placement is None):
        raise TypeError("set_sharding_info takes either placements=(placement,) or placement=placement")
    if placements is not None:
        placements = tuple(placements)
        if len(placements) != 1:
            raise ValueError(f"flex_shard meshes are 1-D: expected one placement, got {len(placements)}")
        placement = placements[0]
    if global_shape is None:
        raise TypeError("set_sharding_info needs global_shape")
    if global_stride is None:
        raise TypeError("set_sharding_info needs global_stride")
    param._fsb_placements = (placement,)
    param._fsb_global_shape = tuple(global_shape)
    param._fsb_global_stride = tuple(global_stride)
    param._fsb_mesh = mesh
    param._fsb_outer_layout = outer_layout


def is_flex_shard_param(param: torch.Tensor) -> bool:
    return hasattr(param, "_fsb_placements")


def get_placements(param: torch.Tensor):
    return getattr(param, "_fsb_placements", None)


def get_global_shape(param: torch.Tensor):
    return getattr(param, "_fsb_global_shape", None)


def get_global_stride(param: torch.Tensor):
    return getattr(param, "_fsb_global_stride", None)


def get_mesh(param: torch.Tensor):
    return getattr(param, "_fsb_mesh", None)


def get_outer_layout(param: torch.Tensor):
    return getattr(param, "_fsb_outer_layout", None)
