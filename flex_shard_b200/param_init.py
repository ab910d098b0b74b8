"""RNG-exact initialisation of sharded parameters.

``init_from_full`` builds the full tensor on every rank (same RNG stream, so the
generator advances exactly as in an unsharded run), applies ``init_fn`` and keeps
this rank's boxes. Parity: ``flex_shard/param_init.py:18-49`` of the reference.
"""
from __future__ import annotations

from typing import Callable

import torch

from .placement_contract import GlobalLayout
from .sharded_param import is_flex_shard_param


@torch.no_grad()
def init_from_full(param: torch.Tensor, layout_or_init_fn, init_fn: Callable[[torch.Tensor], object] | None = None) -> None:
    """``init_from_full(param, init_fn)``: the layout is the one ``flex_shard`` recorded for ``param`` (a plain tensor
    is initialised directly).  ``init_from_full(local, layout, init_fn)``, the reference's form: ``layout`` (a
    ``GlobalLayout``, e.g. from ``get_flex_shard_global_layouts``) says where ``local`` sits in the full tensor."""
    if init_fn is None:
        init_fn = layout_or_init_fn
        if not callable(init_fn):
            raise TypeError("init_from_full(param, init_fn) or init_from_full(local, layout, init_fn)")
        if not is_flex_shard_param(param):
            init_fn(param)
            return
        layout = param._fsb_storage.global_layout_of(param._fsb_info)
    else:
        layout = layout_or_init_fn
        if not isinstance(layout, GlobalLayout):
            raise TypeError(f"layout must be a GlobalLayout, got {type(layout).__name__}")
    full = torch.empty(layout.global_shape, dtype=param.dtype, device=param.device)
    init_fn(full)
    for goff, loff, size in zip(layout.global_offsets, layout.local_offsets, layout.local_sizes):
        src, dst = full, param
        for d, (g, l, s) in enumerate(zip(goff, loff, size)):
            src = src.narrow(d, g, s)
            dst = dst.narrow(d, l, s)
        dst.copy_(src)
