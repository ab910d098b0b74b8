"""RNG-exact initialisation of sharded parameters.

``init_from_full`` builds the full tensor on every rank (same RNG stream, so the
generator advances exactly as in an unsharded run), applies ``init_fn`` and keeps
this rank's boxes. Parity: ``flex_shard/param_init.py:18-49`` of the reference.
"""
from __future__ import annotations

from typing import Callable

import torch

from .sharded_param import is_flex_shard_param


@torch.no_grad()
def init_from_full(param: torch.Tensor, init_fn: Callable[[torch.Tensor], None]) -> None:
    if not is_flex_shard_param(param):
        init_fn(param)
        return
    storage = param._fsb_storage
    info = param._fsb_info
    layout = storage.global_layout_of(info)
    full = torch.empty(layout.global_shape, dtype=param.dtype, device=param.device)
    init_fn(full)
    for goff, loff, size in zip(layout.global_offsets, layout.local_offsets, layout.local_sizes):
        src, dst = full, param
        for d, (g, l, s) in enumerate(zip(goff, loff, size)):
            src = src.narrow(d, g, s)
            dst = dst.narrow(d, l, s)
        dst.copy_(src)
