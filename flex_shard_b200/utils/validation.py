"""Host-side helpers: gradient buffers in parameter layout, host maps, LPT balancing.

Parity: ``flex_shard/utils.py:369-482`` of the reference (``alloc_grads_in_param_layout``,
``mesh_rank_hosts``, ``assign_to_hosts_then_ranks``).
"""
from __future__ import annotations

import os
from typing import Sequence

import torch


def alloc_grads_in_param_layout(storage) -> None:
    """Give every unsharded parameter of ``storage`` a ``.grad`` that is a view of one
    bucket-shaped buffer (the Megatron ``main_grad`` idea), so the reduction can send the
    buffer as it is. No-op when the grads already exist.  Usable as a ``BucketSpec.pre_backward_hook`` as it is (a
    hook's argument carries the storage)."""
    storage = getattr(storage, "storage", storage)
    rt = storage.runtime
    if rt is None or rt.unsharded_params is None:
        return
    ups = [u for u, i in zip(rt.unsharded_params, storage.infos) if i.requires_grad and u.requires_grad]
    if not ups or all(u.grad is not None for u in ups):
        return
    placement = storage.placement
    if hasattr(placement, "alloc_grad_bucket"):
        placement.alloc_grad_bucket(storage, rt.unsharded_params)
        return
    total = sum(u.numel() for u in ups)
    dtype = ups[0].dtype
    buf = torch.zeros(total, dtype=dtype, device=ups[0].device)
    off = 0
    for u in ups:
        n = u.numel()
        if u.grad is None:
            u.grad = buf[off:off + n].view(u.shape)
        off += n


def mesh_rank_hosts(world_size: int, ranks_per_host: int | None = None) -> tuple[int, ...]:
    """Host index of each mesh rank, from ``LOCAL_WORLD_SIZE`` (torchrun) unless given."""
    if ranks_per_host is None:
        ranks_per_host = int(os.environ.get("LOCAL_WORLD_SIZE", world_size))
    ranks_per_host = max(1, min(ranks_per_host, world_size))
    return tuple(r // ranks_per_host for r in range(world_size))


def assign_to_hosts_then_ranks(costs: Sequence[float], hosts: Sequence[int],
                               loads: Sequence[float] | None = None) -> list[int]:
    """Longest-processing-time assignment of items to ranks: pick the least-loaded host first,
    then the least-loaded rank on it. Ties prefer even positions first (0, 2, 4, ..., 1, 3, ...)
    so consecutive items spread over NVLink domains / NICs. ``loads`` carries earlier
    assignments in (and is updated in place when it is a list)."""
    W = len(hosts)
    rank_load = list(loads) if loads is not None else [0.0] * W
    host_ids = sorted(set(hosts))
    host_ranks = {h: [r for r in range(W) if hosts[r] == h] for h in host_ids}

    def tie_order(seq):
        return {v: i for i, v in enumerate(list(seq[0::2]) + list(seq[1::2]))}

    host_tie = tie_order(host_ids)
    rank_tie = {h: tie_order(rs) for h, rs in host_ranks.items()}
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    out = [0] * len(costs)
    for i in order:
        h = min(host_ids, key=lambda x: (sum(rank_load[r] for r in host_ranks[x]), host_tie[x]))
        r = min(host_ranks[h], key=lambda x: (rank_load[x], rank_tie[h][x]))
        out[i] = r
        rank_load[r] += costs[i]
    if isinstance(loads, list):
        loads[:] = rank_load
    return out
