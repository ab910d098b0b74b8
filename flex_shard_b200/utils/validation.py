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


def mesh_rank_hosts(world_size, ranks_per_host: int | None = None) -> tuple[int, ...]:
    """Host index of each mesh rank.  ``world_size`` an int: ranks 0..world_size-1 in hosts of ``ranks_per_host``
    (default ``LOCAL_WORLD_SIZE`` as torchrun sets it, else one host).  ``world_size`` a sequence: the mesh's global
    ranks in mesh order, the reference's form (``flex_shard/utils.py:393-410`` there); hosts are numbered in order of
    first appearance and without ``ranks_per_host`` or ``LOCAL_WORLD_SIZE`` every rank is its own host."""
    if isinstance(world_size, int):
        if ranks_per_host is None:
            ranks_per_host = int(os.environ.get("LOCAL_WORLD_SIZE", world_size))
        ranks_per_host = max(1, min(ranks_per_host, world_size))
        return tuple(r // ranks_per_host for r in range(world_size))
    if ranks_per_host is None:
        ranks_per_host = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
    if ranks_per_host <= 0:
        raise ValueError(f"ranks_per_host must be positive, got {ranks_per_host}")
    seen: dict[int, int] = {}
    return tuple(seen.setdefault(int(r) // ranks_per_host, len(seen)) for r in world_size)


def _even_positions_first(seq):
    return {v: i for i, v in enumerate(list(seq[0::2]) + list(seq[1::2]))}


def assign_to_hosts_then_ranks(costs: Sequence[float], hosts: Sequence[int],
                               loads: Sequence[float] | None = None, *,
                               carried_loads: Sequence[float] | None = None, one_per_rank: bool = False) -> list[int]:
    """Longest-processing-time assignment of items to ranks: pick the least-loaded host first,
    then the least-loaded rank on it. Ties prefer even positions first (0, 2, 4, ..., 1, 3, ...)
    so consecutive items spread over NVLink domains / NICs.

    ``loads`` carries earlier assignments in as part of the load itself (and is updated in place when it is a list):
    successive calls then approach one global balance.  ``carried_loads`` is the reference's rule instead
    (``flex_shard/utils.py:420-482`` there): every call balances what it places by itself and earlier loads only break
    ties (host: placed by this call, then carried; rank likewise); with ``one_per_rank`` a rank takes at most one
    item."""
    W = len(hosts)
    host_ids = sorted(set(hosts))
    host_ranks = {h: [r for r in range(W) if hosts[r] == h] for h in host_ids}
    host_tie = _even_positions_first(host_ids)
    rank_tie = {h: _even_positions_first(rs) for h, rs in host_ranks.items()}
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    out = [0] * len(costs)
    if carried_loads is not None or one_per_rank:
        if loads is not None:
            raise ValueError("give either loads (added to the load) or carried_loads (tie-break only)")
        if host_ids != list(range(len(host_ids))):
            raise ValueError(f"hosts must be numbered 0, 1, ..., got {tuple(hosts)}")
        if one_per_rank and len(costs) > W:
            raise ValueError(f"{len(costs)} items do not fit one per rank on {W} ranks")
        carried = [0.0] * W if carried_loads is None else list(carried_loads)
        if len(carried) != W:
            raise ValueError(f"carried_loads must give each of the {W} ranks a load")
        placed = [0.0] * W
        taken = [False] * W
        for i in order:
            open_hosts = [h for h in host_ids if not one_per_rank or not all(taken[r] for r in host_ranks[h])]
            h = min(open_hosts, key=lambda x: (sum(placed[r] for r in host_ranks[x]),
                                               sum(carried[r] for r in host_ranks[x]), host_tie[x]))
            r = min((r for r in host_ranks[h] if not (one_per_rank and taken[r])),
                    key=lambda x: (placed[x], carried[x], rank_tie[h][x]))
            out[i], taken[r] = r, True
            placed[r] += costs[i]
        return out
    rank_load = list(loads) if loads is not None else [0.0] * W
    for i in order:
        h = min(host_ids, key=lambda x: (sum(rank_load[r] for r in host_ranks[x]), host_tie[x]))
        r = min(host_ranks[h], key=lambda x: (rank_load[x], rank_tie[h][x]))
        out[i] = r
        rank_load[r] += costs[i]
    if isinstance(loads, list):
        loads[:] = rank_load
    return out
