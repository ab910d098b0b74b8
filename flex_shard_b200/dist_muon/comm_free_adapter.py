"""``build_local_dist_muon``: DistMuon over each rank's own storage, no process group involved.

The reference wraps local shards as replicated DTensors on a one-rank gloo mesh so its
DTensor-based optimizer can run without NCCL groups (``dist_muon/comm_free_adapter.py:134-256``);
this implementation's optimizer takes plain local tensors, so the adapter only selects the
matrix parameters, derives their compute layouts from the storage placements and checks that
none of them needs redistribution.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch
import torch.nn as nn

from .optimizer import DistMuon
from .storage_layout import get_flex_shard_muon_compute_layouts


def build_local_dist_muon(module: nn.Module, *, is_muon_param: Callable[[str, nn.Parameter], bool] | None = None,
                          block_rows_by_fqn: Mapping[str, int | tuple[int, ...]] | None = None, **muon_kwargs) -> DistMuon:
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


def muon_checkpoint_state(optimizer: DistMuon, module: nn.Module) -> dict:
    """The optimizer's state in checkpoint form: ``{"momentum": {fqn: tensor}, "param_groups": [...]}``.

    Momentum buffers live in each parameter's storage layout, so every buffer is tagged with its
    parameter's ``GlobalLayout`` and a checkpoint written from it reloads under another placement or world
    size like the parameter itself.  A parameter that has not been stepped yet contributes zeros, which
    keeps the set of keys the same on every rank.  Parity: the momentum translation of the reference's
    adapter (``dist_muon/comm_free_adapter.py:103-131,237-256``)."""
    from ..checkpoint import get_flex_shard_global_layouts
    from ..placement_contract import set_global_layout

    layouts = get_flex_shard_global_layouts(module)
    momentum = {}
    for group in optimizer.param_groups:
        for p in group["params"]:
            name = optimizer._name_of[id(p)]
            buf = optimizer.state[p].get("momentum_buffer") if p in optimizer.state else None
            t = buf if buf is not None else torch.zeros(p.shape, dtype=torch.float32, device=p.device)
            if name in layouts:
                set_global_layout(t, layouts[name])
            momentum[name] = t
    groups = [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
    return {"momentum": momentum, "param_groups": groups}


def load_muon_checkpoint_state(optimizer: DistMuon, state: Mapping) -> None:
    """Install a state produced by ``muon_checkpoint_state`` (after ``checkpoint.load`` filled its tensors)."""
    by_name = {optimizer._name_of[id(p)]: p for g in optimizer.param_groups for p in g["params"]}
    missing = sorted(set(by_name) - set(state["momentum"]))
    if missing:
        raise KeyError(f"checkpoint has no Muon momentum for {missing}")
    for name, p in by_name.items():
        t = state["momentum"][name]
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"momentum of {name!r} has shape {tuple(t.shape)}, parameter has {tuple(p.shape)}")
        optimizer.state[p]["momentum_buffer"] = t.detach().to(device=p.device, dtype=torch.float32).clone()
    for g, saved in zip(optimizer.param_groups, state.get("param_groups", [])):
        for k, v in saved.items():
            if k != "params" and k != "param_names":
                g[k] = tuple(v) if k == "ns_coefficients" else v
    optimizer._buckets = None
