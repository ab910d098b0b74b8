"""Sharded checkpoints: layout tagging plus a save/load that reshards by global offset.

Every tensor of a flex_shard ``state_dict()`` is a plain local shard. Tagging it
with its ``GlobalLayout`` (placement layout composed with any outer TP/EP layout)
makes a checkpoint loadable at another world size or under another placement:
``save`` writes each rank's tagged tensors to ``rank{r}.pt`` and ``load`` fills
every local box from whichever files overlap it.

Parity: ``flex_shard/checkpoint.py:26-161`` of the reference (the three public
helpers, Adam/AdamW optimizer hook, ``step`` left untagged). The reference hands
the tagged tensors to ``torch.distributed.checkpoint``; the installed PyTorch has
no ``CheckpointableTensor`` protocol, so the file format and the resharding reader
live here.
"""
from __future__ import annotations

import os
from typing import Any, Mapping

import torch
import torch.distributed as dist
import torch.nn as nn

from .placement_contract import GlobalLayout, get_global_layout, set_global_layout

_ADAM_STATE_KEYS = ("exp_avg", "exp_avg_sq", "max_exp_avg_sq")


_WRAPPER_PART = "_checkpoint_wrapped_module"


def _strip_wrapper_parts(fqn: str) -> str:
    """The name ``state_dict()`` shows for a parameter under activation-checkpoint wrappers (their
    state-dict hooks drop the wrapper's attribute from every key)."""
    return ".".join(part for part in fqn.split(".") if part != _WRAPPER_PART)


def _sharded_modules(module: nn.Module):
    """(prefix, sharded module) for ``module`` itself and for every sharded module below it, so that the
    helpers here work on a parent whose children went through ``flex_shard`` one by one."""
    for name, sub in module.named_modules(remove_duplicate=True):
        if isinstance(getattr(type(sub), "sharded_bucket_storages", None), property):
            yield (name + "." if name else ""), sub


def _storages_with_prefix(module: nn.Module):
    for prefix, sub in _sharded_modules(module):
        for st in sub.sharded_bucket_storages:
            yield prefix, sub, st


def get_flex_shard_global_layouts(module: nn.Module) -> dict[str, GlobalLayout]:
    """FQN -> layout for every managed parameter of ``module`` and of its sharded submodules, including the
    extra names of tied weights.  Names are relative to ``module``."""
    out: dict[str, GlobalLayout] = {}
    for prefix, _, st in _storages_with_prefix(module):
        for info in st.infos:
            lay = st.global_layout_of(info)
            out[prefix + info.fqn] = lay
            for other in info.shared_fqns:
                out[prefix + other] = lay
    return out


def set_state_dict_global_layouts(module: nn.Module, state_dict: Mapping[str, Any]) -> None:
    """Tag the tensors of ``module.state_dict()`` with their layouts (attributes do not survive a
    copy such as ``.to(dtype)``: tag again afterwards).  A parameter under an activation-checkpoint wrapper
    is found under the key without the wrapper's name; parameters missing from ``state_dict`` are skipped
    (parity: ``flex_shard/checkpoint.py:57-69`` of the reference)."""
    for fqn, lay in get_flex_shard_global_layouts(module).items():
        key = fqn if fqn in state_dict else _strip_wrapper_parts(fqn)
        v = state_dict.get(key)
        if isinstance(v, torch.Tensor):
            set_global_layout(v, lay)


def register_optimizer_checkpoint_hook(optimizer: torch.optim.Optimizer, module: nn.Module):
    """Tag Adam/AdamW state tensors in ``optimizer.state_dict()`` with their parameter's layout.
    ``step`` stays untagged (replicated).  Every parameter of the optimizer must be a sharded parameter of
    ``module``; a state tensor whose shape is not its parameter's local shape cannot be described and raises when
    the state dict is taken; registering again replaces the earlier hook.
    Parity: ``flex_shard/checkpoint.py`` of the reference (behaviours pinned by
    ``tests/test_flex_shard_checkpoint.py:275-378``)."""
    if not isinstance(optimizer, (torch.optim.Adam, torch.optim.AdamW)) and not getattr(
            optimizer, "_fsb_adam_like", False):
        raise NotImplementedError(
            f"register_optimizer_checkpoint_hook supports Adam and AdamW, got {type(optimizer).__name__}")
    layouts_by_param: dict[int, tuple[GlobalLayout, str]] = {}
    for prefix, _, st in _storages_with_prefix(module):
        for info, sp in zip(st.infos, st.sharded_params):
            layouts_by_param[id(sp)] = (st.global_layout_of(info), prefix + info.fqn)
    for g in optimizer.param_groups:
        for p in g["params"]:
            if id(p) not in layouts_by_param:
                raise ValueError(f"optimizer parameter of shape {tuple(p.shape)} is not a sharded parameter of the "
                                 "module; build the optimizer from module.parameters() after flex_shard()")
    old = getattr(optimizer, "_fsb_ckpt_hook", None)
    if old is not None:
        old.remove()

    def post_hook(opt, sd):
        idx = 0
        index_info = {}
        for g in opt.param_groups:
            for p in g["params"]:
                if id(p) in layouts_by_param:
                    index_info[idx] = (*layouts_by_param[id(p)], tuple(p.shape))
                idx += 1
        for pid, st in sd.get("state", {}).items():
            hit = index_info.get(pid)
            if hit is None:
                continue
            lay, fqn, shape = hit
            for key in _ADAM_STATE_KEYS:
                t = st.get(key)
                if isinstance(t, torch.Tensor):
                    if tuple(t.shape) != shape:
                        raise NotImplementedError(
                            f"optimizer state {key!r} of FlexShard parameter {fqn!r} has shape {tuple(t.shape)}, "
                            f"not the parameter's local shape {shape}: it cannot take the parameter's layout")
                    set_global_layout(t, lay)
        return sd

    handle = optimizer.register_state_dict_post_hook(post_hook)
    optimizer._fsb_ckpt_hook = handle
    return handle


# --------------------------------------------------------------------------- file format
def _flatten(d, prefix=""):
    out = {}
    if isinstance(d, Mapping):
        for k, v in d.items():
            out.update(_flatten(v, f"{prefix}{k}/" if isinstance(v, (Mapping,)) else f"{prefix}{k}"))
    else:
        out[prefix] = d
    return out


class PerRank:
    """Marks a non-tensor value of a state dict that differs between ranks (a data loader's position, a
    generator state): ``save`` writes every rank's value into that rank's file, ``load`` gives each rank its own
    back.  Plain objects are taken from rank 0 (they are expected to be the same everywhere).  Loading at another
    world size raises: such a value has no meaning for a different rank count."""

    def __init__(self, value):
        self.value = value

    def __repr__(self):
        return f"PerRank({self.value!r})"


def _walk(d, path=()):
    if isinstance(d, Mapping):
        for k, v in d.items():
            yield from _walk(v, path + (k,))
    else:
        yield path, d


def _agree(error: BaseException | None, what: str, group) -> None:
    """End of a collective save / load: every rank learns whether any rank failed, so that a failure on one rank (a
    shard that the files do not cover, a full disk) raises everywhere instead of leaving the others in a barrier."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        failed: list = [None] * dist.get_world_size(group)
        dist.all_gather_object(failed, None if error is None else f"{type(error).__name__}: {error}", group=group)
        if error is None and any(f is not None for f in failed):
            bad = {r: f for r, f in enumerate(failed) if f is not None}
            raise RuntimeError(f"checkpoint {what} failed on rank(s) {sorted(bad)}: {next(iter(bad.values()))}")
    if error is not None:
        raise error


def save(state_dict: Mapping[str, Any], checkpoint_id: str, group=None) -> None:
    """Write this rank's part of a (nested) state dict of tagged tensors."""
    error = None
    try:
        _save_rank_file(state_dict, checkpoint_id, group)
    except Exception as e:            # agreed on below
        error = e
    _agree(error, "save", group)


def _save_rank_file(state_dict: Mapping[str, Any], checkpoint_id: str, group) -> None:
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    os.makedirs(checkpoint_id, exist_ok=True)
    entries = {}
    for path, v in _walk(state_dict):
        key = "/".join(map(str, path))
        if isinstance(v, torch.Tensor):
            lay = get_global_layout(v)
            if lay is None:
                if rank == 0:
                    entries[key] = {"kind": "replicated", "tensor": v.detach().cpu().clone()}
                continue
            chunks = []
            for goff, loff, size in zip(lay.global_offsets, lay.local_offsets, lay.local_sizes):
                t = v.detach()
                for d, (l, s) in enumerate(zip(loff, size)):
                    t = t.narrow(d, l, s)
                chunks.append((tuple(goff), tuple(size), t.cpu().clone()))
            entries[key] = {"kind": "sharded", "global_shape": tuple(lay.global_shape), "dtype": v.dtype,
                            "chunks": chunks}
        elif isinstance(v, PerRank):
            entries[key] = {"kind": "per_rank", "value": v.value}
        elif rank == 0:
            entries[key] = {"kind": "object", "value": v}
    tmp = os.path.join(checkpoint_id, f"rank{rank}.pt.tmp")
    torch.save({"world_size": world, "entries": entries}, tmp)
    os.replace(tmp, os.path.join(checkpoint_id, f"rank{rank}.pt"))


def load(state_dict: Mapping[str, Any], checkpoint_id: str, group=None) -> None:
    """Fill the tagged tensors of ``state_dict`` in place from a checkpoint written by ``save`` at
    any world size / placement. Untagged tensors are loaded as replicated values."""
    files = sorted((f for f in os.listdir(checkpoint_id) if f.startswith("rank") and f.endswith(".pt")),
                   key=lambda f: int(f[4:-3]))
    if not files:
        raise FileNotFoundError(f"no rank files under {checkpoint_id}")
    blobs = [torch.load(os.path.join(checkpoint_id, f), map_location="cpu", weights_only=False) for f in files]
    my_rank = dist.get_rank(group) if dist.is_initialized() else 0
    my_world = dist.get_world_size(group) if dist.is_initialized() else 1
    if len(blobs) != blobs[0]["world_size"]:
        raise RuntimeError(f"checkpoint {checkpoint_id} is incomplete: {len(blobs)} of {blobs[0]['world_size']} rank files")

    def assign(container, k, value):
        container[k] = value

    def visit(d):
        for k in list(d.keys()) if isinstance(d, dict) else []:
            yield d, k

    def recurse(d, path):
        for k, v in list(d.items()):
            key = "/".join(map(str, path + (k,)))
            if isinstance(v, Mapping):
                recurse(v, path + (k,))
                continue
            if isinstance(v, torch.Tensor):
                lay = get_global_layout(v)
                if lay is None:
                    src = next((b["entries"][key] for b in blobs if key in b["entries"]), None)
                    if src is None:
                        raise KeyError(f"{key} not in checkpoint")
                    if src["kind"] == "replicated":
                        v.detach().copy_(src["tensor"])
                    elif src["kind"] == "sharded":
                        lay = GlobalLayout(tuple(v.shape), (tuple(0 for _ in v.shape),),
                                           (tuple(0 for _ in v.shape),), (tuple(v.shape),))
                        _fill_boxes(v, lay, key, blobs)
                    continue
                _fill_boxes(v, lay, key, blobs)
            elif isinstance(v, PerRank):
                if my_world != len(blobs):
                    raise RuntimeError(f"{key} is per-rank state saved by {len(blobs)} ranks; it cannot be loaded by "
                                       f"{my_world} ranks")
                src = blobs[my_rank]["entries"].get(key)
                if src is None or src["kind"] != "per_rank":
                    raise KeyError(f"{key} (per-rank state) not in checkpoint")
                v.value = src["value"]
            else:
                src = next((b["entries"][key] for b in blobs if key in b["entries"]), None)
                if src is not None and src["kind"] == "object":
                    d[k] = src["value"]

    error = None
    try:
        recurse(state_dict, ())
    except Exception as e:            # agreed on below
        error = e
    _agree(error, "load", group)


@torch.no_grad()
def _fill_boxes(v: torch.Tensor, lay: GlobalLayout, key: str, blobs) -> None:
    if not any(key in b["entries"] for b in blobs):
        raise KeyError(f"{key} not in checkpoint")
    covered = 0
    want = 0
    for goff, loff, size in zip(lay.global_offsets, lay.local_offsets, lay.local_sizes):
        n = 1
        for s in size:
            n *= s
        want += n
        for b in blobs:
            e = b["entries"].get(key)
            if e is None:
                continue
            saved_shape = tuple(e["tensor"].shape) if e["kind"] == "replicated" else tuple(e["global_shape"])
            if saved_shape != tuple(lay.global_shape):
                raise RuntimeError(f"size mismatch for {key}: the checkpoint holds shape {saved_shape}, the model "
                                   f"expects {tuple(lay.global_shape)}")
            if e["kind"] == "replicated":
                src = e["tensor"]
                for d, (g, s) in enumerate(zip(goff, size)):
                    src = src.narrow(d, g, s)
                dst = v.detach()
                for d, (l, s) in enumerate(zip(loff, size)):
                    dst = dst.narrow(d, l, s)
                dst.copy_(src)
                covered += n
                break
            for cgoff, csize, ct in e["chunks"]:
                lo = tuple(max(a, b_) for a, b_ in zip(goff, cgoff))
                hi = tuple(min(a + sa, b_ + sb) for a, sa, b_, sb in zip(goff, size, cgoff, csize))
                if any(h <= l for l, h in zip(lo, hi)):
                    continue
                src, dst = ct, v.detach()
                m = 1
                for d, (l, h) in enumerate(zip(lo, hi)):
                    src = src.narrow(d, l - cgoff[d], h - l)
                    dst = dst.narrow(d, loff[d] + l - goff[d], h - l)
                    m *= h - l
                dst.copy_(src)
                covered += m
    if covered < want:
        raise RuntimeError(f"checkpoint does not cover all of {key}: {covered} of {want} elements")


# --------------------------------------------------------------------------- interop with DTensor checkpoints
def _as_dtensor(local: torch.Tensor, lay: GlobalLayout, mesh):
    """A tagged local tensor as a ``DTensor`` when its layout is one FSDP2 could have produced: at most one
    box, cut along a single dim into the ``torch.chunk`` pieces of a 1-D mesh.  Returns ``None`` otherwise."""
    from torch.distributed.tensor import DTensor, Replicate, Shard as DShard

    shape = tuple(lay.global_shape)
    W, rank = mesh.size(), mesh.get_local_rank()
    if len(lay.global_offsets) > 1:
        return None
    cut = [d for d in range(len(shape)) if tuple(local.shape)[d] != shape[d]] if lay.global_offsets else []
    if lay.global_offsets and not cut:
        placement = Replicate() if W == 1 or all(o == 0 for o in lay.global_offsets[0]) and tuple(local.shape) == shape \
            else None
        if placement is None:
            return None
        return DTensor.from_local(local, mesh, [placement], run_check=False, shape=torch.Size(shape),
                                  stride=local.stride())
    if len(cut) > 1:
        return None
    if not lay.global_offsets:         # an empty shard: find the dim from the zero-sized one
        cut = [d for d in range(len(shape)) if local.shape[d] == 0 and shape[d] != 0][:1]
        if not cut:
            return None
    dim = cut[0]
    chunk = -(-shape[dim] // W)
    lo, hi = min(shape[dim], rank * chunk), min(shape[dim], (rank + 1) * chunk)
    if lay.global_offsets and (lay.global_offsets[0][dim] != lo or lay.local_sizes[0][dim] != hi - lo):
        return None
    full_stride = []
    acc = 1
    for s in reversed(shape):
        full_stride.append(acc)
        acc *= max(s, 1)
    return DTensor.from_local(local, mesh, [DShard(dim)], run_check=False, shape=torch.Size(shape),
                              stride=tuple(reversed(full_stride)))


def _mesh_of(module, storage):
    from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

    if isinstance(storage.mesh, DeviceMesh):
        return storage.mesh
    if storage.mesh is None and dist.is_initialized():
        cache = getattr(module, "_fsb_world_mesh", None)
        if cache is None:
            cache = init_device_mesh(storage.device.type, (dist.get_world_size(),))
            module._fsb_world_mesh = cache
        return cache
    return None


def to_dtensor_state_dict(module: nn.Module, state_dict: Mapping[str, Any], optimizer=None,
                          optim_state_dict: Mapping[str, Any] | None = None):
    """The model's (and optionally an Adam-style optimizer's) local shards wrapped as ``DTensor``s, so that
    ``torch.distributed.checkpoint`` saves and loads them in the very format FSDP2 state dicts use: a
    checkpoint written by ``fully_shard`` loads into a ``flex_shard`` model and back, at any world size.
    Only layouts FSDP2 itself could produce qualify (``Shard(dim)`` buckets on ``DeviceMesh``es or on the world
    group); a parameter stored any other way raises ``ValueError`` (use ``checkpoint.save`` for those).
    The DTensors alias the local shards, so a ``dcp.load`` into the returned dict fills the model in place.
    Parity: the reference hands tagged tensors to DCP directly (``flex_shard/checkpoint.py:57-69``), which
    needs a newer torch; the FSDP2 <-> flex round trips of its tests
    (``tests/test_flex_shard_checkpoint.py:483-538``) are what this provides."""
    layouts, mesh_by_fqn = {}, {}
    for prefix, sub, st in _storages_with_prefix(module):
        for info in st.infos:
            for name in (info.fqn, *info.shared_fqns):
                for key in {prefix + name, _strip_wrapper_parts(prefix + name)}:
                    layouts[key] = st.global_layout_of(info)
                    mesh_by_fqn[key] = _mesh_of(sub, st)
    out = {}
    for k, v in state_dict.items():
        if isinstance(v, torch.Tensor) and k in layouts:
            mesh = mesh_by_fqn.get(k)
            dt = _as_dtensor(v, layouts[k], mesh) if mesh is not None else None
            if dt is None:
                raise ValueError(f"{k!r} is not stored in a layout a DTensor checkpoint can express; "
                                 "use flex_shard_b200.checkpoint.save / load for it")
            out[k] = dt
        else:
            out[k] = v
    if optimizer is None:
        return out
    osd = optim_state_dict if optim_state_dict is not None else optimizer.state_dict()
    names = {id(p): _strip_wrapper_parts(n) for n, p in module.named_parameters()}
    index_name = {}
    idx = 0
    for g in optimizer.param_groups:
        for p in g["params"]:
            index_name[idx] = names.get(id(p))
            idx += 1
    ostate = {}
    for pid, st in osd["state"].items():
        name = index_name.get(pid)
        entry = {}
        for key, t in st.items():
            if isinstance(t, torch.Tensor) and key in _ADAM_STATE_KEYS and name in layouts:
                dt = _as_dtensor(t, layouts[name], mesh_by_fqn[name])
                if dt is None:
                    raise ValueError(f"optimizer state {key!r} of {name!r} has no DTensor form")
                entry[key] = dt
            else:
                entry[key] = t
        ostate[name if name is not None else pid] = entry
    # parameter groups name their parameters by FQN, the form torch's get_optimizer_state_dict writes
    groups, idx = [], 0
    for g in osd["param_groups"]:
        fqns = []
        for _ in g["params"]:
            fqns.append(index_name.get(idx) or idx)
            idx += 1
        groups.append({**{k: v for k, v in g.items() if k != "params"}, "params": fqns})
    return out, {"state": ostate, "param_groups": groups}


def load_dtensor_optim_state(optimizer, module: nn.Module, dcp_optim_state: Mapping[str, Any]) -> None:
    """Install optimizer state keyed by FQN (as ``to_dtensor_state_dict`` writes it and as
    ``get_optimizer_state_dict`` of an FSDP2 model does) into ``optimizer``."""
    names = {_strip_wrapper_parts(n): p for n, p in module.named_parameters()}
    for name, entry in dcp_optim_state["state"].items():
        p = names.get(name)
        if p is None:
            continue
        for key, t in entry.items():
            val = t.to_local() if hasattr(t, "to_local") else t
            cur = optimizer.state[p].get(key)
            if isinstance(cur, torch.Tensor) and isinstance(val, torch.Tensor) and cur.shape == val.shape:
                cur.copy_(val)
            else:
                optimizer.state[p][key] = val.clone() if isinstance(val, torch.Tensor) else val
