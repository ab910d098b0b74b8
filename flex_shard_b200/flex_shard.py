"""Public entry point ``flex_shard(module, buckets)`` and the module-level control surface.

``flex_shard`` assigns every parameter of ``module`` to exactly one bucket,
asks each bucket's ``placement_fn`` how to store its parameters, packs the local
shards into one byte buffer per bucket, replaces the module's parameters by
views of those buffers, mixes ``FlexShardModule`` into the module's class and
installs the runtime hooks.

Parity: ``flex_shard/flex_shard.py:64-600`` of the reference (``FlexShardModule``
methods, ``flex_shard``, ``relayout_bucket``) and its input validation
(``:643-889``). Unlike the reference, CPU meshes (gloo) are accepted: they run the
same runtime without streams and are what the CPU test-suite uses.
"""
from __future__ import annotations

import math

from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .bucket_runtime import (
    BucketCommContext,
    GradientReductionHandle,
    ModuleUnshardHandle,
    install_bucket_hooks,
    _in_backward,
)
from .bucket_storage import (
    BucketSpec,
    ShardedBucketStorage,
    assign_params_to_buckets,
    fsdp2_param_order,
    is_module_pattern_bucket,
)
from .parallel.comm import comm_for
from .placement_contract import Placement
from .placements.shard import Shard, shard_placement_fn
from .sharded_param import is_flex_shard_param

_STATE_ATTR = "_fsb_state"


class _FlexShardState:
    def __init__(self):
        self.storages: list[ShardedBucketStorage] = []
        self.context: BucketCommContext | None = None
        self.specs: list[BucketSpec] = []
        self.hook_modules: list = []
        self.materialized = True
        self.pending_named: list = []


# --------------------------------------------------------------------------- mixin
class FlexShardModule:
    """Methods added to a module's class by ``flex_shard`` (an FSDP2-like control surface)."""

    @property
    def sharded_bucket_storages(self) -> list[ShardedBucketStorage]:
        return getattr(self, _STATE_ATTR).storages

    def _fsb_ctx(self) -> BucketCommContext:
        ctx = getattr(self, _STATE_ATTR).context
        if ctx is None:
            raise RuntimeError("flex_shard runtime is not installed yet (meta module: call to_empty() first)")
        return ctx

    # ---- materialisation of meta modules
    def to_empty(self, *, device, recurse: bool = True):
        state: _FlexShardState = getattr(self, _STATE_ATTR)
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        for st in state.storages:
            st.device = device
            st.allocate()
            slots = {info.fqn: sl for info, sl in zip(st.infos, st.param_slots)}
            olds = st.sharded_params
            st.install_sharded_params(self, slots, olds)
            if st.runtime is not None:
                st.runtime.unsharded_params = None
                st.runtime.persistent = None
                st.runtime._bucket_base = None
                st.runtime.is_unsharded = False
        # buffers and any unmanaged tensors
        for mod in self.modules():
            for k, buf in list(mod._buffers.items()):
                if buf is not None and buf.device.type == "meta":
                    mod._buffers[k] = torch.empty_like(buf, device=device)
        if state.context is None:
            _install_runtime(self, state)
        state.materialized = True
        return self

    # ---- resharding / unsharding
    def reshard(self) -> None:
        ctx = self._fsb_ctx()
        ctx.check_not_poisoned()
        for st in self.sharded_bucket_storages:
            st.runtime.reshard()

    def unshard(self, async_op: bool = False):
        ctx = self._fsb_ctx()
        ctx.check_not_poisoned()
        if _in_backward():
            raise RuntimeError("unshard() cannot run in backward")
        rts = []
        for st in self.sharded_bucket_storages:
            st.runtime.explicit_unshard(async_op=True)
            rts.append(st.runtime)
        handle = ModuleUnshardHandle(rts)
        if not async_op:
            handle.wait()
            return None
        return handle

    # ---- backward finalisation
    def set_manual_backward_finalization(self, enabled: bool) -> None:
        self._fsb_ctx().manual_finalization = bool(enabled)

    def finalize_backward(self, async_op: bool = False):
        ctx = self._fsb_ctx()
        if ctx.pending_finalize_handle is not None:
            raise RuntimeError("finalize_backward(): wait on the previous handle first")
        order = list(reversed(ctx.post_forward_order)) or list(ctx.runtimes)
        for rt in ctx.runtimes:
            if rt not in order:
                order.append(rt)
        saved = ctx.manual_finalization
        ctx.manual_finalization = False
        try:
            for rt in order:
                rt.finalize()
        finally:
            ctx.manual_finalization = saved
        handle = GradientReductionHandle(ctx)
        if async_op:
            ctx.pending_finalize_handle = handle
            return handle
        handle.wait()
        return None

    def finish_deferred_backward(self, param) -> None:
        st = self.bucket_storage_of(param)
        st.runtime.finish_deferred(param)

    def bucket_storage_of(self, param) -> ShardedBucketStorage:
        st = getattr(param, "_fsb_storage", None)
        if st is None:
            raise ValueError("parameter is not managed by flex_shard")
        return st

    # ---- settings broadcast to every bucket
    # The setters keep the reference's signatures (``flex_shard/flex_shard.py:262-394`` there).  ``recurse`` selects
    # the sharded modules below this one as well; nested wrapping is refused, so this module's buckets are all there are.
    def set_gradient_reduce_op(self, op, *, recurse: bool = True) -> None:
        for st in self.sharded_bucket_storages:
            st.set_gradient_reduce_op(op)

    def set_gradient_divide_factor(self, factor, *, recurse: bool = True) -> None:
        for st in self.sharded_bucket_storages:
            st.set_gradient_divide_factor(factor)

    def set_requires_gradient_sync(self, requires_gradient_sync: bool, *, recurse: bool = True) -> None:
        for st in self.sharded_bucket_storages:
            st.set_requires_gradient_sync(requires_gradient_sync)

    def set_reshard_after_backward(self, reshard_after_backward: bool, *, recurse: bool = True) -> None:
        for st in self.sharded_bucket_storages:
            st.set_reshard_after_backward(reshard_after_backward)

    def set_reshard_after_forward(self, reshard_after_forward: bool, *, recurse: bool = True) -> None:
        for st in self.sharded_bucket_storages:
            st.set_reshard_after_forward(reshard_after_forward)

    def set_separate_reduce_scatter_group(self, enable: bool = True, *, recurse: bool = True) -> None:
        """Run reduce-scatters on a second communicator so they can overlap all-gathers."""
        made: dict[int, Any] = {}
        for st in self.sharded_bucket_storages:
            if not enable:
                st.reduce_comm = st.comm
                continue
            if st.reduce_comm is not st.comm:
                continue
            key = id(st.comm)
            if key not in made:
                made[key] = st.comm.new_like()
            st.reduce_comm = made[key]

    def set_max_pending_reduce_grads(self, max_pending_reduce_grads: int = 1, *, recurse: bool = True) -> None:
        if max_pending_reduce_grads < 1:
            raise ValueError("max_pending_reduce_grads must be >= 1")
        self._fsb_ctx().max_pending_reduce_grads = int(max_pending_reduce_grads)


# --------------------------------------------------------------------------- helpers
def _managed_named_params(module: nn.Module):
    """(fqn, param) without duplicates, plus the extra names of tied parameters and every slot."""
    first: dict[int, str] = {}
    shared: dict[str, list[str]] = {}
    slots: dict[str, list[tuple[nn.Module, str]]] = {}
    named = []
    for mod_name, mod in module.named_modules(remove_duplicate=False):
        for attr, p in mod._parameters.items():
            if p is None:
                continue
            fqn = f"{mod_name}.{attr}" if mod_name else attr
            if id(p) in first:
                canon = first[id(p)]
                if fqn != canon and fqn not in shared.setdefault(canon, []):
                    shared[canon].append(fqn)
                if (mod, attr) not in [(m, a) for m, a in slots[canon]]:
                    slots[canon].append((mod, attr))
            else:
                first[id(p)] = fqn
                named.append((fqn, p))
                slots[fqn] = [(mod, attr)]
    return named, {k: tuple(v) for k, v in shared.items()}, slots


def _reject_nested(module: nn.Module) -> None:
    if isinstance(module, FlexShardModule):
        raise ValueError("flex_shard() was already applied to this module")
    for name, child in module.named_modules():
        if child is not module and isinstance(child, FlexShardModule):
            raise ValueError(
                f"flex_shard() was already applied to submodule {name!r}; wrap the root once with explicit buckets")
    for p in module.parameters():
        if is_flex_shard_param(p):
            raise ValueError("module already holds flex_shard parameters (an ancestor or descendant was wrapped)")


def _common_module(root: nn.Module, fqns: Sequence[str]) -> tuple[str, nn.Module]:
    parts = [f.split(".")[:-1] for f in fqns]
    prefix = []
    for level in zip(*parts):
        if all(x == level[0] for x in level):
            prefix.append(level[0])
        else:
            break
    name = ".".join(prefix)
    mod = root.get_submodule(name) if name else root
    # climb to the nearest module that has its own forward
    while name and type(mod).forward is nn.Module.forward:
        name = ".".join(name.split(".")[:-1])
        mod = root.get_submodule(name) if name else root
    return name, mod


def _hook_modules_for(root: nn.Module, spec: BucketSpec, fqns: Sequence[str]):
    if is_module_pattern_bucket(root, spec):
        mods = []
        for pat in spec.patterns:
            m = root.get_submodule(pat)
            if type(m).forward is nn.Module.forward and not isinstance(m, (nn.ModuleList, nn.ModuleDict)):
                pass
            if isinstance(m, (nn.ModuleList, nn.ModuleDict)) or type(m).forward is nn.Module.forward:
                raise ValueError(f"BucketSpec pattern {pat!r} names a container without a forward(); name its children")
            mods.append(m)
        return mods, len(mods) > 1, "+".join(spec.patterns)
    name, mod = _common_module(root, fqns)
    return [mod], False, name or "<root>"


def _unwrap_placements(result, named=()) -> dict:
    """A placement function maps FQN -> Placement; the reference's functions return one-element tuples
    ``(placement,)`` (one entry per mesh dimension of a 1-D mesh), which are accepted as well.  A placement that
    describes the whole bucket (``BucketedOwned`` built from ``{fqn: segments}``) is narrowed to each parameter."""
    out = {f: (v[0] if isinstance(v, (tuple, list)) and len(v) == 1 else v) for f, v in dict(result).items()}
    shapes = {f: tuple(getattr(p, "_fsb_global_shape", None) or p.shape) for f, p in named}
    for f, v in out.items():
        if f in shapes and hasattr(v, "for_param"):
            out[f] = v.for_param(f, shapes[f])
    return out


def _validate_bucket(spec: BucketSpec, named, placements, comm) -> None:
    if spec.offload_policy is not None:
        raise ValueError("offload_policy is not supported: flex_shard keeps buckets on the mesh device")
    missing = [f for f, _ in named if f not in placements]
    if missing:
        raise ValueError(f"placement_fn returned no placement for {missing}")
    known = {f for f, _ in named}
    extra = [f for f in placements if f not in known]
    if extra:
        raise ValueError(f"placement_fn returned placements for names that are not in the bucket: {extra}")
    for f, _ in named:
        if not isinstance(placements[f], Placement):
            raise TypeError(f"placement for {f!r} is not a Placement: {placements[f]!r}")
    keys = {placements[f].bucket_compatibility_key() for f, _ in named}
    if len(keys) > 1:
        raise ValueError(
            f"bucket {spec.patterns!r} mixes incompatible placements {sorted(map(str, keys))}; "
            "split it or use a mixed-bucket placement")
    dtypes = {p.dtype for _, p in named}
    if len(dtypes) > 1 and not getattr(next(iter(placements.values())), "allows_mixed_dtypes", False):
        raise ValueError(f"bucket {spec.patterns!r} mixes parameter dtypes {sorted(map(str, dtypes))}")
    if spec.fsdp2_compatible and not all(isinstance(placements[f], Shard) for f, _ in named):
        raise ValueError("fsdp2_compatible=True requires Shard placements for every parameter of the bucket")
    for f, p in named:
        placements[f].compute_local_shape(tuple(p.shape), comm.rank, comm.world_size)  # raises on bad dims


def _validate_dtype_overrides(buckets: Sequence[BucketSpec], assigned) -> None:
    """Every ``param_dtype_overrides`` pattern must name a parameter of some bucket that uses an equal policy
    (builders often share one policy across buckets, so the parameter may sit in any of them); a pattern that
    matches nothing there would silently leave the parameter in the policy's default dtype.
    Parity: ``flex_shard/flex_shard.py:756-789`` of the reference (exact names there, fnmatch patterns here)."""
    import fnmatch

    groups: list[tuple[Any, list[int], set[str]]] = []
    for idx, (spec, group) in enumerate(zip(buckets, assigned)):
        policy = spec.mp_policy
        if policy is None or not getattr(policy, "param_dtype_overrides", None):
            continue
        for known, indices, fqns in groups:
            if known == policy:
                indices.append(idx)
                fqns.update(f for f, _ in group)
                break
        else:
            groups.append((policy, [idx], {f for f, _ in group}))
    for policy, indices, fqns in groups:
        unknown = sorted(pat for pat in policy.param_dtype_overrides
                         if not any(fnmatch.fnmatchcase(f, pat) for f in fqns))
        if unknown:
            raise ValueError(f"param_dtype_overrides of buckets {indices} names parameters that are in no bucket "
                             f"using that policy: {unknown}")


def _install_runtime(module: nn.Module, state: _FlexShardState) -> None:
    state.context = install_bucket_hooks(module, state.storages, state.hook_modules)


# --------------------------------------------------------------------------- public API
def flex_shard(module: nn.Module, buckets: Sequence[BucketSpec], *,
               storage_allocator: Callable[[int, torch.device], torch.Tensor] | None = None) -> nn.Module:
    """Shard ``module``'s parameters bucket by bucket; returns ``module`` (mutated in place)."""
    if not isinstance(module, nn.Module):
        raise TypeError("flex_shard expects an nn.Module")
    buckets = list(buckets)
    if not buckets:
        raise ValueError("flex_shard needs at least one BucketSpec")
    _reject_nested(module)
    named, shared, slots = _managed_named_params(module)
    if not named:
        raise ValueError("module has no parameters to shard")
    assigned = assign_params_to_buckets(module, named, buckets, shared)

    # resolve meshes first (validates 1-D meshes) and find the target device
    comms = [comm_for(b.mesh) for b in buckets]
    is_meta = any(p.device.type == "meta" for _, p in named)
    device = comms[0].device
    if not is_meta and all(p.device.type == "cpu" for _, p in named) and device.type == "cuda":
        module.to(device)
        named, shared, slots = _managed_named_params(module)
        assigned = assign_params_to_buckets(module, named, buckets, shared)

    _validate_dtype_overrides(buckets, assigned)
    state = _FlexShardState()
    plans = []
    for spec, comm, group in zip(buckets, comms, assigned):
        if not group:
            continue
        if spec.fsdp2_compatible:
            group = fsdp2_param_order(module, group)
        fn = spec.placement_fn or shard_placement_fn(0)
        placements = _unwrap_placements(fn(group, spec.mesh), group)
        _validate_bucket(spec, group, placements, comm)
        # every name of a tied parameter counts: the bucket must be gathered around all the modules that use it
        all_names = [n for f, _ in group for n in (f, *shared.get(f, ()))]
        mods, is_group, name = _hook_modules_for(module, spec, all_names)
        plans.append((spec, comm, group, placements, mods, is_group, name))

    # everything validated: materialise
    for spec, comm, group, placements, mods, is_group, name in plans:
        st = ShardedBucketStorage.from_bucket(
            spec, group, placements, spec.mesh, comm, comm.device if not is_meta else torch.device("meta"),
            shared, name, allocator=storage_allocator, materialize=not is_meta)
        if is_meta:
            st.byte_storage = torch.empty(st.total_bytes, dtype=torch.uint8, device="meta")
        st.install_sharded_params(module, slots, [p for _, p in group])
        st.module_names = [name]
        state.storages.append(st)
        state.specs.append(spec)
        state.hook_modules.append((mods, is_group))

    cls = module.__class__
    module.__class__ = type(f"FlexShard{cls.__name__}", (FlexShardModule, cls), {})
    setattr(module, _STATE_ATTR, state)
    state.materialized = not is_meta
    if not is_meta:
        _install_runtime(module, state)
    return module


@torch.no_grad()
def relayout_bucket(module: nn.Module, bucket_storage: ShardedBucketStorage, placement_fn) -> ShardedBucketStorage:
    """Move one bucket to a new placement, bitwise (gathers in the storage dtype, repacks, frees the
    old buffer). Must run before the first unshard of the bucket and before optimizers are built."""
    storage = bucket_storage
    state: _FlexShardState = getattr(module, _STATE_ATTR)
    if not any(s is storage for s in state.storages):
        raise ValueError("relayout_bucket(): the storage is not one of the module's bucket storages")
    idx = next(i for i, s in enumerate(state.storages) if s is storage)
    rt = storage.runtime
    if rt is not None and (rt.is_unsharded or rt.unsharded_params is not None or rt.pending is not None):
        raise RuntimeError("relayout_bucket() must run before the bucket's first unshard")
    comm = storage.comm
    W, rank = comm.world_size, comm.rank
    # gather every parameter in its storage dtype through the old placement
    fulls = []
    for info in storage.infos:
        local = storage.local_view(info)
        fulls.append(_gather_full(info, local, comm))
    named = [(info.fqn, nn.Parameter(f, requires_grad=info.requires_grad)) for info, f in zip(storage.infos, fulls)]
    for (fqn, p), info, sp in zip(named, storage.infos, storage.sharded_params):
        for k, v in info.param_attrs.items():
            try:
                setattr(p, k, v)
            except Exception:
                pass
        if info.outer_layout is not None:
            from .placement_contract import set_global_layout

            set_global_layout(p, info.outer_layout)
        if info.partial_grad_group is not None:
            from .placement_contract import set_partial_grad_group

            set_partial_grad_group(p, info.partial_grad_group)
    placements = _unwrap_placements(placement_fn(named, storage.mesh), named)
    _validate_bucket(storage.spec, named, placements, comm)
    shared = {info.fqn: info.shared_fqns for info in storage.infos}
    new = ShardedBucketStorage.from_bucket(storage.spec, named, placements, storage.mesh, comm, storage.device,
                                           shared, storage.name, allocator=getattr(storage, "_allocator", None))
    slots = {info.fqn: sl for info, sl in zip(storage.infos, storage.param_slots)}
    new.install_sharded_params(module, slots, [p for _, p in named])
    # carry settings and runtime bindings over
    for attr in ("reshard_after_forward", "reshard_after_backward", "requires_gradient_sync", "reduction",
                 "forward_prefetch", "backward_prefetch", "modules", "module_names"):
        setattr(new, attr, getattr(storage, attr))
    new.reduce_comm = storage.reduce_comm
    if rt is not None:
        rt.storage = new
        new.runtime = rt
    for other in state.storages:
        for lst_name in ("forward_prefetch", "backward_prefetch"):
            lst = getattr(other, lst_name)
            if lst:
                setattr(other, lst_name, [new if s is storage else s for s in lst])
    state.storages[idx] = new
    release = getattr(comm, "release_storage", None)
    if release is not None and storage.byte_storage is not None:
        release(storage.byte_storage)   # a symmetric region of its own: give it back (collective-safe: same order everywhere)
    storage.byte_storage = None
    storage.sharded_params = []
    return new


def _gather_full(info, local: torch.Tensor, comm) -> torch.Tensor:
    """All-gather one parameter through its placement's layout (set-up helper of ``relayout_bucket``).

    Every rank sends its local tensor as bytes, padded to the largest local size, in one ``all_gather_into_tensor``;
    the boxes of every rank's layout are then copied out of its row.  That moves (W-1)/W of the parameter into each
    rank and widens nothing.  When the local sizes are very uneven (an owner holds the whole parameter: the padded
    rows would carry W copies) or the placement cuts the parameter through a bucket-level plan, the pieces are
    summed as integers over zero-padded full tensors instead (every element has exactly one owner, so that sum is a
    bitwise gather too)."""
    W = comm.world_size
    full = torch.zeros(info.global_shape, dtype=info.storage_dtype, device=local.device)
    bucket_level = info.bucket_layout is not None and hasattr(info.placement, "bucket_global_layout")

    def layout_of(r):
        if bucket_level:
            return info.placement.bucket_global_layout(info, r, W)
        return info.placement.global_layout(info.global_shape, r, W)

    def place(src_local, lay):
        for goff, loff, size in zip(lay.global_offsets, lay.local_offsets, lay.local_sizes):
            src, dst = src_local, full
            for d, (g, l, s) in enumerate(zip(goff, loff, size)):
                src = src.narrow(d, l, s)
                dst = dst.narrow(d, g, s)
            dst.copy_(src)

    if W == 1:
        place(local, layout_of(comm.rank))
        return full
    shapes = None if bucket_level else [tuple(info.placement.compute_local_shape(info.global_shape, r, W)) for r in range(W)]
    if shapes is not None:
        numels = [math.prod(sh) for sh in shapes]
        biggest = max(numels)
        if biggest > 0 and biggest * W <= 2 * full.numel() and tuple(local.shape) == shapes[comm.rank]:
            esize = full.element_size()
            send = torch.zeros(biggest * esize, dtype=torch.uint8, device=local.device)
            mine = local.contiguous().view(-1).view(torch.uint8)
            send[:mine.numel()].copy_(mine)
            rows = torch.empty(W * biggest * esize, dtype=torch.uint8, device=local.device)
            dist.all_gather_into_tensor(rows, send, group=comm.group)
            rows = rows.view(W, biggest * esize)
            for r in range(W):
                if numels[r] == 0:
                    continue
                piece = rows[r, :numels[r] * esize].view(info.storage_dtype).view(shapes[r])
                place(piece, layout_of(r))
            return full
    place(local, layout_of(comm.rank))
    as_int = full.view(torch.int32) if full.element_size() == 4 else (
        full.view(torch.int16) if full.element_size() == 2 else full.view(torch.uint8))
    if as_int.dtype == torch.int32:
        dist.all_reduce(as_int, group=comm.group)
    else:
        wide = as_int.to(torch.int32)
        dist.all_reduce(wide, group=comm.group)
        as_int.copy_(wide.to(as_int.dtype))
    return full
