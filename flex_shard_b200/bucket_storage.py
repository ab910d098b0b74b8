"""Bucket specifications and the per-bucket byte storage.

A bucket is a set of parameters that communicate together. Each bucket owns
one contiguous ``uint8`` buffer holding this rank's part of every parameter
(laid out by the bucket's placements); the module's parameters are replaced by
``nn.Parameter`` views into that buffer, so optimizers and ``state_dict`` see
plain local tensors.

Parity: the roles of ``BucketSpec`` / ``MixedPrecisionPolicy`` / ``OffloadPolicy``
(``flex_shard/bucket_storage.py:52-258``), ``ParamInfo`` (``:280-343``) and
``ShardedBucketStorage`` (``:346-969``) of the reference, incl. bucket
assignment errors (``:985-1053``) and the FSDP2 parameter order (``:1095-1125``).
"""
from __future__ import annotations

import fnmatch
import math
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .placement_contract import (
    BucketParamStorageLayout,
    BucketStorageLayout,
    GlobalLayout,
    GradientReduction,
    Placement,
    compose_global_layouts,
    get_global_layout,
    get_partial_grad_group,
)
from .sharded_param import set_sharding_info

PlacementFn = Callable[[list[tuple[str, nn.Parameter]], Any], Mapping[str, Placement]]
class BucketHookArgs(list):
    """What a bucket hook is called with: the bucket's ``(fqn, unsharded parameter)`` pairs, as in the reference
    (``flex_shard/bucket_storage.py:48-49`` there), which also answer for the bucket's storage: ``args.storage`` is the
    ``ShardedBucketStorage`` and its attributes (``name``, ``infos``, ...) can be read from ``args`` directly."""

    def __init__(self, storage, pairs):
        super().__init__(pairs)
        self.storage = storage

    def __getattr__(self, name):
        if name == "storage":
            raise AttributeError(name)
        return getattr(self.storage, name)


BucketHook = Callable[[BucketHookArgs], None]


# --------------------------------------------------------------------------- policies
@dataclass(frozen=True)
class MixedPrecisionPolicy:
    """``param_dtype``: dtype of the gathered (compute) parameters; ``reduce_dtype``: dtype of the
    gradient reduction; ``param_dtype_overrides``: fnmatch pattern -> compute dtype for
    parameters that must stay wider (e.g. router weights in fp32)."""

    param_dtype: torch.dtype | None = None
    reduce_dtype: torch.dtype | None = None
    param_dtype_overrides: Mapping[str, torch.dtype] | None = field(default=None, kw_only=True)

    def __post_init__(self):
        if self.param_dtype_overrides is not None:
            for pat, dt in self.param_dtype_overrides.items():
                if not isinstance(pat, str) or not isinstance(dt, torch.dtype):
                    raise TypeError("param_dtype_overrides maps fnmatch patterns to torch dtypes")
            object.__setattr__(self, "param_dtype_overrides", dict(self.param_dtype_overrides))

    def __hash__(self):
        ov = tuple(sorted((self.param_dtype_overrides or {}).items(), key=lambda kv: kv[0]))
        return hash((self.param_dtype, self.reduce_dtype, ov))

    def compute_dtype_for(self, fqn: str, storage_dtype: torch.dtype) -> torch.dtype:
        if self.param_dtype_overrides:
            for pat, dt in self.param_dtype_overrides.items():
                if fnmatch.fnmatchcase(fqn, pat):
                    return dt
        return self.param_dtype if self.param_dtype is not None else storage_dtype


@dataclass(frozen=True)
class OffloadPolicy:
    """Placeholder: CPU offload is not supported (passing one to ``BucketSpec`` is rejected)."""

    pin_memory: bool = True


@dataclass(frozen=True)
class BucketSpec:
    """Names the parameters of one bucket and how they are stored and reduced.

    ``patterns`` are fnmatch patterns over parameter FQNs, or module names (all their
    parameters). Every managed parameter must match exactly one bucket.
    """

    patterns: Sequence[str]
    placement_fn: PlacementFn | None = None
    mesh: Any = None
    mp_policy: MixedPrecisionPolicy = field(default_factory=MixedPrecisionPolicy)
    offload_policy: OffloadPolicy | None = None
    gradient_reduce_op: Any = dist.ReduceOp.AVG
    gradient_divide_factor: float | None = None
    reshard_after_forward: bool = True
    pre_backward_hook: BucketHook | None = None
    post_reduce_hook: BucketHook | None = None
    defer_post_backward: bool = False
    fsdp2_compatible: bool = False

    def __post_init__(self):
        if isinstance(self.patterns, str):
            raise TypeError("BucketSpec.patterns must be a sequence of patterns, not a string")
        object.__setattr__(self, "patterns", tuple(self.patterns))
        # validates op / factor
        GradientReduction(self.gradient_reduce_op, self.gradient_divide_factor)

    @property
    def reduction(self) -> GradientReduction:
        return GradientReduction(self.gradient_reduce_op, self.gradient_divide_factor)


# --------------------------------------------------------------------------- per-parameter record
@dataclass
class ParamInfo:
    fqn: str
    global_shape: tuple[int, ...]          # shape of the parameter handed to flex_shard()
    global_stride: tuple[int, ...]
    local_shape: tuple[int, ...]
    local_stride: tuple[int, ...]
    byte_offset: int
    storage_nbytes: int
    storage_dtype: torch.dtype             # dtype of the stored (master) shard
    param_dtype: torch.dtype               # dtype of the gathered parameter
    reduce_dtype: torch.dtype              # dtype this parameter's grads want to be reduced in
    grad_dtype: torch.dtype | None         # dtype of the sharded .grad (None: storage dtype)
    placement: Placement
    requires_grad: bool
    outer_layout: GlobalLayout | None = None
    partial_grad_group: Any | None = None
    param_attrs: dict = field(default_factory=dict)
    shared_fqns: tuple[str, ...] = ()
    bucket_layout: Any | None = None
    bucket_reduce_dtype: torch.dtype | None = None
    explicit_reduce_dtype: bool = False    # the bucket's policy names a reduce dtype

    @property
    def unsharded_grad_dtype(self) -> torch.dtype:
        """Dtype in which the gathered parameter's gradient accumulates across backward passes: the
        policy's reduce dtype, else an explicit ``grad_dtype`` set on the parameter before sharding,
        else the storage dtype (parity: ``flex_shard/bucket_storage.py:325-334`` of the reference); it is
        what ``reduce_dtype`` resolves to when the bucket is built."""
        return self.reduce_dtype

    # ---- names of the reference's ParamInfo
    @property
    def placements(self) -> tuple:
        return (self.placement,)

    @property
    def dtype(self) -> torch.dtype:
        return self.storage_dtype

    @property
    def unsharded_dtype(self) -> torch.dtype:
        return self.param_dtype

    @property
    def grad_reduce_dtype(self) -> torch.dtype:
        return self.bucket_reduce_dtype or self.reduce_dtype

    @property
    def has_explicit_grad_dtype(self) -> bool:
        return self.grad_dtype is not None

    @property
    def grad_dtype_override(self) -> torch.dtype | None:
        return self.grad_dtype

    @property
    def local_numel(self) -> int:
        return math.prod(self.local_shape)

    @property
    def global_numel(self) -> int:
        return math.prod(self.global_shape)


@dataclass(frozen=True)
class BucketLayout:
    infos: tuple[ParamInfo, ...]
    total_bytes: int


def _contiguous_stride(shape: Sequence[int]) -> tuple[int, ...]:
    stride, acc = [], 1
    for s in reversed(shape):
        stride.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(stride))


_USER_ATTR_SKIP = {"grad", "data", "requires_grad", "_grad", "grad_fn", "_backward_hooks"}


def _user_attrs(p: torch.Tensor) -> dict:
    d = getattr(p, "__dict__", {})
    return {k: v for k, v in d.items() if k not in _USER_ATTR_SKIP and not k.startswith("_fsb_")}


_OLD_FSDP2: bool | None = None


def installed_fsdp2_accumulates_after_backward() -> bool:
    """True for torch releases whose FSDP2 sums every backward's gradients in the compute dtype, widens a
    kept gradient to the reduce dtype after the backward (``FSDPParam.to_accumulated_grad_if_needed``) and
    reduces in the compute dtype when the policy names no reduce dtype.  ``fsdp2_compatible`` buckets follow
    the installed FSDP2, whichever it is; other buckets accumulate and reduce in the storage dtype."""
    global _OLD_FSDP2
    if _OLD_FSDP2 is None:
        try:
            from torch.distributed.fsdp._fully_shard._fsdp_param import FSDPParam

            _OLD_FSDP2 = hasattr(FSDPParam, "to_accumulated_grad_if_needed")
        except Exception:
            _OLD_FSDP2 = False
    return _OLD_FSDP2


# --------------------------------------------------------------------------- storage
class ShardedBucketStorage:
    """One bucket: its byte buffer, parameter records, sharded parameters and settings."""

    def __init__(self, spec: BucketSpec, infos: list[ParamInfo], total_bytes: int, mesh, comm,
                 device: torch.device, name: str):
        self.spec = spec
        self.infos = infos
        self.total_bytes = total_bytes
        self.mesh = mesh
        self.comm = comm
        self.device = device
        self.name = name
        self.byte_storage: torch.Tensor | None = None
        self.sharded_params: list[nn.Parameter] = []
        self.param_slots: list[list[tuple[nn.Module, str]]] = []  # every (module, attr) a param is installed in
        self.runtime = None  # set by bucket_runtime
        # mutable settings
        self.reshard_after_forward = spec.reshard_after_forward
        self.reshard_after_backward = True
        self.requires_gradient_sync = True
        self.reduction = spec.reduction
        self.forward_prefetch: list["ShardedBucketStorage"] | None = None
        self.backward_prefetch: list["ShardedBucketStorage"] | None = None
        self.reduce_comm = comm  # replaced by set_separate_reduce_scatter_group
        self._grad_bucket: torch.Tensor | None = None
        self.modules: list[nn.Module] = []
        self.module_names: list[str] = []

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_bucket(cls, spec: BucketSpec, named_params: list[tuple[str, nn.Parameter]],
                    placements: Mapping[str, Placement], mesh, comm, device: torch.device,
                    shared_names: Mapping[str, tuple[str, ...]], name: str,
                    allocator: Callable[[int, torch.device], torch.Tensor] | None = None,
                    materialize: bool = True) -> "ShardedBucketStorage":
        infos, total = create_param_infos(spec, named_params, placements, comm.rank, comm.world_size,
                                          shared_names)
        self = cls(spec, infos, total, mesh, comm, device, name)
        self._allocator = allocator
        if materialize:
            self.allocate()
            self.copy_params_from([p for _, p in named_params])
        return self

    def allocate(self) -> None:
        n = max(self.total_bytes, 0)
        buf = None
        if getattr(self, "_allocator", None) is not None:
            buf = self._allocator(n, self.device)
        elif self.device.type == "cuda" and getattr(self.placement, "uniform_storage", False):
            # same size on every rank: the bucket can live in symmetric memory, where the peers' gathers
            # read it in place (a peer-memory communicator offers alloc_storage; others do not)
            alloc = getattr(self.comm, "alloc_storage", None)
            buf = alloc(n) if alloc is not None else None
        self.byte_storage = buf if buf is not None else torch.empty(n, dtype=torch.uint8, device=self.device)
        self.byte_storage.zero_()  # padding must be deterministic zeros

    @property
    def placement(self) -> Placement:
        return self.infos[0].placement

    @property
    def debug_fqn(self) -> str | None:
        """Short name of the bucket for profiler ranges (common module path of its parameters)."""
        from .utils.profiling import bucket_debug_fqn

        return bucket_debug_fqn([i.fqn for i in self.infos])

    def local_view(self, info: ParamInfo) -> torch.Tensor:
        return info.placement.make_local_storage_view(info, self.byte_storage)

    @torch.no_grad()
    def copy_params_from(self, params: Sequence[torch.Tensor]) -> None:
        rank, ws = self.comm.rank, self.comm.world_size
        for info, p in zip(self.infos, params):
            if p.device.type == "meta":
                continue
            view = self.local_view(info)
            src = p.detach()
            if src.device != view.device:
                src = src.to(view.device)
            info.placement.copy_param_to_storage(info, src, view, rank, ws)

    def install_sharded_params(self, root: nn.Module, slots: Mapping[str, list[tuple[nn.Module, str]]],
                               old_params: Sequence[nn.Parameter]) -> None:
        """Replace each managed parameter (in every module slot it is tied into) by a view."""
        self.sharded_params = []
        self.param_slots = []
        for info, old in zip(self.infos, old_params):
            view = self.local_view(info)
            sp = nn.Parameter(view, requires_grad=info.requires_grad)
            for k, v in info.param_attrs.items():
                try:
                    setattr(sp, k, v)
                except Exception:
                    pass
            set_sharding_info(sp, placement=info.placement, global_shape=info.global_shape,
                              global_stride=info.global_stride, mesh=self.mesh,
                              outer_layout=info.outer_layout)
            if info.grad_dtype is not None and hasattr(sp, "grad_dtype"):
                try:
                    sp.grad_dtype = info.grad_dtype
                except Exception:
                    pass
            sp._fsb_info = info
            sp._fsb_storage = self
            sl = slots[info.fqn]
            for mod, attr in sl:
                mod._parameters[attr] = sp
            self.sharded_params.append(sp)
            self.param_slots.append(list(sl))

    # ------------------------------------------------------------------ layouts
    def global_layout_of(self, info: ParamInfo) -> GlobalLayout:
        inner = info.placement.global_layout(info.global_shape, self.comm.rank, self.comm.world_size)
        if info.bucket_layout is not None and hasattr(info.placement, "bucket_global_layout"):
            inner = info.placement.bucket_global_layout(info, self.comm.rank, self.comm.world_size)
        if info.outer_layout is None:
            return inner
        return compose_global_layouts(info.outer_layout, inner)

    # ------------------------------------------------------------------ per-bucket control surface
    def unshard(self, async_op: bool = False):
        return self.runtime.explicit_unshard(async_op=async_op)

    def reshard(self) -> None:
        self.runtime.reshard()

    def set_reshard_after_forward(self, value: bool) -> None:
        self.reshard_after_forward = bool(value)

    def set_reshard_after_backward(self, value: bool) -> None:
        self.reshard_after_backward = bool(value)

    # ---- read-only names the reference's storage offers (``flex_shard/bucket_storage.py:742-800, 961-969`` there)
    @property
    def flat_storage(self) -> torch.Tensor:
        return self.byte_storage

    @property
    def numel(self) -> int:
        """Bytes of the sharded storage."""
        return self.byte_storage.numel()

    @property
    def param_infos(self) -> dict[str, ParamInfo]:
        return {info.fqn: info for info in self.infos}

    @property
    def gradient_reduction(self) -> GradientReduction:
        return self.reduction

    @property
    def gradient_reduce_op(self):
        return self.reduction.op

    @property
    def gradient_divide_factor(self) -> float | None:
        return self.reduction.divide_factor

    @property
    def world_size(self) -> int:
        return self.comm.world_size

    @property
    def reduce_mesh(self):
        """What the bucket reduce-scatters over: its mesh, or the process group of the communicator that
        ``set_separate_reduce_scatter_group`` gave the reduce-scatters (a group, not a ``DeviceMesh``)."""
        return self.mesh if self.reduce_comm is self.comm else self.reduce_comm.group

    def get_local_view(self, fqn: str) -> torch.Tensor:
        """The local tensor of parameter ``fqn`` as a view of the sharded storage."""
        info = self.param_infos[fqn]
        return info.placement.make_local_storage_view(info, self.byte_storage)

    def set_requires_gradient_sync(self, value: bool) -> None:
        self.requires_gradient_sync = bool(value)

    def set_gradient_reduce_op(self, op) -> None:
        self.reduction = GradientReduction(op, None if op == dist.ReduceOp.SUM else self.reduction.divide_factor)

    def set_gradient_divide_factor(self, factor: float | None) -> None:
        self.reduction = GradientReduction(dist.ReduceOp.AVG, factor)

    @staticmethod
    def _prefetch_targets(buckets) -> list["ShardedBucketStorage"]:
        buckets = list(buckets)
        for b in buckets:
            if not isinstance(b, ShardedBucketStorage):
                raise TypeError(f"prefetch targets must be ShardedBucketStorage objects (module.sharded_bucket_storages), "
                                f"got {type(b).__name__}")
        return buckets

    def set_buckets_to_forward_prefetch(self, buckets: Sequence["ShardedBucketStorage"]) -> None:
        self.forward_prefetch = self._prefetch_targets(buckets)

    def set_buckets_to_backward_prefetch(self, buckets: Sequence["ShardedBucketStorage"]) -> None:
        self.backward_prefetch = self._prefetch_targets(buckets)

    @property
    def bucket_reduce_dtype(self) -> torch.dtype:
        """Reduction dtype of the bucket: the promotion over its trainable parameters."""
        dt = None
        for info in self.infos:
            if not info.requires_grad:
                continue
            dt = info.reduce_dtype if dt is None else torch.promote_types(dt, info.reduce_dtype)
        return dt if dt is not None else self.infos[0].reduce_dtype

    def __repr__(self) -> str:
        state = "unsharded" if (self.runtime is not None and self.runtime.is_unsharded) else "sharded"
        return (f"ShardedBucketStorage(name={self.name!r}, params={len(self.infos)}, "
                f"bytes={self.total_bytes}, world={self.comm.world_size}, {state})")


# --------------------------------------------------------------------------- building ParamInfos
def create_param_infos(spec: BucketSpec, named_params: list[tuple[str, nn.Parameter]],
                       placements: Mapping[str, Placement], rank: int, world_size: int,
                       shared_names: Mapping[str, tuple[str, ...]]) -> tuple[list[ParamInfo], int]:
    mp = spec.mp_policy
    first = placements[named_params[0][0]]
    entries = [(fqn, tuple(p.shape), p.dtype, placements[fqn]) for fqn, p in named_params]
    bucket_layout: BucketStorageLayout | None = first.bucket_storage_layout(entries, rank, world_size)
    infos: list[ParamInfo] = []
    offset = 0
    for fqn, p in named_params:
        pl = placements[fqn]
        gshape = tuple(p.shape)
        storage_dtype = p.dtype
        param_dtype = mp.compute_dtype_for(fqn, storage_dtype)
        grad_dtype = getattr(p, "grad_dtype", None)
        if grad_dtype == storage_dtype:
            grad_dtype = None  # only an explicit override (e.g. fp32 grads on bf16 shards) is recorded
        if mp.reduce_dtype is not None:
            reduce_dtype = mp.reduce_dtype
        elif spec.fsdp2_compatible and installed_fsdp2_accumulates_after_backward():
            reduce_dtype = param_dtype     # what the installed FSDP2 reduces in without a reduce dtype
        else:
            # gradients of the gathered parameter accumulate, and are reduced, in the dtype of the sharded
            # .grad: an explicit grad_dtype, else the storage (master) dtype
            wide = grad_dtype or storage_dtype
            reduce_dtype = wide if (wide.is_floating_point and param_dtype.is_floating_point
                                    and wide.itemsize >= param_dtype.itemsize) else param_dtype
        if bucket_layout is not None:
            bl: BucketParamStorageLayout = bucket_layout.param_layouts[fqn]
            local_shape, local_stride = bl.local_shape, bl.local_stride
            byte_offset, nbytes, extra = bl.byte_offset, bl.storage_nbytes, bl.bucket_layout
        else:
            ll = pl.local_storage_layout(gshape, rank, world_size)
            local_shape, local_stride = ll.local_shape, ll.local_stride
            itemsize = storage_dtype.itemsize
            # keep every slot 16-byte aligned so vector copies and TMA can address it
            offset = (offset + 15) // 16 * 16 if _wants_alignment(pl) else offset
            byte_offset, nbytes, extra = offset, ll.storage_numel * itemsize, None
            offset += nbytes
        infos.append(ParamInfo(
            fqn=fqn, global_shape=gshape, global_stride=_contiguous_stride(gshape),
            local_shape=tuple(local_shape), local_stride=tuple(local_stride),
            byte_offset=byte_offset, storage_nbytes=nbytes, storage_dtype=storage_dtype,
            param_dtype=param_dtype, reduce_dtype=reduce_dtype, grad_dtype=grad_dtype,
            placement=pl, requires_grad=p.requires_grad, outer_layout=get_global_layout(p),
            partial_grad_group=get_partial_grad_group(p), param_attrs=_user_attrs(p),
            shared_fqns=tuple(shared_names.get(fqn, ())), bucket_layout=extra,
            explicit_reduce_dtype=mp.reduce_dtype is not None))
    total = bucket_layout.total_bytes if bucket_layout is not None else offset
    brd = None
    for info in infos:
        if info.requires_grad:
            brd = info.reduce_dtype if brd is None else torch.promote_types(brd, info.reduce_dtype)
    for info in infos:
        info.bucket_reduce_dtype = brd if brd is not None else info.reduce_dtype
    return infos, total


def _wants_alignment(pl: Placement) -> bool:
    return getattr(pl, "align_slots", False)


# --------------------------------------------------------------------------- bucket assignment
def _module_names(root: nn.Module) -> dict[str, nn.Module]:
    return dict(root.named_modules())


def is_module_pattern_bucket(root: nn.Module, spec: BucketSpec) -> bool:
    """True when every pattern names a module (then the bucket hooks exactly those modules)."""
    mods = _module_names(root)
    hits = [pat in mods and pat != "" for pat in spec.patterns]
    params = dict(root.named_parameters(remove_duplicate=False))
    if any(hits) and not all(hits):
        others = [pat for pat, h in zip(spec.patterns, hits) if not h]
        if any(pat in params or any(fnmatch.fnmatchcase(n, pat) for n in params) for pat in others):
            raise ValueError(
                f"BucketSpec {spec.patterns!r} mixes module names and parameter patterns; use one kind.")
    return all(hits) and len(hits) > 0


def _matches(fqn: str, pattern: str, modules: Mapping[str, nn.Module]) -> bool:
    if fnmatch.fnmatchcase(fqn, pattern):
        return True
    if pattern in modules and pattern != "":
        return fqn.startswith(pattern + ".")
    # "layers.0" style prefix patterns and glob patterns over modules
    return fnmatch.fnmatchcase(fqn, pattern + ".*")


def assign_params_to_buckets(root: nn.Module, named_params: list[tuple[str, nn.Parameter]],
                             buckets: Sequence[BucketSpec],
                             shared_names: Mapping[str, tuple[str, ...]]) -> list[list[tuple[str, nn.Parameter]]]:
    modules = _module_names(root)
    assigned: list[list[tuple[str, nn.Parameter]]] = [[] for _ in buckets]
    owner: dict[str, int] = {}
    for fqn, p in named_params:
        names = (fqn, *shared_names.get(fqn, ()))
        hits = sorted({i for i, b in enumerate(buckets) for n in names
                       if any(_matches(n, pat, modules) for pat in b.patterns)})
        if not hits:
            raise ValueError(f"Parameter {fqn!r} matches no BucketSpec; every parameter must be in exactly one bucket.")
        if len(names) > 1:
            # every name of a tied parameter must land in the same bucket (as FSDP2 requires of a group)
            where = {n: sorted({i for i, b in enumerate(buckets) if any(_matches(n, pat, modules) for pat in b.patterns)})
                     for n in names}
            if len(hits) > 1 or any(not w for w in where.values()):
                listing = ", ".join(f"{n} -> " + (f"bucket {w[0]}" if len(w) == 1 else "no bucket" if not w else f"buckets {w}")
                                    for n, w in where.items())
                raise ValueError(f"Tied parameter {fqn!r} is shared with {list(names[1:])!r} ({listing}); put every name "
                                 "that refers to the parameter in the same BucketSpec.")
        if len(hits) > 1:
            raise ValueError(f"Parameter {fqn!r} matches more than one BucketSpec (buckets {hits}).")
        owner[fqn] = hits[0]
        assigned[hits[0]].append((fqn, p))
    return assigned


def fsdp2_param_order(root: nn.Module, named_params: list[tuple[str, nn.Parameter]]) -> list[tuple[str, nn.Parameter]]:
    """Order parameters the way ``fully_shard`` on ``root`` would see them: ``named_parameters``
    order of the module the group is applied to (children before a module's later-registered
    direct parameters only if registered so)."""
    want = {id(p): fqn for fqn, p in named_params}
    out, seen = [], set()

    def visit(mod: nn.Module, prefix: str):
        for name, child in mod.named_children():
            visit(child, f"{prefix}{name}.")
        for name, p in mod.named_parameters(recurse=False):
            if id(p) in want and id(p) not in seen:
                seen.add(id(p))
                out.append((want[id(p)], p))

    visit(root, "")
    for fqn, p in named_params:
        if id(p) not in seen:
            out.append((fqn, p))
    return out
