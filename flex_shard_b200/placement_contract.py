"""The contract between the bucket runtime and a storage scheme (a *placement*).

A placement decides which part of every parameter of a bucket a rank stores,
how the bucket's byte buffer is laid out, how the bucket is gathered for
compute and how its gradients are reduced back into the local layout. The
runtime only ever talks to a placement through the methods below, in this
order per use::

    prepare_unshard_bucket -> run_prepared_unshard -> finish_prepared_unshard
    prepare_reduce_grad    -> reduce_prepared_grad

Parity: mirrors the role of ``flex_shard/placement_contract.py:180-454`` of the
reference (the ABC, the four request/result records, ``GradientReduction``,
``GlobalLayout`` and its composition), re-derived for a runtime whose
collectives are objects (``parallel.comm.Comm``) that may be NCCL, gloo or
symmetric-memory kernels.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, Sequence

import torch
import torch.distributed as dist

if TYPE_CHECKING:  # pragma: no cover
    from .bucket_storage import ParamInfo
    from .parallel.comm import Comm


# --------------------------------------------------------------------------- layouts
@dataclass(frozen=True)
class LocalStorageLayout:
    """Shape/stride/extent of one parameter's local shard inside its slot."""

    local_shape: tuple[int, ...]
    local_stride: tuple[int, ...]
    storage_numel: int  # elements reserved for the slot (>= numel of the local shard)


@dataclass(frozen=True)
class BucketParamStorageLayout:
    local_shape: tuple[int, ...]
    local_stride: tuple[int, ...]
    byte_offset: int
    storage_nbytes: int
    bucket_layout: Any | None = None


@dataclass(frozen=True)
class BucketStorageLayout:
    """Placement-owned storage layout for a whole bucket."""

    param_layouts: dict[str, BucketParamStorageLayout]
    total_bytes: int


@dataclass(frozen=True)
class GlobalLayout:
    """Boxes of the full parameter that one rank's local tensor holds.

    Chunk ``i`` of the local tensor starts at ``local_offsets[i]``, has size
    ``local_sizes[i]`` and sits at ``global_offsets[i]`` of a tensor of shape
    ``global_shape``. The four fields are what the sharded checkpoint format
    stores for each tensor.
    """

    global_shape: tuple[int, ...]
    global_offsets: tuple[tuple[int, ...], ...]
    local_offsets: tuple[tuple[int, ...], ...]
    local_sizes: tuple[tuple[int, ...], ...]


_LAYOUT_FIELDS = ("global_shape", "global_offsets", "local_offsets", "local_sizes")


def get_global_layout(tensor: torch.Tensor) -> GlobalLayout | None:
    """Return the layout ``tensor`` declares, or ``None`` if it declares none."""
    if not all(hasattr(tensor, f) for f in _LAYOUT_FIELDS):
        return None
    return GlobalLayout(
        global_shape=tuple(tensor.global_shape),
        global_offsets=tuple(map(tuple, tensor.global_offsets)),
        local_offsets=tuple(map(tuple, tensor.local_offsets)),
        local_sizes=tuple(map(tuple, tensor.local_sizes)),
    )


def set_global_layout(tensor: torch.Tensor, layout: GlobalLayout) -> None:
    """Declare where ``tensor`` sits in the full parameter (outer TP/EP sharding)."""
    tensor.global_shape = layout.global_shape
    tensor.global_offsets = layout.global_offsets
    tensor.local_offsets = layout.local_offsets
    tensor.local_sizes = layout.local_sizes


_PARTIAL_GRAD_GROUP_ATTR = "_fsb_partial_grad_group"


def set_partial_grad_group(tensor: torch.Tensor, group: dist.ProcessGroup) -> None:
    """Each rank of ``group`` computes only part of ``tensor``'s gradient; the runtime sums
    the unsharded gradient over ``group`` before the bucket's reduce-scatter."""
    setattr(tensor, _PARTIAL_GRAD_GROUP_ATTR, group)


def get_partial_grad_group(tensor: torch.Tensor) -> dist.ProcessGroup | None:
    return getattr(tensor, _PARTIAL_GRAD_GROUP_ATTR, None)


def full_layout(shape: Sequence[int]) -> GlobalLayout:
    shape = tuple(shape)
    zero = tuple(0 for _ in shape)
    return GlobalLayout(shape, (zero,), (zero,), (shape,))


def compose_global_layouts(outer: GlobalLayout, inner: GlobalLayout) -> GlobalLayout:
    """``outer``: T -> G, ``inner``: L -> T; the result maps L directly into G.

    Every pair of overlapping boxes in T's coordinates yields one chunk.
    """
    g_off, l_off, sizes = [], [], []
    for og, ol, osz in zip(outer.global_offsets, outer.local_offsets, outer.local_sizes):
        for ig, il, isz in zip(inner.global_offsets, inner.local_offsets, inner.local_sizes):
            lo = tuple(max(a, b) for a, b in zip(ig, ol))
            hi = tuple(min(a + sa, b + sb) for a, sa, b, sb in zip(ig, isz, ol, osz))
            if any(h <= l for l, h in zip(lo, hi)):
                continue
            g_off.append(tuple(g + l - o for g, l, o in zip(og, lo, ol)))
            l_off.append(tuple(b + l - a for b, l, a in zip(il, lo, ig)))
            sizes.append(tuple(h - l for l, h in zip(lo, hi)))
    return GlobalLayout(outer.global_shape, tuple(g_off), tuple(l_off), tuple(sizes))


# --------------------------------------------------------------------------- reduction spec
@dataclass(frozen=True)
class GradientReduction:
    """What a bucket's gradient reduction must produce: the sum over the mesh and, with
    ``op=AVG``, divided by ``divide_factor`` (default: the mesh size)."""

    op: Any = dist.ReduceOp.AVG
    divide_factor: float | None = None

    def __post_init__(self) -> None:
        if self.op not in (dist.ReduceOp.AVG, dist.ReduceOp.SUM):
            raise ValueError(f"gradient_reduce_op must be AVG or SUM, got {self.op!r}.")
        if self.divide_factor is None:
            return
        if not math.isfinite(self.divide_factor) or self.divide_factor <= 0:
            raise ValueError(
                f"gradient_divide_factor must be a positive number, got {self.divide_factor!r}."
            )
        if self.op == dist.ReduceOp.SUM:
            raise ValueError(
                "gradient_divide_factor requires gradient_reduce_op=AVG; SUM does not divide gradients."
            )

    def factor(self, world_size: int) -> float:
        """The number the summed gradient is divided by."""
        if self.op == dist.ReduceOp.SUM:
            return 1.0
        return float(world_size) if self.divide_factor is None else float(self.divide_factor)


# --------------------------------------------------------------------------- request / result records
@dataclass
class PlacementPreparedUnshard:
    """State between ``prepare_unshard_bucket`` and ``finish_prepared_unshard``.

    ``send`` / ``recv`` are the collective's buffers; ``persistent`` (optional) are the
    per-parameter unsharded buffers the runtime owns across steps: a placement with
    ``refills_persistent_buffers_in_finish`` copies into them in ``finish``; others gather
    straight into them in ``run``.
    """

    infos: list["ParamInfo"]
    send: torch.Tensor | None = None
    recv: torch.Tensor | None = None
    work: Any | None = None
    persistent: list[torch.Tensor] | None = None
    local_copy_out: bool = False
    extra: dict = field(default_factory=dict)


@dataclass
class PlacementUnshardResult:
    """Per-parameter unsharded tensors (in ``infos`` order) plus buffers to release later."""

    tensors: list[torch.Tensor]
    keepalive: list[torch.Tensor] = field(default_factory=list)


@dataclass
class PlacementPreparedReduceGrad:
    infos: list["ParamInfo"]
    send: torch.Tensor | None
    reduce_dtype: torch.dtype
    extra: dict = field(default_factory=dict)


@dataclass
class PlacementReduceGradResult:
    """Reduced local gradients (views of ``output``), one per info; ``None`` for empty shards."""

    grads: list[torch.Tensor | None]
    output: torch.Tensor | None = None
    work: Any | None = None


# --------------------------------------------------------------------------- the ABC
class Placement(ABC):
    """A storage scheme for one parameter (and, through the ``*_bucket`` hooks, its bucket)."""

    # True when ``finish_prepared_unshard`` copies from a gather buffer into the runtime's
    # persistent per-parameter buffers (so those need not exist before ``finish``).
    refills_persistent_buffers_in_finish: bool = False

    # ---- identity
    @abstractmethod
    def __eq__(self, other: object) -> bool: ...

    @abstractmethod
    def __hash__(self) -> int: ...

    def bucket_compatibility_key(self) -> Any:
        """Placements of one bucket must share this key (they run one collective together)."""
        return type(self)

    # ---- per-parameter geometry
    @abstractmethod
    def compute_local_shape(self, global_shape: Sequence[int], rank: int, world_size: int) -> tuple[int, ...]: ...

    def compute_local_numel(self, global_shape: Sequence[int], rank: int, world_size: int) -> int:
        return math.prod(self.compute_local_shape(global_shape, rank, world_size))

    @abstractmethod
    def extract_local_shard(self, full: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
        """This rank's part of ``full`` (a view where possible)."""

    @abstractmethod
    def local_storage_layout(self, global_shape: Sequence[int], rank: int, world_size: int) -> LocalStorageLayout: ...

    def bucket_storage_layout(self, infos_in: "list[tuple[str, tuple[int, ...], torch.dtype, Placement]]",
                              rank: int, world_size: int) -> BucketStorageLayout | None:
        """Whole-bucket layout; ``None`` means: pack the per-parameter slots back to back."""
        return None

    def copy_param_to_storage(self, info: "ParamInfo", full: torch.Tensor, storage_view: torch.Tensor,
                              rank: int, world_size: int) -> None:
        storage_view.copy_(self.extract_local_shard(full, rank, world_size))

    def make_local_storage_view(self, info: "ParamInfo", byte_storage: torch.Tensor) -> torch.Tensor:
        flat = byte_storage[info.byte_offset: info.byte_offset + info.storage_nbytes].view(info.storage_dtype)
        return flat.as_strided(info.local_shape, info.local_stride)

    @abstractmethod
    def global_layout(self, global_shape: Sequence[int], rank: int, world_size: int) -> GlobalLayout:
        """Checkpoint layout of the local shard inside the (pre-outer-sharding) parameter."""

    # ---- bucket lifecycle: gather
    @abstractmethod
    def prepare_unshard_bucket(self, infos: "list[ParamInfo]", byte_storage: torch.Tensor, comm: "Comm",
                               persistent: list[torch.Tensor] | None) -> PlacementPreparedUnshard: ...

    @abstractmethod
    def run_prepared_unshard(self, prepared: PlacementPreparedUnshard, comm: "Comm", async_op: bool = False) -> None: ...

    @abstractmethod
    def finish_prepared_unshard(self, prepared: PlacementPreparedUnshard, comm: "Comm",
                                persistent: list[torch.Tensor]) -> PlacementUnshardResult: ...

    # ---- bucket lifecycle: gradient reduction
    @abstractmethod
    def prepare_reduce_grad(self, infos: "list[ParamInfo]", grads: list[torch.Tensor], comm: "Comm",
                            reduce_dtype: torch.dtype) -> PlacementPreparedReduceGrad: ...

    @abstractmethod
    def reduce_prepared_grad(self, prepared: PlacementPreparedReduceGrad, comm: "Comm",
                             reduction: GradientReduction) -> PlacementReduceGradResult: ...

    def reduces_grads_in_param_layout(self, infos: "list[ParamInfo]") -> bool:
        """True when unsharded grads should be allocated as views of one bucket-shaped buffer so
        the reduction can send it as is."""
        return False

    def unsharded_buffer_numel(self, info: "ParamInfo", world_size: int) -> int:
        """Elements of the persistent unsharded buffer of one parameter (may include padding)."""
        return math.prod(info.global_shape)
