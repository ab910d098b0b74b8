"""Collective endpoints used by placements.

A ``Comm`` wraps one 1-D group of ranks and offers the small vocabulary the
placements need (all-gather, reduce-scatter in tensor and list form,
all-reduce). The default endpoint runs on ``torch.distributed`` (NCCL on GPUs,
gloo on CPU); ``parallel.symm`` provides an endpoint whose all-gather and
reduce-scatter are this library's own peer-memory kernels over NVLink.

Reduce-op mapping parity: ``custom_placements/utils.py:116-144`` of the
reference (SUM / AVG / pre-multiplied SUM / fp16 pre+post divide).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Sequence

import torch
import torch.distributed as dist

from ..placement_contract import GradientReduction


@dataclass(frozen=True)
class ReducePlan:
    """How to realise a ``GradientReduction`` on a given group size and dtype."""

    pre_divide: float | None   # divide the input by this before the collective
    op: str                    # "sum" | "avg" | "premul_sum"
    premul: float | None       # factor of a pre-multiplied sum
    post_divide: float | None  # divide the output by this afterwards
    factor: float | None = None  # the divide factor behind "premul_sum" (backends without that op sum, then divide by it)


def plan_reduction(reduction: GradientReduction, world_size: int, dtype: torch.dtype) -> ReducePlan:
    if reduction.op == dist.ReduceOp.SUM:
        return ReducePlan(None, "sum", None, None)
    f = reduction.factor(world_size)
    if world_size == 1:
        return ReducePlan(None, "sum", None, f if f != 1.0 else None)
    if dtype == torch.float16:
        # Split the division around the sum to keep fp16 in range: pre ~ sqrt(f).
        pre = 1
        while f % pre == 0 and f / pre > pre:
            pre *= 2
        return ReducePlan(float(pre), "sum", None, f / pre)
    if f == world_size:
        return ReducePlan(None, "avg", None, None)
    return ReducePlan(None, "premul_sum", 1.0 / f, None, factor=f)


class Comm:
    """Collectives over one process group (or no group at all for a single rank)."""

    def __init__(self, group: dist.ProcessGroup | None, rank: int, world_size: int,
                 device: torch.device):
        self.group = group
        self.rank = rank
        self.world_size = world_size
        self.device = device
        self._backend = None
        if group is not None and world_size > 1:
            self._backend = dist.get_backend(group)

    # ------------------------------------------------------------------ info
    @property
    def is_nccl(self) -> bool:
        return self._backend == "nccl"

    def ranks(self) -> list[int]:
        if self.group is None or self.world_size == 1:
            return [dist.get_rank() if dist.is_initialized() else 0]
        return dist.get_process_group_ranks(self.group)

    def new_like(self) -> "Comm":
        """A second communicator over the same ranks (lets reduce-scatters overlap all-gathers)."""
        if self.world_size == 1:
            return self
        g = dist.new_group(self.ranks(), backend=self._backend, use_local_synchronization=True)
        return type(self)(g, self.rank, self.world_size, self.device)

    # ------------------------------------------------------------------ all-gather
    def all_gather_into_tensor(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        if self.world_size == 1:
            if out.data_ptr() != inp.data_ptr():
                out.view(-1)[: inp.numel()].copy_(inp.view(-1))
            return None
        if not self.is_nccl and inp.untyped_storage().data_ptr() == out.untyped_storage().data_ptr():
            inp = inp.clone()  # gloo does not accept a send buffer inside the gather buffer
        return dist.all_gather_into_tensor(out, inp, group=self.group, async_op=async_op)

    def all_gather_list(self, outs: Sequence[torch.Tensor], inp: torch.Tensor, async_op: bool = False):
        """Uneven rows: ``outs[r]`` receives rank r's ``inp`` (sizes may differ per rank)."""
        if self.world_size == 1:
            if outs[0].data_ptr() != inp.data_ptr():
                outs[0].copy_(inp)
            return None
        if self.is_nccl:
            return dist.all_gather(list(outs), inp, group=self.group, async_op=async_op)
        # gloo has no uneven all-gather: one broadcast per row
        ranks = self.ranks()
        if outs[self.rank].data_ptr() != inp.data_ptr():
            outs[self.rank].copy_(inp)
        for r, t in enumerate(outs):
            if t.numel():
                dist.broadcast(t, src=ranks[r], group=self.group)
        return None

    # ------------------------------------------------------------------ reduce-scatter
    def _apply_plan_pre(self, inp: torch.Tensor, plan: ReducePlan) -> torch.Tensor:
        if plan.pre_divide is not None:
            inp.div_(plan.pre_divide)
        return inp

    def reduce_scatter_tensor(self, out: torch.Tensor, inp: torch.Tensor, plan: ReducePlan,
                              async_op: bool = False):
        """``out = reduce(inp.view(world, -1))[rank]`` under ``plan`` (``inp`` may be modified)."""
        self._apply_plan_pre(inp, plan)
        work = None
        if self.world_size == 1:
            out.copy_(inp.view(-1)[: out.numel()].view_as(out))
        elif self.is_nccl:
            if plan.op == "avg":
                op: Any = dist.ReduceOp.AVG
            elif plan.op == "premul_sum":
                op = dist._make_nccl_premul_sum(plan.premul)
            else:
                op = dist.ReduceOp.SUM
            work = dist.reduce_scatter_tensor(out, inp, op=op, group=self.group, async_op=async_op)
        else:
            # gloo has no pre-multiplied sum: sum, then divide the (smaller) output by the factor, which is
            # what FSDP2 does when told to use plain sums for its collectives. AVG runs natively.
            native_avg = plan.op == "avg" and not getattr(self, "_gloo_no_avg", False)
            try:
                dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.AVG if native_avg else dist.ReduceOp.SUM,
                                           group=self.group)
            except (RuntimeError, NotImplementedError):
                if native_avg:
                    self._gloo_no_avg, native_avg = True, False
                dist.all_reduce(inp, op=dist.ReduceOp.SUM, group=self.group)
                n = out.numel()
                out.copy_(inp.view(-1)[self.rank * n:(self.rank + 1) * n].view_as(out))
            if plan.op == "avg" and not native_avg:
                out.div_(self.world_size)
            if plan.op == "premul_sum" and plan.factor != 1.0:
                out.div_(plan.factor)
        if plan.post_divide is not None:
            if work is not None:
                work.wait()
                work = None
            out.div_(plan.post_divide)
        return work

    def reduce_scatter_list(self, out: torch.Tensor, inps: Sequence[torch.Tensor], plan: ReducePlan):
        """Uneven rows: ``out = reduce over ranks of inps[rank]``; ``inps[r]`` is what this rank
        contributes to rank r's row."""
        for t in inps:
            self._apply_plan_pre(t, plan)
        if self.world_size == 1:
            out.copy_(inps[0])
        elif self.is_nccl:
            if plan.op == "avg":
                op: Any = dist.ReduceOp.AVG
            elif plan.op == "premul_sum":
                op = dist._make_nccl_premul_sum(plan.premul)
            else:
                op = dist.ReduceOp.SUM
            dist.reduce_scatter(out, list(inps), op=op, group=self.group)
        else:
            for r, t in enumerate(inps):
                dist.reduce(t, dst=self.ranks()[r], op=dist.ReduceOp.SUM, group=self.group)
            out.copy_(inps[self.rank])
            if plan.op == "avg":
                out.div_(self.world_size)
            if plan.op == "premul_sum" and plan.factor != 1.0:
                out.div_(plan.factor)
        if plan.post_divide is not None:
            out.div_(plan.post_divide)
        return None

    # ------------------------------------------------------------------ misc
    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM):
        if self.world_size > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.group)


_comm_cache: dict[Any, Comm] = {}
_default_backend = None  # "symm" routes GPU meshes to the peer-memory collectives


def set_default_backend(name: str | None) -> None:
    """``"symm"``: all-gather / reduce-scatter of GPU meshes run on this library's NVLink
    peer-memory kernels; ``None`` / ``"nccl"``: on torch.distributed. Also settable with the
    environment variable ``FSB200_COMM``."""
    global _default_backend
    if name not in (None, "nccl", "symm"):
        raise ValueError(f"unknown comm backend {name!r}")
    _default_backend = None if name == "nccl" else name
    _comm_cache.clear()


def _backend() -> str | None:
    import os

    return _default_backend or (os.environ.get("FSB200_COMM") or None)


def mesh_group(mesh) -> tuple[dist.ProcessGroup | None, int, int, torch.device]:
    """Resolve a 1-D ``DeviceMesh`` / ``ProcessGroup`` / ``None`` to (group, rank, size, device)."""
    from torch.distributed.device_mesh import DeviceMesh

    if mesh is None:
        if dist.is_initialized():
            g = dist.group.WORLD
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
            return g, dist.get_rank(), dist.get_world_size(), dev
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        return None, 0, 1, dev
    if isinstance(mesh, DeviceMesh):
        if mesh.ndim != 1:
            raise ValueError(f"flex_shard needs a 1-D mesh per bucket, got a {mesh.ndim}-D mesh.")
        g = mesh.get_group()
        dev = torch.device(mesh.device_type)
        if dev.type == "cuda":
            dev = torch.device("cuda", torch.cuda.current_device())
        return g, mesh.get_local_rank(), mesh.size(), dev
    if isinstance(mesh, dist.ProcessGroup):
        backend = dist.get_backend(mesh)
        dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        return mesh, dist.get_rank(mesh), dist.get_world_size(mesh), dev
    if hasattr(mesh, "rank") and hasattr(mesh, "world_size"):  # test double (FakeMesh)
        return None, int(mesh.rank), int(mesh.world_size), torch.device(getattr(mesh, "device", "cpu"))
    raise TypeError(f"unsupported mesh object {type(mesh)!r}")


def comm_for(mesh) -> Comm:
    g, rank, ws, dev = mesh_group(mesh)
    key = (id(g), rank, ws, str(dev))
    c = _comm_cache.get(key)
    if c is None:
        if _backend() == "symm" and dev.type == "cuda" and ws > 1:
            from .symm import SymmComm

            c = SymmComm(g, rank, ws, dev)
        else:
            c = Comm(g, rank, ws, dev)
        _comm_cache[key] = c
    return c
