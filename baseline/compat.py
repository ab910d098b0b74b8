"""Forward-compatibility shims that let the unmodified reference package import and run on torch 2.11.

The reference pins ``torch>=2.16.0.dev0`` and uses a handful of symbols that older releases lack.
``install()`` adds stand-ins for exactly those symbols, each defined in terms of an operation the
installed torch already has, *before* ``import flex_shard``; nothing under ``baseline/_ref`` is
edited.  The shims change where a kernel comes from, not what the reference does:

=====================================================  =====================================================
missing symbol (where the reference uses it)            stand-in
=====================================================  =====================================================
``torch.distributed.checkpoint.CheckpointableTensor``   runtime-checkable protocol with the four layout
(``flex_shard/placement_contract.py:16``)               attributes
``dist.all_gather_single``                              ``dist.all_gather_into_tensor`` (same NCCL call)
(``custom_placements/shard.py:396``)
``dist.reduce_scatter_single``                          ``dist.reduce_scatter_tensor``
``torch.ops.fsdp._all_gather_copy_out_``                ``fsdp::split_with_sizes_copy`` (what FSDP2 of this
(``custom_placements/shard.py:292``)                    torch runs) for dim-0 shards; a strided ``copy_`` per
                                                        parameter for inner-dim shards
``torch.ops.fsdp.chunk_cat_mixed_dtype``                ``fsdp::chunk_cat`` (casts while packing) after
(``custom_placements/shard.py:469``)                    bringing stray dtypes / inner-dim chunks into line
``dist._spmd_no_typecheck``                             a null context
(``flex_shard/bucket_runtime.py:428``)
``dist._is_spmd_types_available``                       returns False (the optional ``spmd_types`` checker is
(``flex_shard/bucket_runtime.py:1568``)                 not installed)
``torchao`` (imported by the placement package's         placeholder modules; the FP8 / MXFP8 code that would
``__init__`` through the FP8 placement)                 call them raises
``Tensor._has_grad_dtype_override``                     ``grad_dtype`` differs from the tensor's dtype
(``flex_shard/bucket_storage.py:668``)
=====================================================  =====================================================
"""
from __future__ import annotations

import contextlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys
from typing import Protocol, runtime_checkable

import torch
import torch.distributed as dist

_installed: list[str] = []


def installed() -> list[str]:
    """Names of the symbols this process had to polyfill (empty on a new enough torch)."""
    return list(_installed)


def _all_gather_copy_out(outs, gathered, padded_local_numels, leading_sizes, world_size):
    numels = [int(n) for n in padded_local_numels]
    rows = gathered.view(world_size, -1)
    if all(int(lead) == 1 for lead in leading_sizes):
        torch.ops.fsdp.split_with_sizes_copy(rows, numels, dim=1, out=[o.view(world_size, -1) for o in outs])
        return
    for out, src, lead in zip(outs, rows.split(numels, dim=1), leading_sizes):
        lead = int(lead)
        if lead == 1:
            out.view(world_size, -1).copy_(src)
        else:
            rest = src.shape[1] // lead
            out.view(lead, world_size, rest).copy_(src.reshape(world_size, lead, rest).permute(1, 0, 2))


def _chunk_cat_mixed_dtype(tensors, dim, num_chunks, out, num_leading_dims=None):
    tensors = list(tensors)
    leads = list(num_leading_dims) if num_leading_dims is not None else [0] * len(tensors)
    for i, lead in enumerate(leads):
        if lead:
            tensors[i] = torch.cat(torch.chunk(tensors[i], num_chunks, dim=lead), dim=0)
    dtypes = {t.dtype for t in tensors}
    if len(dtypes) > 1:
        tensors = [t if t.dtype == out.dtype else t.to(out.dtype) for t in tensors]
        if len({t.dtype for t in tensors}) > 1:
            tensors = [t.to(out.dtype) for t in tensors]
    torch.ops.fsdp.chunk_cat(tensors, dim=dim, num_chunks=num_chunks, out=out)


class _AbsentPackage(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Serves ``import <name>.anything`` with empty modules whose attributes raise when *called*.

    The reference's placement package imports its FP8 placement (and with it ``torchao``) from its
    ``__init__``; the ``Shard`` path never calls into it.  With this finder the import succeeds and
    any actual use of the absent package fails with a clear message."""

    def __init__(self, name: str):
        self.name = name

    def find_spec(self, fullname, path=None, target=None):
        if fullname == self.name or fullname.startswith(self.name + "."):
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        pkg = self.name
        module.__path__ = []

        def __getattr__(attr):
            if attr.startswith("__"):
                raise AttributeError(attr)

            def absent(*_a, **_k):
                raise ModuleNotFoundError(f"{pkg} is not installed; {module.__name__}.{attr} is a placeholder")

            absent.__name__ = attr
            return absent

        module.__getattr__ = __getattr__


def install() -> list[str]:
    import torch.distributed.checkpoint as dcp

    if not hasattr(dcp, "CheckpointableTensor"):
        @runtime_checkable
        class CheckpointableTensor(Protocol):
            global_shape: tuple
            global_offsets: tuple
            local_offsets: tuple
            local_sizes: tuple

        dcp.CheckpointableTensor = CheckpointableTensor
        _installed.append("torch.distributed.checkpoint.CheckpointableTensor")

    if not hasattr(dist, "all_gather_single"):
        def all_gather_single(output, input, group=None, async_op=False):
            return dist.all_gather_into_tensor(output, input, group=group, async_op=async_op)

        dist.all_gather_single = all_gather_single
        _installed.append("dist.all_gather_single")

    if not hasattr(dist, "reduce_scatter_single"):
        def reduce_scatter_single(output, input, op=dist.ReduceOp.SUM, group=None, async_op=False):
            return dist.reduce_scatter_tensor(output, input, op=op, group=group, async_op=async_op)

        dist.reduce_scatter_single = reduce_scatter_single
        _installed.append("dist.reduce_scatter_single")

    if not hasattr(dist, "_spmd_no_typecheck"):
        dist._spmd_no_typecheck = contextlib.nullcontext
        _installed.append("dist._spmd_no_typecheck")

    if not hasattr(dist, "_is_spmd_types_available"):
        dist._is_spmd_types_available = lambda: False
        _installed.append("dist._is_spmd_types_available")

    import torch.distributed.fsdp  # noqa: F401  (registers the fsdp:: operator namespace)

    ns = torch.ops.fsdp
    try:
        ns._all_gather_copy_out_
    except (AttributeError, RuntimeError):
        setattr(ns, "_all_gather_copy_out_", _all_gather_copy_out)
        _installed.append("fsdp::_all_gather_copy_out_")
    try:
        ns.chunk_cat_mixed_dtype
    except (AttributeError, RuntimeError):
        setattr(ns, "chunk_cat_mixed_dtype", _chunk_cat_mixed_dtype)
        _installed.append("fsdp::chunk_cat_mixed_dtype")

    if not hasattr(torch.Tensor, "_has_grad_dtype_override"):
        def _has_grad_dtype_override(self):
            g = getattr(self, "grad_dtype", self.dtype)
            return g is not None and g != self.dtype

        torch.Tensor._has_grad_dtype_override = property(_has_grad_dtype_override)
        _installed.append("Tensor._has_grad_dtype_override")
    if importlib.util.find_spec("torchao") is None and not any(
            isinstance(f, _AbsentPackage) and f.name == "torchao" for f in sys.meta_path):
        sys.meta_path.append(_AbsentPackage("torchao"))
        _installed.append("torchao (import placeholder; FP8 / MXFP8 paths unusable)")
    return installed()


__all__ = ["install", "installed"]
