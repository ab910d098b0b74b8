"""Stream/event hand-off between the compute stream and the communication streams.

``begin_bucket_unshard`` runs a bucket's copy-in and all-gather on the unshard
stream behind an event of the caller's stream; ``begin_reduce_grad`` packs
gradients on the caller's stream and reduces on the reduce stream.
``StreamHandoff`` is the allocator-safety primitive: a buffer allocated on one
stream and last read on another is dropped only after its allocation stream
has been made to wait for that last read.

Parity: ``flex_shard/bucket_comm.py:94-217`` (the three ``begin_*`` entry points)
and ``:405-452`` (``StreamHandoff``) of the reference. CPU meshes (gloo) run
the same code with no streams.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from .placement_contract import (
    GradientReduction,
    PlacementPreparedReduceGrad,
    PlacementPreparedUnshard,
    PlacementReduceGradResult,
)


def _is_cuda(device: torch.device) -> bool:
    return device.type == "cuda"


class StreamHandoff:
    @staticmethod
    def release_after_current_stream(tensors: list, alloc_stream) -> None:
        """Make ``alloc_stream`` wait for everything queued so far on the current stream, then
        drop the references (their blocks return to ``alloc_stream``'s pool safely)."""
        if alloc_stream is not None and tensors:
            ev = torch.cuda.current_stream().record_event()
            alloc_stream.wait_event(ev)
        tensors.clear()


@dataclass
class PendingUnshard:
    prepared: PlacementPreparedUnshard
    event: Any | None            # recorded on the unshard stream after the collective
    stream: Any | None           # stream the gather buffers were allocated on
    explicit: bool = False


@dataclass
class PendingReduce:
    runtime: Any
    prepared: PlacementPreparedReduceGrad
    result: PlacementReduceGradResult | None
    event: Any | None
    keep: list = field(default_factory=list)


def begin_bucket_unshard(storage, persistent, stream) -> PendingUnshard:
    placement = storage.placement
    comm = storage.comm
    if stream is None or comm.world_size == 1:
        prep = placement.prepare_unshard_bucket(storage.infos, storage.byte_storage, comm, persistent)
        placement.run_prepared_unshard(prep, comm)
        return PendingUnshard(prep, None, None)
    ev = torch.cuda.current_stream().record_event()
    stream.wait_event(ev)
    with torch.cuda.stream(stream):
        prep = placement.prepare_unshard_bucket(storage.infos, storage.byte_storage, comm, persistent)
        placement.run_prepared_unshard(prep, comm)
        done = stream.record_event()
    return PendingUnshard(prep, done, stream)


def begin_explicit_bucket_unshard(storage, persistent, async_op: bool) -> PendingUnshard:
    """Gather on the caller's stream (for schedules that drive unshards themselves)."""
    placement = storage.placement
    prep = placement.prepare_unshard_bucket(storage.infos, storage.byte_storage, storage.comm, persistent)
    placement.run_prepared_unshard(prep, storage.comm, async_op=async_op)
    return PendingUnshard(prep, None, None, explicit=True)


def begin_reduce_grad(runtime, grads, reduce_dtype, reduction: GradientReduction, stream) -> PendingReduce:
    storage = runtime.storage
    placement = storage.placement
    comm = storage.reduce_comm
    prep = placement.prepare_reduce_grad(storage.infos_for_reduce, grads, comm, reduce_dtype)
    fused_opt = getattr(storage, "_fused_opt", None)
    if fused_opt is not None and prep.extra.get("peer_bucket") is not None:
        adam = fused_opt.fused_bucket_args(storage)
        if adam is not None:
            prep.extra["adam"] = adam
    if stream is None or comm.world_size == 1:
        res = placement.reduce_prepared_grad(prep, comm, reduction)
        runtime.accumulate_sharded_grads(res)
        ctx = runtime.context
        if (fused_opt is not None and comm.world_size == 1 and ctx.cuda and not ctx.manual_finalization):
            # one rank: the gradients are final here; let the optimizer update this bucket on the side
            # stream while the rest of the backward pass keeps the tensor cores busy
            fused_opt.step_bucket_in_backward(storage, ctx.reduce_stream)
        return PendingReduce(runtime, prep, res, None)
    ev = torch.cuda.current_stream().record_event()
    stream.wait_event(ev)
    with torch.cuda.stream(stream):
        res = placement.reduce_prepared_grad(prep, comm, reduction)
        runtime.accumulate_sharded_grads(res)
        done = stream.record_event()
    return PendingReduce(runtime, prep, res, done, keep=[prep.send])
