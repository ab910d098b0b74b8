"""``BucketedBlockShard``: each rank stores one contiguous range of a flat, parameter-major bucket
(the FSDP1 / Megatron distributed-optimizer / veScale-FSDP layout).

Planning (parity: ``custom_placements/block_shard.py:711-754`` of the reference): parameters are
laid out back to back, each starting on a multiple of ``align = lcm(row sizes)``; the total is
padded to a multiple of ``align * sum(blocks_per_rank)``; rank r holds
``blocks_per_rank[r]`` blocks of ``padded_total / sum(blocks)`` elements. Because every cut falls
on a multiple of every row size, each parameter's local part is a whole number of rows.

Gather: the local buffer *is* the send buffer and the all-gather lands straight in the persistent
unsharded bucket, of which the parameters are views (no copy-in, no copy-out). Reduction: when the
gradients are views of one bucket-shaped buffer it is reduce-scattered as it is; otherwise they are
first copied into a zeroed bucket.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ..parallel.comm import plan_reduction
from ..placement_contract import (
    BucketParamStorageLayout,
    BucketStorageLayout,
    GlobalLayout,
    GradientReduction,
    LocalStorageLayout,
    Placement,
    PlacementPreparedReduceGrad,
    PlacementPreparedUnshard,
    PlacementReduceGradResult,
    PlacementUnshardResult,
)
from ..ops.segments import run_segment_ops
from ..utils.profiling import record
from .sliced import contig_stride


def _lcm(values):
    out = 1
    for v in values:
        out = out * v // math.gcd(out, v)
    return out


class FlatBucketPlan:
    """Geometry of one flat bucket (in elements)."""

    def __init__(self, shapes: Sequence[tuple[int, ...]], blocks_per_rank: Sequence[int]):
        self.shapes = [tuple(s) for s in shapes]
        self.blocks = tuple(int(b) for b in blocks_per_rank)
        rows = [math.prod(s[1:]) if len(s) > 1 else 1 for s in self.shapes]
        self.row_sizes = rows
        self.align = _lcm([r for r in rows if r > 0] or [1])
        self.param_off = []
        off = 0
        for s in self.shapes:
            off = -(-off // self.align) * self.align
            self.param_off.append(off)
            off += math.prod(s)
        self.total = off
        unit = self.align * sum(self.blocks)
        self.padded_total = max(unit, -(-off // unit) * unit)
        self.block = self.padded_total // sum(self.blocks)

    def rank_range(self, r: int) -> tuple[int, int]:
        lo = sum(self.blocks[:r]) * self.block
        return lo, lo + self.blocks[r] * self.block

    def local_rows(self, i: int, r: int) -> tuple[int, int]:
        """Global row range [r0, r1) of parameter i held by rank r."""
        lo, hi = self.rank_range(r)
        p0 = self.param_off[i]
        p1 = p0 + math.prod(self.shapes[i])
        a, b = max(lo, p0), min(hi, p1)
        if b <= a:
            return 0, 0
        rs = self.row_sizes[i]
        return (a - p0) // rs, (b - p0) // rs

    @property
    def uniform(self) -> bool:
        return len(set(self.blocks)) == 1


class BucketedBlockShard(Placement):
    refills_persistent_buffers_in_finish = False

    def __init__(self, blocks_per_rank: Sequence[int], dims: Sequence[int] = (0,)):
        self.blocks_per_rank = tuple(int(b) for b in blocks_per_rank)
        self.dims = tuple(dims)
        if self.dims != (0,):
            raise ValueError("BucketedBlockShard supports dims=(0,) (row-major flat buckets)")
        if any(b < 0 for b in self.blocks_per_rank) or sum(self.blocks_per_rank) <= 0:
            raise ValueError("blocks_per_rank must be non-negative with a positive sum")

    def __eq__(self, other):
        return type(other) is type(self) and other.blocks_per_rank == self.blocks_per_rank

    def __hash__(self):
        return hash((type(self).__name__, self.blocks_per_rank))

    def __repr__(self):
        return f"{type(self).__name__}(blocks_per_rank={self.blocks_per_rank})"

    def bucket_compatibility_key(self):
        return (type(self).__name__, self.blocks_per_rank)

    # ---- per-parameter geometry (nominal: the real cut needs the whole bucket)
    def compute_local_shape(self, global_shape, rank, world_size):
        if len(self.blocks_per_rank) != world_size:
            raise ValueError(f"placement has {len(self.blocks_per_rank)} ranks, the mesh has {world_size}")
        n = global_shape[0]
        c = -(-n // world_size)
        lo, hi = min(n, rank * c), min(n, (rank + 1) * c)
        return (hi - lo, *global_shape[1:])

    def extract_local_shard(self, full, rank, world_size):
        raise RuntimeError("BucketedBlockShard cuts parameters through its bucket plan; use the bucket storage")

    def local_storage_layout(self, global_shape, rank, world_size):
        ls = self.compute_local_shape(global_shape, rank, world_size)
        return LocalStorageLayout(ls, contig_stride(ls), math.prod(ls))

    def global_layout(self, global_shape, rank, world_size):
        ls = self.compute_local_shape(global_shape, rank, world_size)
        c = -(-global_shape[0] // world_size)
        nd = len(global_shape)
        if ls[0] == 0:
            return GlobalLayout(tuple(global_shape), (), (), ())
        return GlobalLayout(tuple(global_shape), ((min(global_shape[0], rank * c),) + (0,) * (nd - 1),),
                            ((0,) * nd,), (ls,))

    # ---- whole-bucket layout
    def plan(self, shapes) -> FlatBucketPlan:
        return FlatBucketPlan(shapes, self.blocks_per_rank)

    def bucket_storage_layout(self, entries, rank, world_size):
        dtypes = {e[2] for e in entries}
        if len(dtypes) != 1:
            raise ValueError("a BucketedBlockShard bucket needs one parameter dtype")
        itemsize = next(iter(dtypes)).itemsize
        plan = self.plan([e[1] for e in entries])
        lo, hi = plan.rank_range(rank)
        layouts = {}
        for i, (fqn, shape, dtype, _) in enumerate(entries):
            r0, r1 = plan.local_rows(i, rank)
            ls = (r1 - r0, *shape[1:])
            start = plan.param_off[i] + r0 * plan.row_sizes[i]
            off = (max(start, lo) - lo) if r1 > r0 else 0
            layouts[fqn] = BucketParamStorageLayout(ls, contig_stride(ls), off * itemsize, math.prod(ls) * itemsize,
                                                    bucket_layout={"index": i, "rows": (r0, r1), "plan": plan})
        return BucketStorageLayout(layouts, (hi - lo) * itemsize)

    def copy_param_to_storage(self, info, full, storage_view, rank, world_size):
        r0, r1 = info.bucket_layout["rows"]
        if r1 > r0:
            storage_view.copy_(full[r0:r1])

    def bucket_global_layout(self, info, rank, world_size):
        r0, r1 = info.bucket_layout["rows"]
        g = tuple(info.global_shape)
        nd = len(g)
        if r1 <= r0:
            return GlobalLayout(g, (), (), ())
        return GlobalLayout(g, ((r0,) + (0,) * (nd - 1),), ((0,) * nd,), ((r1 - r0, *g[1:]),))

    # ---- unsharded bucket owned by the runtime (one buffer, parameters are views)
    def alloc_unsharded_bucket(self, storage):
        plan: FlatBucketPlan = storage.infos[0].bucket_layout["plan"]
        dtype = storage.infos[0].param_dtype
        base = torch.empty(plan.padded_total, dtype=dtype, device=storage.device)
        views = [base[plan.param_off[i]: plan.param_off[i] + info.global_numel].view(info.global_shape)
                 for i, info in enumerate(storage.infos)]
        return base, views

    # ---- gather
    def prepare_unshard_bucket(self, infos, byte_storage, comm, persistent):
        prep = PlacementPreparedUnshard(infos=infos, persistent=persistent)
        plan: FlatBucketPlan = infos[0].bucket_layout["plan"]
        prep.extra["plan"] = plan
        src_dtype, dst_dtype = infos[0].storage_dtype, infos[0].param_dtype
        local = byte_storage.view(src_dtype)
        if src_dtype != dst_dtype:
            with record("FlexShard::copy_in"):
                local = local.to(dst_dtype)
        prep.send = local
        return prep

    def run_prepared_unshard(self, prepared, comm, async_op=False):
        plan: FlatBucketPlan = prepared.extra["plan"]
        base = prepared.persistent[0]._base if prepared.persistent[0]._base is not None else prepared.persistent[0]
        base = prepared.extra.get("base", base)
        bucket = base.view(-1)[: plan.padded_total] if base.numel() >= plan.padded_total else None
        if bucket is None:
            raise RuntimeError("unsharded bucket buffer is missing")
        prepared.extra["bucket"] = bucket
        W = comm.world_size
        with record("FlexShard::all_gather"):
            if W == 1:
                bucket[: prepared.send.numel()].copy_(prepared.send)
            elif plan.uniform:
                prepared.work = comm.all_gather_into_tensor(bucket, prepared.send, async_op=async_op)
            else:
                rows = [bucket[slice(*plan.rank_range(r))] for r in range(W)]
                prepared.work = comm.all_gather_list(rows, prepared.send, async_op=async_op)

    def finish_prepared_unshard(self, prepared, comm, persistent):
        if prepared.work is not None:
            prepared.work.wait()
            prepared.work = None
        return PlacementUnshardResult(list(persistent))  # view-out: the parameters alias the bucket

    # ---- gradients
    def reduces_grads_in_param_layout(self, infos) -> bool:
        return all(i.param_dtype == (i.bucket_reduce_dtype or i.reduce_dtype) for i in infos)

    def alloc_grad_bucket(self, storage, unsharded_params):
        plan: FlatBucketPlan = storage.infos[0].bucket_layout["plan"]
        dtype = storage.bucket_reduce_dtype
        buf = torch.zeros(plan.padded_total, dtype=dtype, device=storage.device)
        for i, (info, up) in enumerate(zip(storage.infos, unsharded_params)):
            if info.requires_grad and up.requires_grad and up.grad is None and up.dtype == dtype:
                up.grad = buf[plan.param_off[i]: plan.param_off[i] + info.global_numel].view(info.global_shape)
        storage._grad_bucket = buf

    def prepare_reduce_grad(self, infos, grads, comm, reduce_dtype):
        plan: FlatBucketPlan = infos[0].bucket_layout["plan"]
        # path (a): every gradient already is the matching view of one bucket-shaped buffer
        base = None
        in_place = True
        for info, g in zip(infos, grads):
            i = info.bucket_layout["index"]
            b = g._base if g._base is not None else None
            if (b is None or b.numel() != plan.padded_total or b.dtype != reduce_dtype
                    or g.storage_offset() != b.storage_offset() + plan.param_off[i] or not g.is_contiguous()
                    or (base is not None and b.data_ptr() != base.data_ptr())):
                in_place = False
                break
            base = b
        with record("FlexShard::reduce_scatter_copy_in"):
            if in_place and base is not None and len(infos) == len(plan.shapes):
                send = base
            elif all(g.dtype == reduce_dtype or {g.dtype, reduce_dtype} == {torch.float32, torch.bfloat16} for g in grads):
                # path (b): one pass writes every gradient (cast to the reduce dtype) and zeroes the gaps
                # between parameters and the padded tail; copies and zero-fills touch disjoint bytes, so they
                # share one launch
                send = torch.empty(plan.padded_total, dtype=reduce_dtype, device=grads[0].device)
                spans = sorted((plan.param_off[info.bucket_layout["index"]], info.global_numel, g, info)
                               for info, g in zip(infos, grads))
                ops, pos = [], 0
                for off, n, g, info in spans:
                    if off > pos:
                        ops.append((send[pos:off], None))
                    ops.append((send[off:off + n].view(info.global_shape), g))
                    pos = off + n
                if pos < plan.padded_total:
                    ops.append((send[pos:], None))
                run_segment_ops(ops)
            else:
                # path (c): zero the bucket, then copy parameter by parameter
                send = torch.zeros(plan.padded_total, dtype=reduce_dtype, device=grads[0].device)
                for info, g in zip(infos, grads):
                    i = info.bucket_layout["index"]
                    send[plan.param_off[i]: plan.param_off[i] + info.global_numel].view(info.global_shape).copy_(g)
        prep = PlacementPreparedReduceGrad(infos=infos, send=send, reduce_dtype=reduce_dtype)
        prep.extra["plan"] = plan
        return prep

    def reduce_prepared_grad(self, prepared, comm, reduction: GradientReduction):
        plan: FlatBucketPlan = prepared.extra["plan"]
        W, rank = comm.world_size, comm.rank
        rplan = plan_reduction(reduction, W, prepared.reduce_dtype)
        lo, hi = plan.rank_range(rank)
        with record("FlexShard::reduce_scatter"):
            if W == 1:
                out = prepared.send
                if rplan.post_divide is not None:
                    out.div_(rplan.post_divide)
            elif plan.uniform:
                out = torch.empty(hi - lo, dtype=prepared.reduce_dtype, device=prepared.send.device)
                comm.reduce_scatter_tensor(out, prepared.send, rplan)
            else:
                out = torch.empty(hi - lo, dtype=prepared.reduce_dtype, device=prepared.send.device)
                comm.reduce_scatter_list(out, [prepared.send[slice(*plan.rank_range(r))] for r in range(W)], rplan)
        grads = []
        for info in prepared.infos:
            i = info.bucket_layout["index"]
            r0, r1 = plan.local_rows(i, rank)
            if r1 <= r0:
                grads.append(torch.zeros(info.local_shape, dtype=prepared.reduce_dtype, device=out.device))
                continue
            start = plan.param_off[i] + r0 * plan.row_sizes[i] - lo
            grads.append(out[start:start + info.local_numel].view(info.local_shape))
        return PlacementReduceGradResult(grads=grads, output=out)


def make_bucketed_block_shard_placement_fn(blocks_per_rank: Sequence[int] | None = None, *,
                                           dims: Sequence[int] = (0,)):
    if tuple(dims) != (0,):
        raise ValueError("BucketedBlockShard supports dims=(0,) (row-major flat buckets)")

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        if blocks_per_rank and len(blocks_per_rank) != W:
            raise ValueError(f"blocks_per_rank names {len(blocks_per_rank)} ranks, the mesh has {W}")
        pl = BucketedBlockShard(tuple(blocks_per_rank) if blocks_per_rank else (1,) * W)
        return {f: pl for f, _ in named_params}

    return fn
