"""Blockwise-quantised all-gather placements.

``BlockwiseQuantBucketedBlockShard`` stores dense master rows (bf16/fp32) cut on whole quantisation
blocks, so that each rank can quantise its own rows locally and the all-gather moves quantised
bytes plus scales: about half the bytes of a bf16 gather for FP8. The gathered weight is bitwise
what "gather bf16, then quantise" would give, because a tile's data and scale depend on that tile
only and no tile is split between ranks.

* Planner (parity ``custom_placements/blockwise_quant_bucketed_block_shard.py:411-519`` of the
  reference): the bucket is a parameter-major list of units of ``shard_block_rows`` rows; the units
  are cut into W contiguous runs minimising the largest run cost (payload bytes: data + scales),
  found by binary search on the cost followed by greedy cuts.
* Rank payload: ``[qdata | pad to 16 B | scales | pad to 16 B]`` as bytes, all ranks padded to the
  largest (parity ``:633-674``); one ``all_gather_into_tensor`` of ``uint8``.
* The forward's payload is kept for the backward re-gather (activation-checkpoint recompute) and
  dropped as soon as the master storage changes (parity ``:899-971``).
* Gradients are dense and reduce through the slice engine (each rank's row range is one slice).

``Fp8BucketedBlockShard``: e4m3 data, one fp32 reciprocal scale per 128x128 tile, quantised by
``fsb_fp8_quant_weight`` (parity ``custom_placements/fp8_bucketed_block_shard.py:114-218``).
"""
from __future__ import annotations

import math
from typing import Callable, Protocol, Sequence

import torch

from ..placement_contract import PlacementPreparedUnshard, PlacementUnshardResult
from ..ops.segments import run_segment_ops
from ..utils.profiling import record
from .sliced import Piece, SlicedPlacement


# --------------------------------------------------------------------------- planner
def partition_min_max(costs: Sequence[int], parts: int) -> list[int]:
    """Cut ``costs`` into ``parts`` contiguous runs (some possibly empty) minimising the largest run
    sum; returns the ``parts + 1`` cut indices."""
    n = len(costs)
    if n == 0:
        return [0] * (parts + 1)

    def cuts_for(limit):
        cuts, run = [0], 0
        for i, c in enumerate(costs):
            if run + c > limit and run > 0:
                cuts.append(i)
                run = 0
            run += c
        cuts.append(n)
        return cuts

    lo, hi = max(costs), sum(costs)
    while lo < hi:
        mid = (lo + hi) // 2
        if len(cuts_for(mid)) - 1 <= parts:
            hi = mid
        else:
            lo = mid + 1
    cuts = cuts_for(lo)
    # split the largest runs until there are exactly `parts` of them (or units run out), then pad
    while len(cuts) - 1 < parts:
        sizes = [(sum(costs[cuts[i]:cuts[i + 1]]), i) for i in range(len(cuts) - 1) if cuts[i + 1] - cuts[i] > 1]
        if not sizes:
            break
        _, i = max(sizes)
        a, b = cuts[i], cuts[i + 1]
        half, acc, cut = sum(costs[a:b]) / 2, 0, a + 1
        for j in range(a, b - 1):
            acc += costs[j]
            cut = j + 1
            if acc >= half:
                break
        cuts.insert(i + 1, cut)
    while len(cuts) - 1 < parts:
        cuts.append(n)
    return cuts


class BlockwiseQuantBucketedBlockShard(SlicedPlacement):
    """One parameter's row ranges per rank (decided by the bucket planner) + the quantiser."""

    refills_persistent_buffers_in_finish = True
    shard_block_rows = 128
    allows_mixed_dtypes = False

    def __init__(self, row_ranges: Sequence[tuple[int, int]], weight_factory: Callable | None = None):
        if weight_factory is not None and not callable(weight_factory):
            raise TypeError("weight_factory must be callable")
        self.row_ranges = tuple((int(a), int(b)) for a, b in row_ranges)
        # builds the tensor the consumer sees from the gathered operands (default: this library's wrapper class)
        self.weight_factory = weight_factory

    def __eq__(self, other):
        return (type(other) is type(self) and other.row_ranges == self.row_ranges
                and other.weight_factory is self.weight_factory)

    def __hash__(self):
        return hash((type(self).__name__, self.row_ranges))

    def __repr__(self):
        return f"{type(self).__name__}(row_ranges={self.row_ranges})"

    def bucket_compatibility_key(self):
        return type(self).__name__

    def pieces(self, global_shape, rank, world_size):
        if len(self.row_ranges) != world_size:
            raise ValueError(f"placement planned for {len(self.row_ranges)} ranks, the mesh has {world_size}")
        a, b = self.row_ranges[rank]
        return [Piece(0, a, b - a)] if b > a else []

    @staticmethod
    def matrix_dims(shape, rows: int) -> tuple[int, int]:
        """The matrix that ``rows`` leading rows of a weight are quantised as: a 2-D weight ``[out, in]`` is its
        own matrix; a stacked weight ``[*stack, out, in]`` (experts) is the stack's matrices one under the other,
        ``[prod(stack) * out, in]``, and ``rows`` counts entries of the leading dimension. ``out`` is a multiple
        of the block height for stacked weights, so no quantisation block straddles two matrices and the
        result equals quantising every matrix alone (parity: the reference's "matrix a stacked weight is
        quantized as", ``custom_placements/blockwise_quant_bucketed_block_shard.py:101``)."""
        return rows * math.prod(shape[1:-1]), shape[-1]

    # ---- format hooks
    def qdata_nbytes(self, rows: int, cols: int) -> int:
        raise NotImplementedError

    def scale_nbytes(self, rows: int, cols: int) -> int:
        raise NotImplementedError

    def quantize_into(self, w: torch.Tensor, qdata_bytes: torch.Tensor, scale_bytes: torch.Tensor) -> None:
        raise NotImplementedError

    def make_weight(self, qdata_bytes: torch.Tensor, scale_bytes: torch.Tensor, shape, dtype, requires_grad=True):
        raise NotImplementedError

    # ---- payload geometry
    def _payload_layout(self, infos, W):
        """Per rank: [(param index, rows, q_off, q_bytes, s_off, s_bytes)], and the padded row size."""
        per_rank, sizes = [], []
        for r in range(W):
            items, off = [], 0
            for i, info in enumerate(infos):
                a, b = info.placement.row_ranges[r]
                if b - a <= 0:
                    continue
                rows, cols = self.matrix_dims(info.global_shape, b - a)
                qb = info.placement.qdata_nbytes(rows, cols)
                items.append([i, rows, off, qb, 0, 0])
                off = (off + qb + 15) // 16 * 16
            for it in items:
                info = infos[it[0]]
                sb = info.placement.scale_nbytes(it[1], info.global_shape[-1])
                it[4], it[5] = off, sb
                off = (off + sb + 15) // 16 * 16
            per_rank.append([tuple(it) for it in items])
            sizes.append(off)
        return per_rank, max(sizes) if sizes else 0

    def unsharded_buffer_numel(self, info, world_size):
        rows, cols = self.matrix_dims(info.global_shape, info.global_shape[0])
        nbytes = (self.qdata_nbytes(rows, cols) + 15) // 16 * 16 + (self.scale_nbytes(rows, cols) + 15) // 16 * 16
        return -(-nbytes // info.param_dtype.itemsize)

    # ---- gather: quantise locally, gather bytes, compact
    def prepare_unshard_bucket(self, infos, byte_storage, comm, persistent):
        W, rank = comm.world_size, comm.rank
        per_rank, row_bytes = self._payload_layout(infos, W)
        prep = PlacementPreparedUnshard(infos=infos, persistent=persistent)
        prep.extra.update(per_rank=per_rank, row_bytes=row_bytes)
        cache = getattr(self, "_payload_cache", None)
        key = (byte_storage.data_ptr(), byte_storage._version, row_bytes)
        in_backward = torch._C._current_graph_task_id() != -1
        if not in_backward:
            self._payload_cache = None  # a forward always re-quantises
            cache = None
        if cache is not None and cache[0] == key:
            # the backward re-gather (or a recompute inside backward) reuses the forward's payload once
            prep.recv = cache[1]
            prep.extra["cached"] = True
            self._payload_cache = None
            return prep
        recv = torch.empty(W, row_bytes, dtype=torch.uint8, device=byte_storage.device)
        # quantise-on-push: on a peer-memory mesh the quantiser writes this rank's payload row straight into
        # symmetric memory, where the peers' gather reads it in place (no staging copy of the FP8 bytes)
        push_row = self._push_row(comm, row_bytes) if W > 1 else None
        with record("FlexShard::copy_in"):
            row = push_row if push_row is not None else recv[rank]
            for i, rows, qo, qb, so, sb in per_rank[rank]:
                info = infos[i]
                cols = info.global_shape[-1]
                w = info.placement.make_local_storage_view(info, byte_storage).reshape(rows, cols)
                if w.dtype != info.param_dtype:
                    w = w.to(info.param_dtype)  # quantise from the compute dtype, as the dense path would
                info.placement.quantize_into(w, row[qo:qo + qb], row[so:so + sb])
        prep.recv = recv
        prep.send = push_row if push_row is not None else recv[rank]
        prep.extra["key"] = key
        return prep

    def _push_row(self, comm, row_bytes):
        """This placement object's payload row inside a symmetric region (one per bucket: all parameters of a
        bucket share the first parameter's placement for the bucket-level calls), or None on other meshes.
        The row is rewritten by every gather, so the previous gather's readers must be done first."""
        alloc = getattr(comm, "alloc_storage", None)
        if alloc is None or not getattr(comm, "resident_storage", False):
            return None
        row = getattr(self, "_symm_row", None)
        if row is None or row.numel() != row_bytes:
            row = self._symm_row = alloc(row_bytes)
            if row is None:
                return None
        comm.wait_readers_done(row)
        return row

    def run_prepared_unshard(self, prepared, comm, async_op=False):
        if comm.world_size == 1 or prepared.extra.get("cached"):
            return
        with record("FlexShard::all_gather"):
            prepared.work = comm.all_gather_into_tensor(prepared.recv.view(-1), prepared.send, async_op=async_op)

    def finish_prepared_unshard(self, prepared, comm, persistent):
        if prepared.work is not None:
            prepared.work.wait()
            prepared.work = None
        infos, W = prepared.infos, comm.world_size
        recv = prepared.recv
        outs = []
        copies = []
        with record("FlexShard::copy_out"):
            for i, (info, buf) in enumerate(zip(infos, persistent)):
                pl = info.placement
                rows_total, cols = self.matrix_dims(info.global_shape, info.global_shape[0])
                raw = buf.view(torch.uint8)
                q_total = pl.qdata_nbytes(rows_total, cols)
                s_start = (q_total + 15) // 16 * 16
                s_total = pl.scale_nbytes(rows_total, cols)
                qdst, sdst = raw[:q_total], raw[s_start:s_start + s_total]
                for r in range(W):
                    a, b = pl.row_ranges[r]
                    if b <= a:
                        continue
                    item = next(it for it in prepared.extra["per_rank"][r] if it[0] == i)
                    _, rows, qo, qb, so, sb = item
                    first = self.matrix_dims(info.global_shape, a)[0]
                    q_at = pl.qdata_nbytes(first, cols)
                    s_at = pl.scale_nbytes(first, cols)  # whole blocks precede the first row
                    copies.append((qdst[q_at:q_at + qb], recv[r, qo:qo + qb]))
                    copies.append((sdst[s_at:s_at + sb], recv[r, so:so + sb]))
                outs.append((pl, qdst, sdst, info))
            # compaction: every rank's payload and scale bytes of every weight land in the persistent
            # compact buffer with one segment-copy launch; the weight wrappers (which may derive further
            # scale tensors from the gathered bytes) are built afterwards
            run_segment_ops(copies)
            outs = [pl.make_weight(q, sc, info.global_shape, info.param_dtype, info.requires_grad)
                    for pl, q, sc, info in outs]
        if not prepared.extra.get("cached") and "key" in prepared.extra:
            self._payload_cache = (prepared.extra["key"], recv)
        return PlacementUnshardResult(outs, keepalive=[])


    def prepare_reduce_grad(self, infos, grads, comm, reduce_dtype):
        self._payload_cache = None  # the master rows are about to change
        return super().prepare_reduce_grad(infos, grads, comm, reduce_dtype)


class Fp8BucketedBlockShard(BlockwiseQuantBucketedBlockShard):
    block_size = 128

    def qdata_nbytes(self, rows, cols):
        return rows * cols

    def scale_nbytes(self, rows, cols):
        return -(-rows // 128) * -(-cols // 128) * 4

    def quantize_into(self, w, qdata_bytes, scale_bytes):
        from ..ops.fp8 import FP8, quantize_blockwise

        rows, cols = w.shape
        q = qdata_bytes.view(FP8).view(rows, cols)
        s = scale_bytes.view(torch.float32).view(-(-rows // 128), -(-cols // 128))
        quantize_blockwise(w.contiguous(), out_q=q, out_scale=s)

    def make_weight(self, qdata_bytes, scale_bytes, shape, dtype, requires_grad=True):
        from ..ops.fp8 import FP8
        from ..quant.weight import BlockwiseFp8Weight

        rows, cols = math.prod(shape[:-1]), shape[-1]
        q = qdata_bytes.view(FP8).view(rows, cols)
        scale = scale_bytes.view(torch.float32).view(-(-rows // 128), -(-cols // 128))
        if self.weight_factory is not None:
            # the consumer's own tensor: data in the parameter's shape, one reciprocal scale per 128x128 block of
            # the [prod(shape[:-1]), shape[-1]] matrix; it must view (not copy) both, which are refilled in place
            return self.weight_factory(q.view(tuple(shape)), scale, self.block_size, orig_dtype=dtype,
                                       requires_grad=requires_grad)
        return BlockwiseFp8Weight(q, scale, shape, dtype)


class Mxfp8BucketedBlockShard(BlockwiseQuantBucketedBlockShard):
    """MXFP8 payload: every rank owns whole 128-row units, quantises them to e4m3 with 32x32 tile
    scales and sends the data plus one exponent byte per tile; after the gather each rank expands
    the tile exponents into the two blocked scale tensors the tensor core reads (forward and
    input-gradient orientation), so no swizzled scale bytes cross the wire.
    Parity: ``custom_placements/mxfp8_bucketed_block_shard.py:202-350`` of the reference (which gathers
    both pre-swizzled scale tensors)."""

    block_size = 32

    def __init__(self, row_ranges, scaling_mode: str = "rceil", weight_factory: Callable | None = None):
        if scaling_mode != "rceil":
            raise ValueError(f"unsupported MXFP8 scaling mode {scaling_mode!r} (only 'rceil': round the scale up)")
        super().__init__(row_ranges, weight_factory)
        self.scaling_mode = scaling_mode

    def qdata_nbytes(self, rows, cols):
        return rows * cols

    def scale_nbytes(self, rows, cols):
        return -(-rows // 32) * -(-cols // 32)

    def quantize_into(self, w, qdata_bytes, scale_bytes):
        from ..ops.mxfp8 import FP8, mx_quantize_weight

        rows, cols = w.shape
        mx_quantize_weight(w.contiguous(), out_q=qdata_bytes.view(FP8).view(rows, cols),
                           out_e=scale_bytes.view(-(-rows // 32), -(-cols // 32)))

    def make_weight(self, qdata_bytes, scale_bytes, shape, dtype, requires_grad=True):
        from ..ops.mxfp8 import FP8
        from ..quant.weight import BlockwiseMxfp8Weight

        rows, cols = math.prod(shape[:-1]), shape[-1]
        w = BlockwiseMxfp8Weight.from_tile_exponents(qdata_bytes.view(FP8).view(rows, cols),
                                                     scale_bytes.view(-(-rows // 32), -(-cols // 32)), shape, dtype)
        if self.weight_factory is not None:
            # the consumer's own tensor from the data (parameter's shape) and the two blocked scale tensors
            return self.weight_factory(w.qdata.view(tuple(shape)), w.fwd_scale, w.dgrad_scale, orig_dtype=dtype,
                                       requires_grad=requires_grad)
        return w


def plan_row_ranges(shapes: Sequence[tuple[int, ...]], world_size: int, block_rows: int,
                    cost_of: Callable[[int, int], int]) -> list[list[tuple[int, int]]]:
    """Row range of every parameter on every rank: ``result[param][rank] = (r0, r1)``."""
    units = []  # (param, r0, r1, cost)
    for i, s in enumerate(shapes):
        # 2-D weights are cut on whole blocks of rows; a stacked weight [*stack, out, in] on whole entries of
        # its leading dimension (each one or more matrices of `out` rows)
        step = block_rows if len(s) <= 2 else 1
        for r0 in range(0, s[0], step):
            r1 = min(s[0], r0 + step)
            units.append((i, r0, r1, cost_of(*BlockwiseQuantBucketedBlockShard.matrix_dims(s, r1 - r0))))
    cuts = partition_min_max([u[3] for u in units], world_size)
    out = [[(0, 0)] * world_size for _ in shapes]
    for r in range(world_size):
        mine = units[cuts[r]:cuts[r + 1]]
        for i in sorted({u[0] for u in mine}):
            rows = [u for u in mine if u[0] == i]
            out[i][r] = (rows[0][1], rows[-1][2])
    for i, s in enumerate(shapes):  # ranks without rows still carry a valid empty range
        pos = 0
        for r in range(world_size):
            a, b = out[i][r]
            if b <= a:
                out[i][r] = (pos, pos)
            else:
                pos = b
    return out


def _check_quantisable(fqn: str, p, block_rows: int, who: str) -> None:
    if p.dim() < 2:
        raise ValueError(f"{who} only supports 2-D or stacked 2-D weights, {fqn!r} has shape {tuple(p.shape)}")
    if p.dim() > 2 and math.prod(p.shape[1:-1]) % block_rows:
        raise ValueError(f"{who}: the matrices of the stacked weight {fqn!r} {tuple(p.shape)} must have a multiple "
                         f"of {block_rows} rows, so that no quantisation block straddles two of them")


class BlockwiseFp8WeightFactory(Protocol):
    """``weight_factory`` of the FP8 placement: builds the consumer's tensor from the gathered operands, which it
    must view rather than copy.  Parity: ``custom_placements/fp8_bucketed_block_shard.py:43-65`` of the reference."""

    def __call__(self, fp8_data: torch.Tensor, recip_scale: torch.Tensor, block_size: int, *,
                 orig_dtype: torch.dtype, requires_grad: bool) -> torch.Tensor: ...


class BlockwiseMxfp8WeightFactory(Protocol):
    """``weight_factory`` of the MXFP8 placement (data, forward-orientation and input-gradient-orientation blocked
    scales).  Parity: ``custom_placements/mxfp8_bucketed_block_shard.py:68-90`` of the reference."""

    def __call__(self, fp8_data: torch.Tensor, fwd_scale: torch.Tensor, dgrad_scale: torch.Tensor, *,
                 orig_dtype: torch.dtype, requires_grad: bool) -> torch.Tensor: ...


def make_fp8_bucketed_block_shard_placement_fn(block_size: int = 128, *, weight_factory=None,
                                               fp8_dtype: torch.dtype = torch.float8_e4m3fn):
    """Placement function for FP8 buckets: 2-D weights ``[out, in]`` or stacked weights ``[*stack, out, in]``
    whose ``out`` is a multiple of the block size.  ``weight_factory``: see ``BlockwiseFp8WeightFactory``."""
    if block_size != 128:
        raise ValueError(f"the FP8 kernels quantise in 128x128 blocks, got block_size={block_size}")
    if fp8_dtype != torch.float8_e4m3fn:
        raise ValueError(f"the FP8 kernels use torch.float8_e4m3fn, got {fp8_dtype}")

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        shapes = [tuple(p.shape) for _, p in named_params]
        for (f, p) in named_params:
            _check_quantisable(f, p, block_size, "Fp8BucketedBlockShard")
        cost = lambda rows, cols: rows * cols + -(-rows // block_size) * -(-cols // block_size) * 4
        ranges = plan_row_ranges(shapes, W, block_size, cost)
        return {f: Fp8BucketedBlockShard(ranges[i], weight_factory) for i, (f, _) in enumerate(named_params)}

    return fn


def make_mxfp8_bucketed_block_shard_placement_fn(scaling_mode: str = "rceil", *, weight_factory=None):
    """Placement function for MXFP8 buckets: 2-D weights (rows handed out in whole 128-row units) or stacked
    weights ``[*stack, out, in]`` with ``out`` a multiple of 128 (handed out matrix by matrix).
    ``weight_factory``: see ``BlockwiseMxfp8WeightFactory``."""

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        shapes = [tuple(p.shape) for _, p in named_params]
        for (f, p) in named_params:
            _check_quantisable(f, p, 128, "Mxfp8BucketedBlockShard")
        cost = lambda rows, cols: rows * cols + -(-rows // 32) * -(-cols // 32)
        ranges = plan_row_ranges(shapes, W, 128, cost)
        return {f: Mxfp8BucketedBlockShard(ranges[i], scaling_mode, weight_factory)
                for i, (f, _) in enumerate(named_params)}

    return fn
