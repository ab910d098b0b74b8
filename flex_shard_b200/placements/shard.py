"""``Shard(dim)``: equal chunks along one dim, the FSDP2-compatible placement.

Layout facts (parity: ``custom_placements/shard.py:118-244`` of the reference):
chunk = ceil(n/W); rank r holds ``[min(n, r*c), min(n, (r+1)*c))``; only dim 0 may be
uneven and then every rank reserves a rank-0-sized slot whose tail is zero, so the
bucket's byte buffer *is* the all-gather send buffer when no cast is needed. The
gathered ``[W, row]`` buffer is copied out into per-parameter padded buffers; gradients
are packed into ``[W, row]`` rows (cast to the reduce dtype on the way) and
reduce-scattered.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ..placement_contract import (
    GlobalLayout,
    GradientReduction,
    LocalStorageLayout,
    Placement,
    PlacementPreparedReduceGrad,
    PlacementPreparedUnshard,
    PlacementReduceGradResult,
    PlacementUnshardResult,
)
from ..parallel.comm import plan_reduction
from ..utils.profiling import record
from .sliced import _copy_or_loop


def _contig(shape):
    stride, acc = [], 1
    for s in reversed(shape):
        stride.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(stride))


class Shard(Placement):
    refills_persistent_buffers_in_finish = True
    uniform_storage = True   # every rank reserves rank-0-sized slots: the bucket's byte size is the same everywhere

    def __init__(self, dim: int = 0, grad_bucket: bool = False):
        self.dim = int(dim)
        # With grad_bucket=True the runtime allocates the reduce-scatter send buffer before the
        # bucket's backward and gives every unsharded parameter a ``main_grad`` view of its rows,
        # so weight-gradient kernels write the reduction layout directly (no pack/cast pass).
        self.grad_bucket = bool(grad_bucket)

    def __eq__(self, other):
        return isinstance(other, Shard) and other.dim == self.dim

    def __hash__(self):
        return hash(("Shard", self.dim))

    def __repr__(self):
        return f"Shard({self.dim})"

    def bucket_compatibility_key(self):
        return Shard  # one bucket may mix shard dims

    # ------------------------------------------------------------------ geometry
    def _chunk(self, n: int, W: int) -> int:
        return -(-n // W)

    def _range(self, n: int, r: int, W: int) -> tuple[int, int]:
        c = self._chunk(n, W)
        return min(n, r * c), min(n, (r + 1) * c)

    def _check(self, shape: Sequence[int], W: int) -> None:
        if self.dim >= len(shape) or self.dim < 0:
            raise ValueError(f"Shard({self.dim}) does not apply to a tensor of shape {tuple(shape)}")
        if self.dim > 0 and shape[self.dim] % W != 0:
            raise ValueError(
                f"Shard({self.dim}) needs dim {self.dim} (size {shape[self.dim]}) to divide evenly by the "
                f"mesh size {W}; only Shard(0) may be uneven.")

    def compute_local_shape(self, global_shape, rank, world_size):
        self._check(global_shape, world_size)
        lo, hi = self._range(global_shape[self.dim], rank, world_size)
        s = list(global_shape)
        s[self.dim] = hi - lo
        return tuple(s)

    def padded_shape(self, global_shape, world_size):
        s = list(global_shape)
        s[self.dim] = self._chunk(global_shape[self.dim], world_size)
        return tuple(s)

    def padded_numel(self, global_shape, world_size) -> int:
        return math.prod(self.padded_shape(global_shape, world_size))

    def extract_local_shard(self, full, rank, world_size):
        lo, hi = self._range(full.shape[self.dim], rank, world_size)
        return full.narrow(self.dim, lo, hi - lo)

    def local_storage_layout(self, global_shape, rank, world_size):
        ls = self.compute_local_shape(global_shape, rank, world_size)
        return LocalStorageLayout(ls, _contig(ls), self.padded_numel(global_shape, world_size))

    def global_layout(self, global_shape, rank, world_size):
        lo, hi = self._range(global_shape[self.dim], rank, world_size)
        gshape = tuple(global_shape)
        if hi <= lo:
            return GlobalLayout(gshape, (), (), ())
        goff = tuple(lo if d == self.dim else 0 for d in range(len(gshape)))
        size = tuple((hi - lo) if d == self.dim else gshape[d] for d in range(len(gshape)))
        return GlobalLayout(gshape, (goff,), (tuple(0 for _ in gshape),), (size,))

    def unsharded_buffer_numel(self, info, world_size):
        return self.padded_numel(info.global_shape, world_size) * world_size

    @staticmethod
    def unshard_aliases_storage(infos, world_size) -> bool:
        """On a one-rank mesh with no dtype change the "gathered" parameters are the stored shards
        themselves: the runtime then uses views of the byte storage and copies nothing."""
        return world_size == 1 and all(i.param_dtype == i.storage_dtype for i in infos)

    # ------------------------------------------------------------------ gather
    @staticmethod
    def _send_layout(infos, W):
        """Byte offsets of each parameter's padded slot in one rank's gather row."""
        offs, off = [], 0
        for info in infos:
            n = info.placement.padded_numel(info.global_shape, W) * info.param_dtype.itemsize
            offs.append((off, n))
            off += n
        return offs, off

    @staticmethod
    def gathers_into_persistent(infos, comm) -> bool:
        """With a peer-memory communicator each rank's chunk is pulled straight into its place in the
        per-parameter unsharded buffers: no gather buffer, no copy-out pass."""
        return (comm.world_size > 1 and hasattr(comm, "all_gather_segments")
                and all(i.placement.dim == 0 for i in infos))

    def _prepare_direct(self, infos, byte_storage, comm, persistent, offs, row_bytes, same):
        W = comm.world_size
        prep = PlacementPreparedUnshard(infos=infos, persistent=persistent)
        prep.extra.update(offs=offs, row_bytes=row_bytes, direct=True)
        with record("FlexShard::copy_in"):
            if same:
                send = byte_storage
            else:
                send = torch.zeros(row_bytes, dtype=torch.uint8, device=byte_storage.device)
                _copy_or_loop([(send[o:o + info.local_numel * info.param_dtype.itemsize].view(info.param_dtype),
                                info.placement.make_local_storage_view(info, byte_storage).reshape(-1))
                               for info, (o, n) in zip(infos, offs)])
        prep.send = send
        segs = []
        for info, (o, n), buf in zip(infos, offs, persistent):
            if n == 0:
                continue
            base = buf.data_ptr()
            for r in range(W):
                segs.append((r, o, base + r * n, n))
        prep.extra["segments"] = segs
        return prep

    def prepare_unshard_bucket(self, infos, byte_storage, comm, persistent):
        W = comm.world_size
        offs, row_bytes = self._send_layout(infos, W)
        if persistent and self.gathers_into_persistent(infos, comm):
            same = all(i.param_dtype == i.storage_dtype for i in infos) and all(
                i.byte_offset == o for i, (o, _) in zip(infos, offs)) and row_bytes == byte_storage.numel()
            return self._prepare_direct(infos, byte_storage, comm, persistent, offs, row_bytes, same)
        same = all(i.param_dtype == i.storage_dtype for i in infos) and all(
            i.byte_offset == o for i, (o, _) in zip(infos, offs)) and row_bytes == byte_storage.numel()
        prep = PlacementPreparedUnshard(infos=infos, persistent=persistent)
        prep.extra["offs"] = offs
        prep.extra["row_bytes"] = row_bytes
        if W == 1:
            prep.local_copy_out = True
            prep.extra["storage"] = byte_storage
            return prep
        with record("FlexShard::copy_in"):
            if same:
                prep.send = byte_storage  # zero-copy: the padded byte storage is the send buffer
                prep.recv = torch.empty(W * row_bytes, dtype=torch.uint8, device=byte_storage.device)
            else:
                prep.recv = torch.empty(W * row_bytes, dtype=torch.uint8, device=byte_storage.device)
                row = prep.recv[comm.rank * row_bytes:(comm.rank + 1) * row_bytes]
                row.zero_()
                _copy_or_loop([(row[o:o + info.local_numel * info.param_dtype.itemsize].view(info.param_dtype),
                                info.placement.make_local_storage_view(info, byte_storage).reshape(-1))
                               for info, (o, n) in zip(infos, offs)])
                prep.send = row  # in-place all-gather: the send row aliases the gather buffer
        return prep

    def run_prepared_unshard(self, prepared, comm, async_op=False):
        if comm.world_size == 1:
            return
        if prepared.extra.get("direct"):
            with record("FlexShard::all_gather"):
                comm.all_gather_segments(prepared.send, prepared.extra["segments"])
            return
        with record("FlexShard::all_gather"):
            prepared.work = comm.all_gather_into_tensor(prepared.recv, prepared.send, async_op=async_op)

    def finish_prepared_unshard(self, prepared, comm, persistent):
        W = comm.world_size
        infos = prepared.infos
        if prepared.work is not None:
            prepared.work.wait()
            prepared.work = None
        outs = []
        if prepared.extra.get("direct"):
            for info, buf in zip(infos, persistent):
                outs.append(buf[: info.global_numel].view(info.global_shape))
            return PlacementUnshardResult(outs, keepalive=[prepared.send])
        with record("FlexShard::copy_out"):
            if W == 1 and not persistent:
                storage = prepared.extra["storage"]
                outs = [info.placement.make_local_storage_view(info, storage) for info in infos]
                return PlacementUnshardResult(outs)
            copies = []
            if W == 1:
                storage = prepared.extra["storage"]
                for info, buf in zip(infos, persistent):
                    src = info.placement.make_local_storage_view(info, storage)
                    copies.append((buf[: info.global_numel].view(info.global_shape), src))
                    outs.append(buf[: info.global_numel].view(info.global_shape))
                _copy_or_loop(copies)
                return PlacementUnshardResult(outs)
            row_bytes = prepared.extra["row_bytes"]
            recv = prepared.recv.view(W, row_bytes)
            for info, (o, n), buf in zip(infos, prepared.extra["offs"], persistent):
                pl: Shard = info.placement
                padded = pl.padded_numel(info.global_shape, W)
                src = recv[:, o:o + n].view(info.param_dtype)  # [W, padded] (row-strided)
                if pl.dim == 0:
                    copies.append((buf.view(W, padded), src))
                    outs.append(buf[: info.global_numel].view(info.global_shape))
                else:
                    full = buf[: info.global_numel].view(info.global_shape)
                    ps = pl.padded_shape(info.global_shape, W)
                    c = ps[pl.dim]
                    for r in range(W):
                        copies.append((full.narrow(pl.dim, r * c, c), src[r].view(ps)))
                    outs.append(full)
            _copy_or_loop(copies)   # the whole bucket's copy-out (every rank's chunk of every parameter): one launch
        return PlacementUnshardResult(outs, keepalive=[prepared.recv])

    # ------------------------------------------------------------------ gradient reduction
    @staticmethod
    def _reduce_layout(infos, W):
        offs, off = [], 0
        for info in infos:
            n = info.placement.padded_numel(info.global_shape, W)
            offs.append((off, n))
            off += n
        return offs, off

    def wants_grad_bucket(self, infos) -> bool:
        return all(getattr(i.placement, "grad_bucket", False) for i in infos)

    def alloc_grad_bucket(self, storage, unsharded_params) -> None:
        """Allocate the ``[W, row]`` reduce-scatter send buffer now and hand each trainable
        dim-0 parameter a ``main_grad`` view of its rows (``[W, chunk, ...]`` strided, or the
        plain parameter shape on one rank)."""
        if getattr(storage, "_grad_bucket", None) is not None:
            return
        W = storage.comm.world_size
        pairs = [(i, u) for i, u in zip(storage.infos, unsharded_params) if i.requires_grad and u.requires_grad]
        infos = [i for i, _ in pairs]
        if not infos:
            return
        reduce_dtype = storage.bucket_reduce_dtype
        if reduce_dtype not in (torch.float32, torch.bfloat16):
            return
        offs, row = self._reduce_layout(infos, W)
        needs_zero = any(i.global_shape[i.placement.dim] % W != 0 for i in infos)
        comm = storage.reduce_comm
        if (W > 1 and getattr(comm, "fused_reduce", False) and reduce_dtype == torch.float32 and not needs_zero
                and all(i.placement.dim == 0 and i.partial_grad_group is None for i in infos) and row % 4 == 0):
            self._alloc_peer_bucket(storage, pairs, offs, row, comm)
            return
        buf = (torch.zeros if needs_zero else torch.empty)(W, row, dtype=reduce_dtype, device=storage.device)
        for (info, up), (o, n) in zip(pairs, offs):
            pl: Shard = info.placement
            if pl.dim != 0:
                continue
            if W == 1:
                view = buf[0, o:o + n].view(info.global_shape)
            else:
                ps = pl.padded_shape(info.global_shape, W)
                view = buf.as_strided((W, *ps), (row, *_contig(ps)), o)
            view._fsb_bucket = buf
            up.main_grad = view
            up.main_grad_written = False
        storage._grad_bucket = buf

    def _alloc_peer_bucket(self, storage, pairs, offs, row, comm) -> None:
        """Fused path: every 2-D+ parameter's ``main_grad`` is a ``PeerBlocked`` destination whose
        block i is rank i's incoming row for this rank, so the weight-gradient GEMM's epilogue is the
        all-to-all leg of the reduce-scatter. Vectors are scattered at reduce time."""
        from ..ops.gemm import PeerBlocked
        from ..parallel.symm import PeerBucket

        W, me = comm.world_size, comm.rank
        ctx = storage.runtime.context
        biggest = 0
        for rt in ctx.runtimes:
            st = rt.storage
            if st.reduce_comm is comm:
                tr = [i for i in st.infos if i.requires_grad]
                if tr and all(isinstance(i.placement, Shard) for i in tr):
                    biggest = max(biggest, W * self._reduce_layout(tr, W)[1] * 4)
        if not any(len(i.global_shape) >= 2 for i, _ in pairs):
            return  # nothing a GEMM would write in place: use the ordinary reduction
        ring = comm.grad_ring(biggest)
        k, use = ring.acquire()
        bucket = PeerBucket(ring, k, use, row)
        for (info, up), (o, n) in zip(pairs, offs):
            if len(info.global_shape) < 2:
                continue
            cols = math.prod(info.global_shape[1:])
            c = info.global_shape[0] // W
            addrs = [ring.write_addr(me, i, k, row, o) for i in range(W)]
            view = PeerBlocked(addrs, c, info.global_shape[0], cols, torch.float32, storage.device,
                               local=ring.pull)
            view._fsb_bucket = bucket
            up.main_grad = view
            up.main_grad_written = False
        storage._grad_bucket = bucket

    def _prepare_peer_reduce(self, infos, grads, comm, bucket, offs):
        """Scatter the gradients that were not written in place (vectors, autograd-produced ones)."""
        W, me = comm.world_size, comm.rank
        ring, k, row = bucket.ring, bucket.k, bucket.row
        segs, keep = [], []
        for info, g, (o, n) in zip(infos, grads, offs):
            if getattr(g, "_fsb_bucket", None) is bucket:
                continue
            gf = g.reshape(-1).float().contiguous() if g.dtype != torch.float32 else g.reshape(-1).contiguous()
            keep.append(gf)
            for i in range(W):
                segs.append((gf.data_ptr() + i * n * 4, ring.write_addr(me, i, k, row, o), n * 4))
        comm.scatter_to_peers(segs)
        prep = PlacementPreparedReduceGrad(infos=infos, send=None, reduce_dtype=torch.float32)
        prep.extra.update(offs=offs, row=row, peer_bucket=bucket, keep=keep)
        return prep

    def prepare_reduce_grad(self, infos, grads, comm, reduce_dtype):
        W = comm.world_size
        offs, row = self._reduce_layout(infos, W)
        pb = None
        for g in grads:
            for attr in ("_fsb_bucket", "_fsb_peer_target"):
                cand = getattr(g, attr, None)
                if cand is not None and not isinstance(cand, torch.Tensor) and getattr(cand, "kind", None) == "peer":
                    pb = cand
                    break
            if pb is not None:
                break
        if pb is not None:
            return self._prepare_peer_reduce(infos, grads, comm, pb, offs)
        needs_zero = any(info.global_shape[info.placement.dim] % W != 0 for info in infos)
        bucket = next((getattr(g, "_fsb_bucket", None) for g in grads
                       if isinstance(getattr(g, "_fsb_bucket", None), torch.Tensor)), None)
        if bucket is not None and (bucket.dtype != reduce_dtype or tuple(bucket.shape) != (W, row)):
            bucket = None
        with record("FlexShard::reduce_scatter_copy_in"):
            if bucket is not None:
                send = bucket
            else:
                alloc = torch.zeros if needs_zero else torch.empty
                send = alloc(W, row, dtype=reduce_dtype, device=grads[0].device)
            copies = []
            for info, g, (o, n) in zip(infos, grads, offs):
                if bucket is not None and getattr(g, "_fsb_bucket", None) is bucket:
                    continue  # already written in place by the weight-gradient kernel
                if getattr(g, "_fsb_bucket", None) is not None:
                    g = self._dense_from_main(info, g, W)
                pl: Shard = info.placement
                dst = send[:, o:o + n]
                if pl.dim == 0:
                    flat = g.reshape(-1)
                    full_ranks = flat.numel() // n if n > 0 else 0
                    full_ranks = min(full_ranks, W)
                    if full_ranks:
                        copies.append((dst[:full_ranks], flat[: full_ranks * n].view(full_ranks, n)))
                    rem = flat.numel() - full_ranks * n
                    if rem > 0:
                        copies.append((dst[full_ranks, :rem], flat[full_ranks * n:]))
                else:
                    ps = pl.padded_shape(info.global_shape, W)
                    c = ps[pl.dim]
                    for r in range(W):
                        copies.append((dst[r].view(ps), g.narrow(pl.dim, r * c, c)))
            _copy_or_loop(copies)   # pack (and cast to the reduce dtype) every gradient of the bucket in one launch
        prep = PlacementPreparedReduceGrad(infos=infos, send=send, reduce_dtype=reduce_dtype)
        prep.extra["offs"] = offs
        prep.extra["row"] = row
        return prep

    @staticmethod
    def _dense_from_main(info, g, W):
        """A ``main_grad`` view of a foreign bucket back in the parameter's own shape."""
        if g.dim() == len(info.global_shape):
            return g
        return g.reshape(-1, *g.shape[2:])[: info.global_shape[0]]

    def reduce_prepared_grad(self, prepared, comm, reduction: GradientReduction):
        W = comm.world_size
        plan = plan_reduction(reduction, W, prepared.reduce_dtype)
        row = prepared.extra["row"]
        pb = prepared.extra.get("peer_bucket")
        if pb is not None:
            scale = {"avg": 1.0 / W, "premul_sum": plan.premul or 1.0}.get(plan.op, 1.0)
            if plan.post_divide is not None:
                scale /= plan.post_divide
            adam = prepared.extra.get("adam")
            with record("FlexShard::fused_reduce_scatter"):
                out = None if adam is not None else torch.empty(row, dtype=torch.float32, device=comm.device)
                comm.reduce_incoming(pb, scale, out, adam)
            if out is None:
                return PlacementReduceGradResult(grads=[None] * len(prepared.infos), output=None)
            grads = [out[o:o + i.local_numel].view(i.local_shape) for i, (o, n) in zip(prepared.infos, prepared.extra["offs"])]
            return PlacementReduceGradResult(grads=grads, output=out)
        with record("FlexShard::reduce_scatter"):
            if W == 1:
                out = prepared.send.view(-1)
                if plan.post_divide is not None:
                    out.div_(plan.post_divide)
            else:
                out = torch.empty(row, dtype=prepared.reduce_dtype, device=prepared.send.device)
                comm.reduce_scatter_tensor(out, prepared.send.view(-1), plan)
        grads = []
        for info, (o, n) in zip(prepared.infos, prepared.extra["offs"]):
            ln = info.local_numel
            grads.append(out[o:o + ln].view(info.local_shape) if ln > 0 else out[o:o].view(info.local_shape))
        return PlacementReduceGradResult(grads=grads, output=out)


def shard_placement_fn(dim: int = 0, grad_bucket: bool = False):
    """``placement_fn`` that stores every parameter as ``Shard(dim)``."""

    def fn(named_params, mesh):
        return {fqn: Shard(dim, grad_bucket=grad_bucket) for fqn, _ in named_params}

    return fn
