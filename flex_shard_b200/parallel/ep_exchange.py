"""Expert-parallel token exchange over NVLink peer memory with no host in the loop.

``SymmExpertExchange`` moves token rows between a rank's *sender layout* (its (token, choice) pairs in
expert-major order, blocks padded to 128 rows, as ``plan_routes`` lays them out) and the *receiver layout* of the
rank that owns the experts (rows of its local experts from every rank, expert-major, padded: what the grouped
GEMM reads).  Counts never reach the CPU: each rank publishes its per-expert counts and block offsets in a
symmetric table, the receiver derives the landing row of every (source rank, local expert) run on the device,
publishes that table for the way back, and rows are pulled out of the peers' memory by a kernel whose grid is
sized for the worst case.  The receive buffer holds ``capacity_factor x T x k`` rows; a step that routes more
rows than that to one rank sets the device status word (``ops.check_status()`` raises) instead of overrunning.

Two autograd functions wrap the two directions; each is the other's backward, with the tables of the forward
pass kept on the device for the backward pass.

Parity: the role of the reference's all-to-all dispatcher (``examples/deepseek_v3/expert_parallel.py:30-128``:
counts exchange, host read of the split sizes, two ``all_to_all_single`` and a permute); here the permute is
folded into the pull and nothing synchronises with the host.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe as moe_ops
from ..ops._lib import count_launch
from .symm import SymmRegion

_declared = False


def _ensure():
    global _declared
    if _declared:
        return
    c = ctypes
    vp, i32, i64, u32 = c.c_void_p, c.c_int, c.c_longlong, c.c_uint
    _lib.declare("fsb_ep_receiver_setup", [vp, i32, i32, i32, i32, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, vp, vp])
    _lib.declare("fsb_ep_sender_setup", [vp, i32, i32, i32, i32, i64, vp, vp, vp, vp, u32, u32, vp, vp])
    _lib.declare("fsb_ep_pull_rows", [vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, vp, u32, u32, vp, vp])
    _declared = True


class _Tables:
    """Device tables of one direction of one layer: runs (n, srow, drow) and, on the receiver, padding and plan."""

    def __init__(self, pairs, le, cap_rows, dev, receiver):
        i32 = dict(dtype=torch.int32, device=dev)
        self.n, self.srow, self.drow = (torch.zeros(pairs, **i32) for _ in range(3))
        if receiver:
            self.pad_lo, self.pad_hi = torch.zeros(le, **i32), torch.zeros(le, **i32)
            self.offs = torch.zeros(le + 1, **i32)
            self.tile_expert = torch.zeros(cap_rows // 128, **i32)
            self.num_mtiles = torch.zeros(1, **i32)


class SymmExpertExchange:
    SLOT_TABLES, SLOT_RECV_BASE, SLOT_A_READY, SLOT_B_READY, SLOT_A_DONE, SLOT_B_DONE = 8, 9, 10, 11, 12, 13

    def __init__(self, group, num_experts: int, row_elems: int, max_pairs: int, device: torch.device,
                 capacity_factor: float = 2.0, dtype: torch.dtype = torch.bfloat16):
        _ensure()
        self.group, self.device, self.dtype = group, device, dtype
        self.ep, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.le, self.D = num_experts, num_experts // self.ep, row_elems
        self.row_bytes = row_elems * dtype.itemsize
        if self.row_bytes % 16:
            raise ValueError("token rows must be a multiple of 16 bytes")
        self.send_rows = moe_ops.max_rows_for(max_pairs, num_experts)
        cap = int(max_pairs * capacity_factor) + self.le * 127
        self.cap_rows = (cap + 127) // 128 * 128
        self.table_bytes = (4 * (3 * num_experts + 1) + 255) // 256 * 256
        self.a_off = self.table_bytes                                   # sender-layout rows
        self.b_off = self.a_off + (self.send_rows * self.row_bytes + 255) // 256 * 256   # receiver-layout rows
        total = self.b_off + self.cap_rows * self.row_bytes
        self.region = SymmRegion(group, total, device)
        self.region.name = ("expert exchange region (slots: 8 tables, 9 landing rows, 10/11 area A/B ready, "
                            "12/13 area A/B done)")
        self.epochs = {k: 0 for k in ("tables", "recv_base", "a", "b")}
        self.exchanges = 0

    # ---- addresses
    def _peer(self, off):
        return (ctypes.c_ulonglong * self.ep)(*[self.region.peer_payload_addr(r, off) for r in range(self.ep)])

    def _local(self, off, nbytes):
        return self.region.payload[off:off + nbytes]

    def _flags(self, slot):
        return self.region.flag_row_addr(self.rank, slot)

    def _status(self):
        return _lib.status_word(self.device).data_ptr()

    # ---- forward of "to experts": publish tables + rows, build receiver tables, pull
    def publish_tables(self, plan) -> None:
        """Write this rank's counts and block offsets into its symmetric table (the rows follow in area A).
        The peers read a rank's tables while they set up their pulls of the previous exchange, so the tables
        may only change once every peer has finished those pulls in both directions."""
        for area, done in (("a", self.SLOT_A_DONE), ("b", self.SLOT_B_DONE)):
            if self.epochs[area] > 0:
                self.region.wait(done, self.epochs[area])
        tb = self._local(0, 4 * (2 * self.E + 1)).view(torch.int32)
        tb[: self.E].copy_(plan.counts)
        tb[self.E:2 * self.E + 1].copy_(plan.offs)

    def stage(self, area: str, rows: torch.Tensor) -> None:
        """Copy ``rows`` into area A (sender layout) or B (receiver layout) once every peer is done with its
        previous content, then announce it."""
        reg = self.region
        done = self.SLOT_A_DONE if area == "a" else self.SLOT_B_DONE
        ready = self.SLOT_A_READY if area == "a" else self.SLOT_B_READY
        e = self.epochs[area]
        if e > 0:
            reg.wait(done, e)
        off = self.a_off if area == "a" else self.b_off
        n = rows.shape[0] * self.row_bytes
        self._local(off, n).copy_(rows.contiguous().view(torch.uint8).view(-1))
        self.epochs[area] = e + 1
        reg.signal(ready, e + 1)

    def receiver_setup(self) -> _Tables:
        t = _Tables(self.ep * self.le, self.le, self.cap_rows, self.device, receiver=True)
        self.epochs["tables"] += 1
        e = self.epochs["tables"]
        self.region.signal(self.SLOT_TABLES, e)
        rc = _lib.load().fsb_ep_receiver_setup(
            self._peer(0), self.E, self.le, self.ep, self.rank, self.cap_rows, t.n.data_ptr(), t.srow.data_ptr(),
            t.drow.data_ptr(), t.pad_lo.data_ptr(), t.pad_hi.data_ptr(), t.offs.data_ptr(), t.tile_expert.data_ptr(),
            t.num_mtiles.data_ptr(), self._flags(self.SLOT_TABLES), e, self.region.max_polls, self._status(),
            _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_ep_receiver_setup")
        count_launch()
        self.epochs["recv_base"] += 1
        self.region.signal(self.SLOT_RECV_BASE, self.epochs["recv_base"])
        return t

    def sender_setup(self) -> _Tables:
        t = _Tables(self.ep * self.le, self.le, self.cap_rows, self.device, receiver=False)
        rc = _lib.load().fsb_ep_sender_setup(
            self._peer(0), self.E, self.le, self.ep, self.rank, self.cap_rows, t.n.data_ptr(), t.srow.data_ptr(),
            t.drow.data_ptr(), self._flags(self.SLOT_RECV_BASE), self.epochs["recv_base"], self.region.max_polls, self._status(),
            _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_ep_sender_setup")
        count_launch()
        return t

    def pull(self, area: str, t: _Tables, out_rows: int, clear_padding: bool) -> torch.Tensor:
        """Pull the runs of ``t`` out of the peers' area into a fresh ``[out_rows, D]`` tensor."""
        out = torch.empty(out_rows, self.D, dtype=self.dtype, device=self.device)
        off = self.a_off if area == "a" else self.b_off
        ready = self.SLOT_A_READY if area == "a" else self.SLOT_B_READY
        done = self.SLOT_A_DONE if area == "a" else self.SLOT_B_DONE
        pad = clear_padding and hasattr(t, "pad_lo")
        rc = _lib.load().fsb_ep_pull_rows(
            self._peer(off), t.n.data_ptr(), t.srow.data_ptr(), t.drow.data_ptr(),
            t.pad_lo.data_ptr() if pad else None, t.pad_hi.data_ptr() if pad else None, out.data_ptr(), self.row_bytes,
            self.ep, self.le, 16, self._flags(ready), self.epochs[area], self.region.max_polls, self._status(),
            _lib.stream_ptr(self.device))
        _lib.check(rc, "fsb_ep_pull_rows")
        count_launch()
        self.region.signal(done, self.epochs[area])
        self.exchanges += 1
        return out


class _ToExperts(torch.autograd.Function):
    """Sender-layout rows -> receiver-layout rows of the experts' owners (backward: the way back)."""

    @staticmethod
    def forward(ctx, rows, ex: SymmExpertExchange, recv_tables, holder):
        ex.stage("a", rows)
        out = ex.pull("a", recv_tables, ex.cap_rows, clear_padding=True)
        ctx.ex, ctx.holder, ctx.n_rows = ex, holder, rows.shape[0]
        return out

    @staticmethod
    def backward(ctx, d_out):
        ex = ctx.ex
        ex.stage("b", d_out)
        back = ex.pull("b", ctx.holder["send_tables"], ctx.n_rows, clear_padding=False)
        return back, None, None, None


class _FromExperts(torch.autograd.Function):
    """Receiver-layout rows (expert outputs) -> sender-layout rows (backward: to the experts again)."""

    @staticmethod
    def forward(ctx, rows, ex: SymmExpertExchange, send_tables, recv_tables, n_send_rows):
        ex.stage("b", rows)
        out = ex.pull("b", send_tables, n_send_rows, clear_padding=False)
        ctx.ex, ctx.recv_tables = ex, recv_tables
        return out

    @staticmethod
    def backward(ctx, d_out):
        ex = ctx.ex
        ex.stage("a", d_out)
        d_rows = ex.pull("a", ctx.recv_tables, ex.cap_rows, clear_padding=True)
        return d_rows, None, None, None, None


class SymmDispatcher:
    """Drop-in for ``AllToAllDispatcher`` on peer-memory meshes: same result, no host synchronisation."""

    def __init__(self, group, num_experts: int, capacity_factor: float = 2.0):
        self.group, self.num_experts, self.capacity_factor = group, num_experts, capacity_factor
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local_experts = num_experts // self.ep
        self._ex: SymmExpertExchange | None = None
        self._symm = None          # attribute the NCCL/peer-pull dispatcher also has (tests look at it)

    # One exchange (symmetric staging areas + tables) serves every MoE layer of a model: layers run one after the
    # other in the same order on every rank, each use waits for the peers' "done" flags of the previous use, and
    # the per-layer tables that the backward pass needs are kept outside the region. 26 layers of the 16B example
    # would otherwise hold 26 x 0.6 GB of staging memory per rank.
    _shared: dict = {}

    def exchange_for(self, xt, k) -> SymmExpertExchange:
        pairs = xt.shape[0] * k
        # the group object itself is part of the key (and so stays alive): an id() could be reused by a later group
        key = (self.group, self.num_experts, xt.shape[1], pairs, xt.dtype, self.capacity_factor, xt.device)
        ex = self._ex
        # a batch of another size (an evaluation batch, say) takes the exchange built for that size; every rank of the
        # group must see the same sizes in the same order, since building an exchange is a collective step
        if ex is None or ex.D != xt.shape[1] or ex.dtype != xt.dtype or moe_ops.max_rows_for(pairs, self.num_experts) != ex.send_rows:
            ex = SymmDispatcher._shared.get(key)
            if ex is None:
                ex = SymmDispatcher._shared[key] = SymmExpertExchange(
                    self.group, self.num_experts, xt.shape[1], pairs, xt.device, self.capacity_factor, xt.dtype)
            self._ex = ex
        return ex

    def __call__(self, xt, idx, weights, experts):
        T, k = idx.shape
        ex = self.exchange_for(xt, k)
        plan = moe_ops.plan_routes(idx, self.num_experts)        # one launch; counts and offsets stay on the device
        if plan.max_rows != ex.send_rows:
            raise RuntimeError("token count changed between steps beyond the exchange's buffers")
        ex.publish_tables(plan)
        send_rows = moe_ops.moe_dispatch(xt, plan)               # sender layout [send_rows, D]
        recv_t = ex.receiver_setup()
        holder = {}
        recv_rows = _ToExperts.apply(send_rows, ex, recv_t, holder)
        recv_plan = moe_ops.RoutePlan(pos=None, src=None, offs=recv_t.offs, tile_expert=recv_t.tile_expert,
                                      num_mtiles=recv_t.num_mtiles, max_rows=ex.cap_rows,
                                      num_experts=self.local_experts)
        y_rows = experts(recv_rows, recv_plan)
        send_t = ex.sender_setup()
        holder["send_tables"] = send_t
        back = _FromExperts.apply(y_rows, ex, send_t, recv_t, plan.max_rows)
        return moe_ops.moe_combine(back, weights, plan)
