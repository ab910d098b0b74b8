"""Expert parallelism: each rank of the EP group keeps ``E / ep`` experts; token rows travel to the
owning rank and back with all-to-alls.

``apply_expert_parallel(model, ep_group)`` slices every MoE layer's stacked expert weights down to
the local experts, declares where they sit in the full weights (``set_global_layout``, so
``init_from_full`` and checkpoints still see full tensors) and installs an ``AllToAllDispatcher``.

The dispatcher sorts (token, choice) pairs by destination expert, exchanges per-(rank, expert)
counts, moves the rows each way (with the peer-memory backend: every rank pulls its rows out of the
senders' memory over NVLink with one kernel; otherwise one uneven NCCL all-to-all), and runs the
local experts through the grouped tcgen05 GEMMs on an expert-major layout planned on the device.
The only host synchronisation is the read of the row-count table, which sizes the receive buffers (as in the reference's dispatcher, ``examples/deepseek_v3/expert_parallel.py:59-165``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import moe as moe_ops
from ..placement_contract import GlobalLayout, set_global_layout


def _exchange_rows(out, x, out_splits, in_splits, table, group, symm):
    """Rows of ``x`` grouped by destination rank -> rows grouped by source rank. ``table[src][dst]`` is
    the full row-count table; with a peer-memory communicator every rank pulls its rows out of the
    senders' memory over NVLink with one kernel, otherwise NCCL's all-to-all moves them."""
    x = x.contiguous()
    if symm is not None and x.is_cuda:
        row_bytes = x[0].numel() * x.element_size() if x.dim() > 1 else x.element_size()
        if symm.all_to_all_pull(out, x, [[n * row_bytes for n in row] for row in table]):
            symm.p2p_row_exchanges = getattr(symm, "p2p_row_exchanges", 0) + 1
            return
    dist.all_to_all_single(out, x, out_splits, in_splits, group=group)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, table, group, symm):
        ctx.group, ctx.out_splits, ctx.in_splits, ctx.table, ctx.symm = group, out_splits, in_splits, table, symm
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        _exchange_rows(out, x, out_splits, in_splits, table, group, symm)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = dy.new_empty(sum(ctx.in_splits), *dy.shape[1:])
        back = [list(col) for col in zip(*ctx.table)]   # the way back: transposed table
        _exchange_rows(dx, dy, ctx.in_splits, ctx.out_splits, back, ctx.group, ctx.symm)
        return dx, None, None, None, None, None


class AllToAllDispatcher:
    def __init__(self, group: dist.ProcessGroup, num_experts: int):
        self.group = group
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts = num_experts
        self.local_experts = num_experts // self.ep
        self._symm = None

    def _symm_comm(self, device):
        """Peer-memory communicator of the EP group when that backend is selected (CUDA only)."""
        from . import comm as _comm

        if device.type != "cuda" or self.ep <= 1 or _comm._backend() != "symm":
            return None
        if self._symm is None:
            from .symm import SymmComm

            self._symm = SymmComm(self.group, self.rank, self.ep, device)
        return self._symm

    def __call__(self, xt, idx, weights, experts):
        T, k = idx.shape
        E, ep, le = self.num_experts, self.ep, self.local_experts
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)                     # expert-major == destination-rank-major
        counts = torch.bincount(flat, minlength=E).view(ep, le)      # [dst rank, local expert]
        all_counts = torch.empty(ep, ep, le, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts.view(-1), counts.reshape(-1), group=self.group)  # [src, dst, expert]
        recv_counts = all_counts[:, self.rank, :].contiguous()       # [src rank, local expert]
        table = all_counts.sum(-1).tolist()                           # the one host sync of this layer
        in_splits = table[self.rank]
        out_splits = [table[r][self.rank] for r in range(ep)]
        symm = self._symm_comm(xt.device)
        send_rows = xt[order // k]
        recv_rows = _AllToAll.apply(send_rows, out_splits, in_splits, table, self.group, symm)
        # rows arrive grouped by (src rank, local expert); name each row's local expert
        local_e = torch.repeat_interleave(
            torch.arange(le, device=xt.device).repeat(ep), recv_counts.reshape(-1),
            output_size=sum(out_splits))
        if local_e.numel() == 0:
            local_e = torch.zeros(0, dtype=torch.int64, device=xt.device)
        plan = moe_ops.plan_routes(local_e.view(-1, 1), le)
        rows = moe_ops.moe_dispatch(recv_rows, plan)
        y_rows = experts(rows, plan)
        ones = torch.ones(local_e.numel(), 1, dtype=torch.float32, device=xt.device)
        back = moe_ops.moe_combine(y_rows, ones, plan)               # undo the local expert-major order
        ret = _AllToAll.apply(back, in_splits, out_splits, [list(col) for col in zip(*table)], self.group, symm)
        # ret[i] is the expert output of pair order[i]; weight and sum the k choices of every token
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        gathered = ret[inv].view(T, k, -1)
        return (gathered.float() * weights[..., None]).sum(1).to(xt.dtype)


def make_dispatcher(ep_group, num_experts: int, device):
    """The host-free peer-memory dispatcher on CUDA meshes with the peer-memory backend selected (and
    ``FSB200_EP_DISPATCH`` not set to ``a2a``), else the all-to-all dispatcher."""
    import os

    from . import comm as _comm

    if (device.type == "cuda" and dist.get_world_size(ep_group) > 1 and _comm._backend() == "symm"
            and os.environ.get("FSB200_EP_DISPATCH", "symm") != "a2a"):
        from .ep_exchange import SymmDispatcher

        return SymmDispatcher(ep_group, num_experts)
    return AllToAllDispatcher(ep_group, num_experts)


def apply_expert_parallel(model, ep_group: dist.ProcessGroup) -> None:
    """Keep this rank's experts in every MoE layer and route tokens over ``ep_group``."""
    ep, rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
    for moe in model.moe_layers():
        E = moe.cfg.n_experts
        if E % ep:
            raise ValueError(f"expert-parallel degree {ep} must divide the {E} experts")
        le = E // ep
        for name in ("w13", "w2"):
            full = getattr(moe.routed_experts, name)
            local = torch.nn.Parameter(full.detach()[rank * le:(rank + 1) * le].clone()
                                       if full.device.type != "meta" else
                                       torch.empty(le, *full.shape[1:], dtype=full.dtype, device="meta"),
                                       requires_grad=full.requires_grad)
            shape = tuple(full.shape)
            nd = len(shape)
            set_global_layout(local, GlobalLayout(shape, ((rank * le,) + (0,) * (nd - 1),), ((0,) * nd,),
                                                  ((le, *shape[1:]),)))
            setattr(moe.routed_experts, name, local)
        moe.dispatcher = make_dispatcher(ep_group, E, full.device)
