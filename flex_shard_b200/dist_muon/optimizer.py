"""DistMuon: Muon over local shards, communication-free where storage equals compute layout.

Every managed parameter has a *local compute layout*:

* ``owned``       the local tensor is a whole matrix (or empty on non-owners): orthogonalise it;
* ``row_blocks``  the local tensor is a stack of whole dim-0 blocks (attention heads, experts):
                  orthogonalise each block;
* ``matrix_batch`` a 3-D local tensor ``[n, rows, cols]``: each slice is a matrix;
* ``row_shard``   ``Shard(0)`` storage: rows are exchanged with an owner rank (uneven
                  all-to-all), the owner runs Newton-Schulz, updates are sent back.

With ``BucketedOwned`` / ``BlockShard`` storage only the first three occur and ``step()`` issues no
collective at all. Math (parity ``dist_muon/optimizer.py:2031-2151`` of the reference)::

    M <- lerp(M, g, 1-mu);  u = lerp(g, M, mu) if nesterov else M
    X = NS_k(u_bf16 / max(|u|_F, eps));  p <- p (1 - lr wd) - lr ratio X

with ``ratio`` chosen by ``adjust_lr_fn``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Mapping, Sequence

import torch
import torch.distributed as dist

from ..ops.newton_schulz import NS_COEFFS, muon_apply_, muon_direction_
from ..placements.owned import newton_schulz_cost
from ..utils.validation import assign_to_hosts_then_ranks, mesh_rank_hosts


@dataclass(frozen=True)
class LocalMuonComputeLayout:
    kind: str                                  # owned | row_blocks | matrix_batch | row_shard
    block_rows: tuple[int, ...] | None = None  # row_blocks: rows of each local block
    global_shape: tuple[int, ...] | None = None
    row_range: tuple[int, int] | None = None   # row_shard: this rank's [start, end) rows


def lr_ratio(mode: str | None, rows: int, cols: int) -> float:
    if mode is None:
        return 1.0
    if mode == "original":
        return math.sqrt(max(1.0, rows / cols))
    if mode == "match_rms_adamw":
        return 0.2 * math.sqrt(max(rows, cols))
    if mode == "spectral_unclamped":
        return math.sqrt(rows / cols)
    raise ValueError(f"unknown adjust_lr_fn {mode!r}")


class DistMuon(torch.optim.Optimizer):
    def __init__(self, params, *, param_names: Sequence[str] | None = None, lr: float = 1e-3,
                 weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 ns_coefficients=NS_COEFFS, eps: float = 1e-7, ns_steps: int = 5,
                 adjust_lr_fn: str | None = None,
                 compute_layouts: Mapping[str, LocalMuonComputeLayout] | None = None,
                 group: dist.ProcessGroup | None = None, ranks_per_host: int | None = None,
                 owner_by_fqn: Mapping[str, int] | None = None):
        params = list(params)
        if param_names is None:
            param_names = [f"param_{i}" for i in range(len(params))]
        if len(param_names) != len(params):
            raise ValueError("param_names must name every parameter")
        lr_ratio(adjust_lr_fn, 1, 1)  # validates the mode
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_coefficients=tuple(ns_coefficients), eps=eps, ns_steps=ns_steps,
                        adjust_lr_fn=adjust_lr_fn)
        super().__init__(params, defaults)
        self.param_names = list(param_names)
        self._name_of = {id(p): n for p, n in zip(params, param_names)}
        self.compute_layouts = dict(compute_layouts or {})
        self.group = group
        self.collectives_issued = 0
        self.p2p_exchanges = 0
        self._owner_by_fqn = dict(owner_by_fqn or {})
        self._ranks_per_host = ranks_per_host
        self._row_shard_plan = None

    # ------------------------------------------------------------------ helpers
    def _layout(self, p) -> LocalMuonComputeLayout:
        name = self._name_of[id(p)]
        lay = self.compute_layouts.get(name)
        if lay is not None:
            return lay
        return LocalMuonComputeLayout("matrix_batch" if p.dim() == 3 else "owned")

    def _momentum(self, p) -> torch.Tensor:
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        return st["momentum_buffer"]

    def _preflight(self):
        """Host-side validation before any update (a missing gradient rejects the whole step)."""
        for group in self.param_groups:
            for p in group["params"]:
                if p.numel() > 0 and p.grad is None:
                    raise RuntimeError(f"DistMuon: parameter {self._name_of[id(p)]!r} has no gradient")
                if p.grad is not None and p.grad.shape != p.shape:
                    raise RuntimeError(f"DistMuon: gradient shape mismatch for {self._name_of[id(p)]!r}")

    def _matrix_step(self, p2d, g2d, m2d, group):
        if p2d.numel() == 0:
            return
        rows, cols = p2d.shape
        x = muon_direction_(m2d, g2d, group["momentum"], group["nesterov"], group["ns_steps"],
                            group["ns_coefficients"], group["eps"])
        muon_apply_(p2d, x, float(group["lr"]), group["weight_decay"], lr_ratio(group["adjust_lr_fn"], rows, cols))

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._preflight()
        for group in self.param_groups:
            row_shard = []
            for p in group["params"]:
                lay = self._layout(p)
                if lay.kind == "row_shard":
                    row_shard.append((p, lay))
                    continue
                if p.numel() == 0:
                    continue
                g, m = p.grad, self._momentum(p)
                if lay.kind == "owned":
                    if p.dim() == 2:
                        self._matrix_step(p.data, g, m, group)
                    else:
                        self._matrix_step(p.data.view(p.shape[0], -1), g.reshape(p.shape[0], -1),
                                          m.view(p.shape[0], -1), group)
                elif lay.kind == "matrix_batch":
                    for i in range(p.shape[0]):
                        self._matrix_step(p.data[i], g[i], m[i], group)
                elif lay.kind == "row_blocks":
                    pos = 0
                    p2, g2, m2 = (t.reshape(p.shape[0], -1) for t in (p.data, g, m))
                    for rows in (lay.block_rows or (p.shape[0],)):
                        self._matrix_step(p2[pos:pos + rows], g2[pos:pos + rows].contiguous()
                                          if not g2[pos:pos + rows].is_contiguous() else g2[pos:pos + rows],
                                          m2[pos:pos + rows], group)
                        pos += rows
                else:
                    raise ValueError(f"unknown compute layout kind {lay.kind!r}")
            if row_shard:
                self._row_shard_step(row_shard, group)
        return loss

    # ------------------------------------------------------------------ Shard(0)-stored matrices
    def _row_shard_step(self, items, group):
        """Redistribute rows to owners (one uneven all-to-all each way per call), compute there."""
        pg = self.group
        W = dist.get_world_size(pg) if dist.is_initialized() else 1
        rank = dist.get_rank(pg) if dist.is_initialized() else 0
        # momentum is applied on the storage layout first (it is elementwise), then u travels
        names = [self._name_of[id(p)] for p, _ in items]
        shapes = [lay.global_shape for _, lay in items]
        if self._row_shard_plan is None or self._row_shard_plan[0] != names:
            hosts = mesh_rank_hosts(W, self._ranks_per_host)
            loads = [0.0] * W
            fixed = {i: self._owner_by_fqn[n] for i, n in enumerate(names) if n in self._owner_by_fqn}
            for i, r in fixed.items():
                loads[r] += newton_schulz_cost(shapes[i], group["ns_steps"])
            free = [i for i in range(len(names)) if i not in fixed]
            owners_free = assign_to_hosts_then_ranks(
                [newton_schulz_cost(shapes[i], group["ns_steps"]) for i in free], hosts, loads)
            owners = [0] * len(names)
            for i, r in zip(free, owners_free):
                owners[i] = r
            for i, r in fixed.items():
                owners[i] = r
            self._row_shard_plan = (names, owners)
        owners = self._row_shard_plan[1]
        dev = items[0][0].device
        mu, nesterov = group["momentum"], group["nesterov"]
        # 1. momentum on local rows, Nesterov direction u (fp32) packed per destination owner
        send_chunks = [[] for _ in range(W)]
        for (p, lay), owner in zip(items, owners):
            if p.numel() == 0:
                continue
            m = self._momentum(p)
            gf = p.grad.float()
            m.lerp_(gf, 1 - mu)
            u = gf.lerp(m, mu) if nesterov else m
            send_chunks[owner].append(u.reshape(-1))
        send_sizes = [sum(c.numel() for c in ch) for ch in send_chunks]
        send = torch.cat([c for ch in send_chunks for c in ch]) if sum(send_sizes) else torch.empty(0, device=dev)
        # rows every rank holds of each matrix follow Shard(0) geometry
        def rows_of(shape, r):
            c = -(-shape[0] // W)
            return max(0, min(shape[0], (r + 1) * c) - min(shape[0], r * c))
        recv_sizes = [0] * W
        for shape, owner in zip(shapes, owners):
            if owner == rank:
                for r in range(W):
                    recv_sizes[r] += rows_of(shape, r) * math.prod(shape[1:])
        recv = torch.empty(sum(recv_sizes), dtype=torch.float32, device=dev)
        # sizes[r][o]: elements rank r sends to owner o (every rank can compute the whole table)
        sizes = [[0] * W for _ in range(W)]
        for shape, owner in zip(shapes, owners):
            cols = math.prod(shape[1:])
            for r in range(W):
                sizes[r][owner] += rows_of(shape, r) * cols
        if W > 1:
            self._exchange(recv, send, [sizes[r][rank] for r in range(W)],
                           [[sizes[r][o] for o in range(W)] for r in range(W)], pg, rank)
            self.collectives_issued += 1
        else:
            recv.copy_(send)
        # 2. owners assemble full matrices, orthogonalise, cut the update back into row pieces
        offs = [sum(recv_sizes[:r]) for r in range(W)]
        cursor = list(offs)
        back_chunks = [[] for _ in range(W)]
        for shape, owner in zip(shapes, owners):
            if owner != rank:
                continue
            cols = math.prod(shape[1:])
            parts = []
            for r in range(W):
                n = rows_of(shape, r) * cols
                parts.append(recv[cursor[r]:cursor[r] + n].view(-1, cols))
                cursor[r] += n
            full = torch.cat(parts, dim=0)
            zero_m = torch.zeros_like(full)
            # momentum already applied: run the iteration on u directly (mu=0 keeps u unchanged)
            x = muon_direction_(zero_m, full, 0.0, False, group["ns_steps"], group["ns_coefficients"], group["eps"])
            pos = 0
            for r in range(W):
                n = rows_of(shape, r)
                back_chunks[r].append(x[pos:pos + n].reshape(-1).float())
                pos += n
        back_send_sizes = [sum(c.numel() for c in ch) for ch in back_chunks]
        back_send = torch.cat([c for ch in back_chunks for c in ch]) if sum(back_send_sizes) else torch.empty(0, device=dev)
        back_recv = torch.empty(sum(send_sizes), dtype=torch.float32, device=dev)
        if W > 1:
            # the way back: owner o returns to rank r exactly what r sent it
            self._exchange(back_recv, back_send, [sizes[rank][o] for o in range(W)],
                           [[sizes[r][o] for r in range(W)] for o in range(W)], pg, rank)
            self.collectives_issued += 1
        else:
            back_recv.copy_(back_send)
        # 3. apply the update on local rows
        cursor = [sum(send_sizes[:r]) for r in range(W)]
        for (p, lay), owner, shape in zip(items, owners, shapes):
            if p.numel() == 0:
                continue
            n = p.numel()
            x = back_recv[cursor[owner]:cursor[owner] + n].view(p.shape)
            cursor[owner] += n
            rows, cols = shape[0], math.prod(shape[1:])
            muon_apply_(p.data, x.to(torch.bfloat16).contiguous(), float(group["lr"]), group["weight_decay"],
                        lr_ratio(group["adjust_lr_fn"], rows, cols))

    def _exchange(self, recv, send, recv_from, send_table, pg, rank):
        """Uneven all-to-all of fp32 elements. ``send_table[r][d]``: elements rank r sends to rank d, laid
        out in r's ``send`` in order of d; ``recv_from[r]``: elements this rank receives from r, stored
        in ``recv`` in order of r.

        On NVLink meshes with the peer-memory backend every rank publishes its send buffer in the
        symmetric region and *pulls* its pieces from the owners' memory with one kernel (no packing on
        the receiving side, no NCCL all-to-all); otherwise ``all_to_all_single``. The reference moves
        these row regions with ``all_to_all_single`` (``dist_muon/optimizer.py``)."""
        W = len(send_table)
        sc = self._symm_comm(pg, rank, W, send.device)
        if sc is not None and sc.all_to_all_pull(recv, send, [[4 * n for n in row] for row in send_table]):
            self.p2p_exchanges += 1
            return
        dist.all_to_all_single(recv, send, list(recv_from), list(send_table[rank]), group=pg)

    def _symm_comm(self, pg, rank, W, device):
        from ..parallel import comm as _comm

        if device.type != "cuda" or W <= 1 or _comm._backend() != "symm":
            return None
        sc = getattr(self, "_symm", None)
        if sc is None:
            from ..parallel.symm import SymmComm

            sc = self._symm = SymmComm(pg if pg is not None else dist.group.WORLD, rank, W, device)
        return sc

    # ------------------------------------------------------------------ state dict
    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._row_shard_plan = None  # replan after a reload (hyper-parameters may have changed)
