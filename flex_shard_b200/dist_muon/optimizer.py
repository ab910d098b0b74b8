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


@dataclass
class _Item:
    """One managed parameter with everything the step needs to know about it."""

    param: torch.Tensor
    name: str
    storage: LocalMuonComputeLayout
    resolved: object = None     # ResolvedCompute


class DistMuon(torch.optim.Optimizer):
    """Muon over plain local tensors.

    ``compute_layouts`` (from ``get_flex_shard_muon_compute_layouts``) says how each parameter is *stored*;
    ``compute_sharding_by_fqn`` (public ``ComputeLayout`` records) says what Muon's matrices are and how
    they are spread while it computes; ``bucket_configs`` groups parameters that are exchanged and
    computed together, in order.  Parameters whose storage already holds whole matrices are updated in
    place with no communication; the others go through validated redistribution plans and the two-slot
    pipelined runtime (``reshard_plan`` / ``reshard_runtime``).  Parameter groups, names, layouts and
    plans are frozen after construction; ``load_state_dict`` re-plans.

    Parity: ``dist_muon/optimizer.py:162-653`` of the reference (one frozen group, hyper-parameters,
    ``ranks_per_host`` / ``owner_by_fqn`` balancing with loads carried from bucket to bucket, preflight before
    any update, momentum kept in the storage layout)."""

    def __init__(self, params, *, param_names: Sequence[str] | None = None, lr: float = 1e-3,
                 weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 ns_coefficients=NS_COEFFS, eps: float = 1e-7, ns_steps: int = 5,
                 adjust_lr_fn: str | None = None,
                 compute_layouts: Mapping[str, LocalMuonComputeLayout] | None = None,
                 compute_sharding_by_fqn: Mapping | None = None, bucket_configs: Sequence | None = None,
                 group: dist.ProcessGroup | None = None, ranks_per_host: int | None = None,
                 owner_by_fqn: Mapping[str, int] | None = None, payload_dtype: torch.dtype = torch.bfloat16):
        params = list(params)
        if params and isinstance(params[0], dict):
            if len(params) != 1:
                raise ValueError("DistMuon requires exactly one parameter group")
            if param_names is None and "param_names" in params[0]:
                param_names = list(params[0]["param_names"])
            params = list(params[0]["params"])
        if param_names is None:
            param_names = [f"param_{i}" for i in range(len(params))]
        if len(param_names) != len(params):
            raise ValueError("param_names must name every parameter")
        if len(set(param_names)) != len(param_names):
            raise ValueError("param_names must be unique")
        if ranks_per_host is not None and ranks_per_host <= 0:
            raise ValueError(f"ranks_per_host must be positive, got {ranks_per_host}")
        if not (isinstance(ns_steps, int) and ns_steps >= 0):
            raise ValueError(f"ns_steps must be a non-negative integer, got {ns_steps!r}")
        if len(tuple(ns_coefficients)) != 3:
            raise ValueError("ns_coefficients must be three numbers")
        if not 0.0 <= momentum < 1.0:
            raise ValueError(f"momentum must be in [0, 1), got {momentum}")
        lr_ratio(adjust_lr_fn, 1, 1)  # validates the mode
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_coefficients=tuple(ns_coefficients), eps=eps, ns_steps=ns_steps,
                        adjust_lr_fn=adjust_lr_fn)
        self._frozen = False
        super().__init__(params, defaults)
        self._frozen = True
        self.param_names = list(param_names)
        self._name_of = {id(p): n for p, n in zip(params, param_names)}
        self.compute_layouts = dict(compute_layouts or {})
        self.compute_sharding_by_fqn = dict(compute_sharding_by_fqn or {})
        self.bucket_configs = list(bucket_configs) if bucket_configs is not None else None
        self.group = group
        self.payload_dtype = payload_dtype
        self.collectives_issued = 0
        self.p2p_exchanges = 0
        self._owner_by_fqn = dict(owner_by_fqn or {})
        self._ranks_per_host = ranks_per_host
        self._buckets = None
        self._runtime = None
        self._validated_across_ranks = False
        self.owners: dict[str, tuple[int, ...]] = {}   # owner rank of every matrix of every travelling parameter
        # fail early on layouts that cannot be realised (before any state exists)
        from .compute_resolution import resolve_all

        self._resolved = resolve_all(self.param_names, {n: self._storage_of(p) for p, n in zip(params, param_names)},
                                     self.compute_sharding_by_fqn)

    def add_param_group(self, param_group) -> None:
        if getattr(self, "_frozen", False):
            raise RuntimeError("DistMuon parameter groups are frozen")
        super().add_param_group(param_group)

    # ------------------------------------------------------------------ helpers
    def _storage_of(self, p) -> LocalMuonComputeLayout:
        lay = self.compute_layouts.get(self._name_of[id(p)])
        if lay is None:
            return LocalMuonComputeLayout("matrix_batch" if p.dim() == 3 else "owned", global_shape=tuple(p.shape))
        if lay.global_shape is None:
            return LocalMuonComputeLayout(lay.kind, lay.block_rows, tuple(p.shape), lay.row_range)
        return lay

    def _layout(self, p) -> LocalMuonComputeLayout:
        return self._storage_of(p)

    def _momentum(self, p) -> torch.Tensor:
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        return st["momentum_buffer"]

    def _world(self) -> tuple[int, int]:
        if dist.is_initialized():
            return dist.get_world_size(self.group), dist.get_rank(self.group)
        return 1, 0

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

    # ------------------------------------------------------------------ planning
    def _plan(self):
        """Bind parameters to buckets, pick owners, build and validate the redistribution plans."""
        import fnmatch

        from .optimizer_reshard import BucketConfig
        from .reshard_plan import packed_schedule, plan_digest, plan_rows
        from .reshard_runtime import LocalBucket, RedistributedBucket, RedistributionRuntime
        from .compute_resolution import contiguous_owners

        group = self.param_groups[0]
        W, rank = self._world()
        items = [_Item(p, self._name_of[id(p)], self._storage_of(p), self._resolved[self._name_of[id(p)]])
                 for p in group["params"]]
        configs = self.bucket_configs if self.bucket_configs is not None else [BucketConfig(("*",), "all")]
        bound: list[list[_Item]] = [[] for _ in configs]
        for it in items:
            hits = [i for i, c in enumerate(configs) if any(fnmatch.fnmatchcase(it.name, pat) for pat in c.patterns)]
            if len(hits) != 1:
                raise ValueError(f"optimizer parameter {it.name!r} must match one bucket, matches {len(hits)}")
            bound[hits[0]].append(it)
        hosts = mesh_rank_hosts(W, self._ranks_per_host)
        loads = [0.0] * W                      # Newton-Schulz work per rank, carried from bucket to bucket
        steps = group["ns_steps"]
        buckets = []
        self.owners = {}
        row_plans: dict = {}     # identical layers (same shape, same storage rows, same owners) share one row plan
        for cfg, members in zip(configs, bound):
            if not members:
                continue
            local = [it for it in members if it.resolved.mode == "local"]
            moving = [it for it in members if it.resolved.mode == "redistributed"]
            if not moving:
                buckets.append(LocalBucket(tuple(local), cfg.name or ""))
                continue
            # owners: fixed ones first, contiguous spreads next, then the balancer over what is left
            owner_of: dict[tuple[str, int], int] = {}
            free: list[tuple[str, int, float]] = []
            for it in moving:
                res = it.resolved
                shapes = res.matrix_shapes()
                fixed = self._owner_by_fqn.get(it.name)
                if res.spread == "contiguous":
                    for b, o in enumerate(contiguous_owners(len(res.blocks), W)):
                        owner_of[(it.name, b)] = o
                        loads[o] += newton_schulz_cost(shapes[b], steps)
                elif fixed is not None:
                    seq = [fixed] * len(res.blocks) if isinstance(fixed, int) else list(fixed)
                    if len(seq) != len(res.blocks) or any(not 0 <= o < W for o in seq):
                        raise ValueError(f"owner_by_fqn[{it.name!r}] must give a rank in [0, {W}) per matrix")
                    for b, o in enumerate(seq):
                        owner_of[(it.name, b)] = o
                        loads[o] += newton_schulz_cost(shapes[b], steps)
                else:
                    free += [(it.name, b, newton_schulz_cost(shapes[b], steps)) for b in range(len(res.blocks))]
            for (name, b, _), o in zip(free, assign_to_hosts_then_ranks([c for _, _, c in free], hosts, loads)):
                owner_of[(name, b)] = o
            plans = []
            for it in moving:
                res = it.resolved
                rows = res.logical_shape[0]
                chunk = -(-rows // W)
                storage_rows = [(min(rows, r * chunk), min(rows, (r + 1) * chunk)) for r in range(W)]
                mine = it.storage.row_range
                if mine is not None and tuple(mine) != storage_rows[rank]:
                    raise ValueError(f"{it.name!r}: stored rows {tuple(mine)} are not the Shard(0) rows "
                                     f"{storage_rows[rank]} of rank {rank}")
                mats = [(lo, hi, owner_of[(it.name, b)]) for b, (lo, hi) in enumerate(res.blocks)]
                self.owners[it.name] = tuple(o for _, _, o in mats)
                key = (tuple(res.logical_shape), tuple(storage_rows), tuple(mats))
                if key not in row_plans:
                    row_plans[key] = plan_rows(res.logical_shape, storage_rows, mats)
                plans.append(row_plans[key])
            digest = plan_digest(plans, [(it.name, str(self.payload_dtype)) for it in members])
            buckets.append(RedistributedBucket(
                items=tuple(moving), plans=tuple(plans), to_compute=packed_schedule(plans, rank, True),
                to_storage=packed_schedule(plans, rank, False), local_items=tuple(local), name=cfg.name or "",
                digest=digest))
        dev = items[0].param.device if items else torch.device("cpu")
        self._buckets = buckets
        self._runtime = RedistributionRuntime(dev, self.group, self.payload_dtype, exchange=self._exchange)
        self._validated_across_ranks = False

    def _validate_across_ranks(self) -> None:
        from .reshard_plan import check_plans_across_ranks
        from .reshard_runtime import RedistributedBucket

        if self._validated_across_ranks:
            return
        for b in self._buckets:
            if isinstance(b, RedistributedBucket):
                check_plans_across_ranks(b.digest, self.group, self._runtime.device)
        self._validated_across_ranks = True

    @property
    def bucket_plans(self):
        if self._buckets is None:
            self._plan()
        return self._buckets

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._preflight()
        if self._buckets is None:
            self._plan()
        self._validate_across_ranks()
        self._runtime.run(self._buckets, self._prepare, self._compute, self._finalize, self._local_step)
        from ..ops import _lib

        _lib.poll_status()
        return loss

    # ---- parameters computed where they are stored
    def _stack_step(self, p3, g3, m3, group) -> bool:
        """One step for a stack ``[n, rows, cols]`` of equal matrices in one go (momentum over the whole stack,
        per-matrix normalisation, the batched Newton-Schulz iteration, one update): used when the batched
        iteration applies (CUDA, dimensions multiples of 128), else the caller loops over the matrices."""
        from ..ops.newton_schulz import batched_ns_supported, muon_momentum_direction_, newton_schulz

        if not (p3.dim() == 3 and p3.is_contiguous() and m3.is_contiguous() and batched_ns_supported(p3)):
            return False
        u = muon_momentum_direction_(m3, g3.contiguous(), group["momentum"], group["nesterov"])
        x = newton_schulz(u, group["ns_steps"], group["ns_coefficients"], group["eps"])
        muon_apply_(p3, x.contiguous(), float(group["lr"]), group["weight_decay"],
                    lr_ratio(group["adjust_lr_fn"], p3.shape[1], p3.shape[2]))
        return True

    def _local_step(self, it: _Item) -> None:
        p, lay, group = it.param, it.storage, self.param_groups[0]
        if p.numel() == 0:
            return
        g, m = p.grad, self._momentum(p)
        if lay.kind in ("owned", "matrix_batch") and p.dim() == 3 and self._stack_step(p.data, g, m, group):
            return
        if lay.kind == "row_blocks":
            blocks = lay.block_rows or (p.shape[0],)
            if len(blocks) > 1 and len(set(blocks)) == 1 and p.data.is_contiguous():
                n, rows = len(blocks), blocks[0]
                if self._stack_step(p.data.view(n, rows, -1), g.reshape(n, rows, -1), m.view(n, rows, -1), group):
                    return
        if lay.kind == "owned":
            if p.dim() == 2:
                self._matrix_step(p.data, g, m, group)
            elif p.dim() == 3:
                for i in range(p.shape[0]):
                    self._matrix_step(p.data[i], g[i], m[i], group)
            else:
                self._matrix_step(p.data.view(p.shape[0], -1), g.reshape(p.shape[0], -1), m.view(p.shape[0], -1), group)
        elif lay.kind == "matrix_batch":
            for i in range(p.shape[0]):
                self._matrix_step(p.data[i], g[i], m[i], group)
        elif lay.kind == "row_blocks":
            pos = 0
            p2, g2, m2 = (t.reshape(p.shape[0], -1) for t in (p.data, g, m))
            for rows in (lay.block_rows or (p.shape[0],)):
                gs = g2[pos:pos + rows]
                self._matrix_step(p2[pos:pos + rows], gs if gs.is_contiguous() else gs.contiguous(),
                                  m2[pos:pos + rows], group)
                pos += rows
        else:
            raise ValueError(f"unknown compute layout kind {lay.kind!r}")

    # ---- parameters that travel (stage callbacks of the pipelined runtime)
    def _prepare(self, it: _Item) -> torch.Tensor:
        """Momentum on the stored rows; returns the (Nesterov) direction in the storage layout."""
        from ..ops.newton_schulz import muon_momentum_direction_

        group = self.param_groups[0]
        p = it.param
        if p.numel() == 0:
            return torch.empty(p.shape, dtype=self.payload_dtype, device=p.device)
        return muon_momentum_direction_(self._momentum(p), p.grad, group["momentum"], group["nesterov"])

    def _compute(self, it: _Item, plan, full: torch.Tensor) -> torch.Tensor:
        """Newton-Schulz over this rank's matrices of one parameter, stacked along dim 0 in ``full``."""
        from ..ops.newton_schulz import newton_schulz

        group = self.param_groups[0]
        W, rank = self._world()
        out = torch.empty_like(full)
        mine = [hi - lo for lo, hi, owner in plan.matrices if owner == rank]
        if len(mine) > 1 and len(set(mine)) == 1:
            # equal matrices (heads, experts) stacked back to back: one batched iteration for all of them
            k, n = len(mine), mine[0]
            blk = full[:k * n]
            stack = (blk.reshape(k, blk.shape[-2], blk.shape[-1]) if it.resolved.batch else blk.reshape(k, n, -1))
            from ..ops.newton_schulz import batched_ns_supported

            if batched_ns_supported(stack):
                x = newton_schulz(stack, group["ns_steps"], group["ns_coefficients"], group["eps"])
                out[:k * n].copy_(x.reshape(blk.shape))
                return out
        pos = 0
        for lo, hi, owner in plan.matrices:
            if owner != rank:
                continue
            n = hi - lo
            blk = full[pos:pos + n]
            mat = blk.reshape(blk.shape[-2], blk.shape[-1]) if it.resolved.batch else blk.reshape(n, -1)
            x = newton_schulz(mat, group["ns_steps"], group["ns_coefficients"], group["eps"])
            out[pos:pos + n].copy_(x.reshape(blk.shape))
            pos += n
        return out

    def _finalize(self, it: _Item, update: torch.Tensor) -> None:
        """Apply the returned rows (bf16, storage layout) to the stored parameter."""
        group = self.param_groups[0]
        p = it.param
        if p.numel() == 0:
            return
        res = it.resolved
        lr, wd, mode = float(group["lr"]), group["weight_decay"], group["adjust_lr_fn"]
        shapes = res.matrix_shapes()
        ratios = {lr_ratio(mode, r, c) for r, c in shapes}
        upd = update.contiguous() if update.dtype == torch.bfloat16 else update.to(torch.bfloat16).contiguous()
        if len(ratios) == 1:
            muon_apply_(p.data, upd, lr, wd, ratios.pop())
            return
        lo0 = it.storage.row_range[0] if it.storage.row_range is not None else 0
        for (lo, hi), (r, c) in zip(res.blocks, shapes):   # blocks of different heights scale differently
            a, b = max(lo, lo0), min(hi, lo0 + p.shape[0])
            if b > a:
                muon_apply_(p.data[a - lo0:b - lo0], upd[a - lo0:b - lo0].contiguous(), lr, wd, lr_ratio(mode, r, c))

    def _exchange(self, recv, send, sched) -> None:
        """One uneven all-to-all of payload elements under ``sched``.

        On NVLink meshes with the peer-memory backend every rank publishes its packed send buffer in a
        symmetric region and *pulls* its pieces out of the senders' memory with one kernel (no NCCL
        all-to-all); otherwise ``all_to_all_single``.  The reference moves these regions with
        ``all_to_all_single`` (``dist_muon/_optimizer_reshard_runtime.py:103-120``)."""
        W, rank = self._world()
        if W == 1:
            recv.copy_(send)
            return
        self.collectives_issued += 1
        sc = self._symm_comm(self.group, rank, W, send.device)
        isz = send.element_size()
        if sc is not None and sc.all_to_all_pull(recv, send, [[isz * n for n in row] for row in sched.table]):
            self.p2p_exchanges += 1
            return
        dist.all_to_all_single(recv, send, list(sched.recv_splits), list(sched.send_splits), group=self.group)

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
        for p, st in self.state.items():   # the base class casts state to the parameter dtype: momentum stays fp32
            if "momentum_buffer" in st and st["momentum_buffer"].dtype != torch.float32:
                st["momentum_buffer"] = st["momentum_buffer"].float()
        self._buckets = None  # re-plan after a reload (hyper-parameters that shape the plans may have changed)
