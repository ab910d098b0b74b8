"""Training-loop helpers over sharded parameters: gradient-norm clipping, LR schedule, JSON metrics.

Parity: the helper functions of the reference's example (``examples/deepseek_v3/train.py:230-291``:
warm-up / stable / decay LR schedule, sharded grad-norm clip with one all-reduce per mesh).
"""
from __future__ import annotations

import json
import sys
import time

import torch
import torch.distributed as dist


def lr_lambda(step: int, warmup_steps: int, total_steps: int, decay_ratio: float = 0.0, min_lr_factor: float = 0.0):
    """Linear warm-up, constant plateau, linear decay over the last ``decay_ratio`` of training."""
    if warmup_steps > 0 and step < warmup_steps:
        return (step + 1) / (warmup_steps + 1)
    decay_steps = int(total_steps * decay_ratio)
    stable_end = total_steps - decay_steps
    if decay_steps <= 0 or step < stable_end:
        return 1.0
    progress = min(1.0, (step - stable_end + 1) / decay_steps)
    return 1.0 - progress * (1.0 - min_lr_factor)


@torch.no_grad()
def clip_grad_norm_(module, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    """Global gradient norm over every bucket's local shards (one all-reduce per distinct mesh), then
    scale the local gradients in place. Returns the total norm.  The per-parameter norms and the scaling run as
    multi-tensor (``_foreach``) operations: a handful of launches instead of several per parameter."""
    by_group: dict = {}
    all_grads = []
    for st in module.sharded_bucket_storages:
        # every rank takes part in every mesh's all-reduce, with zero when it holds no gradient there (an owner
        # placement can leave a rank without any local rows)
        acc = by_group.setdefault(id(st.comm.group), [st.comm, torch.zeros((), dtype=torch.float32, device=st.device)])
        grads = [p.grad for p in st.sharded_params if p.grad is not None and p.grad.numel() > 0]
        if not grads:
            continue
        all_grads += grads
        norms = torch.stack(torch._foreach_norm(grads, norm_type, dtype=torch.float32))
        acc[1] = acc[1] + (norms ** norm_type).sum()
    total = None
    for comm, v in by_group.values():
        if comm.world_size > 1:
            dist.all_reduce(v, group=comm.group)
        total = v if total is None else total + v
    if total is None:
        return torch.zeros(())
    total_norm = total ** (1.0 / norm_type)
    coef = (max_norm / (total_norm + 1e-6)).clamp(max=1.0)
    if all_grads:
        torch._foreach_mul_(all_grads, coef)
    return total_norm


class JsonMetrics:
    """One JSON line per step: loss, grad-norm, lr, tokens/s (device-timed), peak memory."""

    def __init__(self, stream=None, rank: int = 0, module=None):
        """``module``: a ``flex_shard`` module; when given, every record also carries ``exposed_comm_ms``,
        the device time its compute stream spent blocked on gathers and reductions during the step."""
        self.stream = stream or sys.stdout
        self.rank = rank
        self._ev = None
        self._t = None
        self._ctx = None
        if module is not None and torch.cuda.is_available():
            self._ctx = module._fsb_ctx()
            self._ctx.measure_exposed_comm(True)

    def start_step(self):
        if torch.cuda.is_available():
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        self._t = time.perf_counter()

    def end_step(self, step: int, tokens: int, **fields):
        if self._ev is not None:
            self._ev[1].record()
            self._ev[1].synchronize()
            ms = self._ev[0].elapsed_time(self._ev[1])
            from ..ops import _lib

            if _lib._status:       # the step has synchronised: a failed device-side wait raises on every rank that saw it
                _lib.check_status()
        else:
            ms = (time.perf_counter() - self._t) * 1e3
        rec = {"step": step, "ms": round(ms, 3), "tokens_per_s_per_gpu": round(tokens / (ms / 1e3), 1)}
        if torch.cuda.is_available():
            rec["peak_mem_gib"] = round(torch.cuda.max_memory_allocated() / 2**30, 2)
        if self._ctx is not None:
            rec["exposed_comm_ms"] = round(self._ctx.exposed_comm_ms(), 3)
        for k, v in fields.items():
            rec[k] = float(v) if isinstance(v, torch.Tensor) else v
        if self.rank == 0:
            self.stream.write(json.dumps(rec) + "\n")
            self.stream.flush()
        return rec
