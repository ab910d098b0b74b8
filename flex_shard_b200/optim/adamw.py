"""AdamW over local shards, one kernel launch per bucket.

The optimizer holds ordinary local ``nn.Parameter`` views (as any optimizer would
after ``flex_shard``). When all of a bucket's parameters sit in this optimizer and
their reduced gradients are views of the bucket's reduce-scatter output at matching
offsets, the update runs as ONE flat sm_100a kernel over the bucket's storage;
otherwise it falls back to one launch per parameter. State (``exp_avg``,
``exp_avg_sq`` in fp32, ``step``) is exposed per parameter, so ``state_dict`` and
the checkpoint hook look like ``torch.optim.AdamW``'s.

Replaces ``torch.optim.AdamW(fused=True)`` as used by the reference's example
(``examples/deepseek_v3/train.py:297-310``).
"""
from __future__ import annotations

import torch

from ..ops import _lib
from ..ops.elementwise import adamw_step_


class FusedAdamW(torch.optim.Optimizer):
    _fsb_adam_like = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self._flat: dict[int, dict] = {}  # id(storage) -> flat m/v buffers

    # ------------------------------------------------------------------ state
    def _bucket_of(self, p):
        return getattr(p, "_fsb_storage", None)

    def _init_bucket_state(self, storage, params):
        """Flat fp32 moment buffers covering the whole bucket shard; per-parameter state tensors
        are views into them."""
        first = params[0]
        itemsize = first.element_size()
        n = storage.byte_storage.numel() // itemsize
        m = torch.zeros(n, dtype=torch.float32, device=first.device)
        v = torch.zeros(n, dtype=torch.float32, device=first.device)
        for p in params:
            off = p._fsb_info.byte_offset // itemsize
            st = self.state[p]
            st["step"] = torch.zeros((), dtype=torch.float32)
            st["exp_avg"] = m[off:off + p.numel()].view(p.shape)
            st["exp_avg_sq"] = v[off:off + p.numel()].view(p.shape)
        self._flat[id(storage)] = {"m": m, "v": v, "n": n}
        return self._flat[id(storage)]

    def _init_param_state(self, p):
        st = self.state[p]
        st["step"] = torch.zeros((), dtype=torch.float32)
        st["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        st["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)

    def load_state_dict(self, state_dict) -> None:
        """Loads like ``torch.optim.Optimizer.load_state_dict`` but keeps the moments in fp32.

        The base class casts floating-point state to each parameter's dtype, so after loading into
        bf16 parameters ``exp_avg`` / ``exp_avg_sq`` would be bf16 while the kernel reads and writes
        them as fp32.  Here the loaded values are taken in fp32 straight from ``state_dict`` and, for
        buckets updated as one flat launch, copied into freshly built flat buffers whose views replace
        the per-parameter tensors (stale flat buffers from before the load are dropped)."""
        import itertools

        loaded = state_dict["state"]
        super().load_state_dict(state_dict)
        # map the positional ids of the saved groups onto this optimizer's parameters
        saved_ids = itertools.chain.from_iterable(g["params"] for g in state_dict["param_groups"])
        mine = itertools.chain.from_iterable(g["params"] for g in self.param_groups)
        self._flat = {}
        by_bucket: dict[int, tuple] = {}
        for pid, p in zip(saved_ids, mine):
            src = loaded.get(pid)
            if src is None or p not in self.state:
                continue
            st = self.state[p]
            for key in ("exp_avg", "exp_avg_sq"):
                if key in src:
                    st[key] = src[key].detach().to(device=p.device, dtype=torch.float32).reshape(p.shape).clone()
            if "step" in src:
                step = src["step"]
                st["step"] = (step.detach().to("cpu", torch.float32).reshape(()).clone() if torch.is_tensor(step)
                              else torch.tensor(float(step), dtype=torch.float32))
            storage = self._bucket_of(p)
            if storage is not None and storage.byte_storage is not None:
                by_bucket.setdefault(id(storage), (storage, []))[1].append(p)
        for storage, plist in by_bucket.values():
            complete = (len(plist) == len(storage.sharded_params) and len({p.dtype for p in plist}) == 1
                        and all("exp_avg" in self.state[p] and "step" in self.state[p] for p in plist))
            if not complete:
                continue
            old = [(self.state[p]["exp_avg"], self.state[p]["exp_avg_sq"], self.state[p]["step"]) for p in plist]
            self._init_bucket_state(storage, plist)
            for p, (m, v, step) in zip(plist, old):
                self.state[p]["exp_avg"].copy_(m)
                self.state[p]["exp_avg_sq"].copy_(v)
                self.state[p]["step"] = step

    # ------------------------------------------------------------------ optimizer inside backward
    def fuse_into_backward(self, module) -> None:
        """Apply this optimizer's update to a bucket the moment its gradients are complete, while the
        backward pass of the remaining layers is still running: on multi-rank peer-memory meshes inside
        the fused reduce-scatter kernel (no gradient is materialised for those buckets), on 1-rank meshes
        as one flat AdamW launch on a side stream. ``step()`` then only covers what is left and joins
        the side stream. Not compatible with gradient clipping, which needs every gradient before any
        update, nor with reusing a layer's parameters later in the same backward pass."""
        for st in module.sharded_bucket_storages:
            plist = [p for p in st.sharded_params]
            mine = {id(p) for g in self.param_groups for p in g["params"]}
            if all(id(p) in mine for p in plist) and len({p.dtype for p in plist}) == 1:
                st._fused_opt = self
        self._stepped_in_backward: set[int] = set()
        self._backward_events: list = []

    def step_bucket_in_backward(self, storage, stream) -> bool:
        """1-rank path: the bucket's gradients are final; update it on ``stream`` after everything queued
        so far on the current stream. Returns False when the bucket cannot be updated as one flat launch."""
        plist = list(storage.sharded_params)
        if not plist or any(p.grad is None for p in plist) or not self._grads_flat(plist, storage):
            return False
        if len({p.grad.dtype for p in plist}) != 1:
            return False
        ev = torch.cuda.current_stream().record_event()
        stream.wait_event(ev)
        with torch.cuda.stream(stream):
            self.step_bucket(storage)
            self._backward_events.append(stream.record_event())
        self._stepped_in_backward.add(id(storage))
        return True

    def fused_bucket_args(self, storage):
        """Hyper-parameters and flat state for one bucket, or ``None`` when it cannot be fused."""
        plist = list(storage.sharded_params)
        group = next((g for g in self.param_groups if any(p is plist[0] for p in g["params"])), None)
        if group is None or not all(p.requires_grad for p in plist):
            return None
        flat = self._flat.get(id(storage))
        if flat is None:
            if any("step" in self.state[p] for p in plist):
                return None
            flat = self._init_bucket_state(storage, plist)
        step = None
        for p in plist:
            self.state[p]["step"] += 1
            step = int(self.state[p]["step"])
        self._stepped_in_backward.add(id(storage))
        return dict(p=storage.byte_storage.view(plist[0].dtype), m=flat["m"], v=flat["v"], lr=float(group["lr"]),
                    beta1=group["betas"][0], beta2=group["betas"][1], eps=group["eps"],
                    weight_decay=group["weight_decay"], step=step)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        done = getattr(self, "_stepped_in_backward", None)
        for ev in getattr(self, "_backward_events", ()):   # updates issued on the side stream during backward
            torch.cuda.current_stream().wait_event(ev)
        if getattr(self, "_backward_events", None):
            self._backward_events.clear()
        for group in self.param_groups:
            hp = dict(lr=float(group["lr"]), beta1=group["betas"][0], beta2=group["betas"][1],
                      eps=group["eps"], weight_decay=group["weight_decay"])
            by_bucket: dict[int, list] = {}
            loose = []
            for p in group["params"]:
                st = self._bucket_of(p)
                if st is None or st.byte_storage is None:
                    loose.append(p)
                else:
                    by_bucket.setdefault(id(st), []).append(p)
            for key, plist in by_bucket.items():
                if done and key in done:
                    continue  # already updated by the fused reduce kernel during backward
                self._step_bucket(plist, hp)
            for p in loose:
                if p.grad is not None:
                    self._step_param(p, hp)
        if done:
            done.clear()
        _lib.poll_status()   # a bounded device wait that ran out (late or missing peer) raises here, one step late at most
        return loss

    def step_bucket(self, storage) -> None:
        """Update one bucket now (used to apply the optimizer inside backward, right after the
        bucket's gradient reduction, so its gradients can be freed immediately)."""
        with torch.no_grad():
            for group in self.param_groups:
                plist = [p for p in group["params"] if self._bucket_of(p) is storage]
                if plist:
                    hp = dict(lr=float(group["lr"]), beta1=group["betas"][0], beta2=group["betas"][1],
                              eps=group["eps"], weight_decay=group["weight_decay"])
                    self._step_bucket(plist, hp)

    def _step_param(self, p, hp):
        st = self.state[p]
        if "step" not in st:
            self._init_param_state(p)
        st["step"] += 1
        if p.numel() == 0:
            return
        pf = p.data if p.is_contiguous() else None
        g = p.grad
        if pf is None or not g.is_contiguous():
            raise RuntimeError("FusedAdamW needs contiguous parameters and gradients")
        adamw_step_(pf.view(-1), g.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                    step=int(st["step"]), **hp)

    def _step_bucket(self, plist, hp):
        storage = self._bucket_of(plist[0])
        have_grads = [p for p in plist if p.grad is not None]
        if not have_grads:
            return
        flat = self._flat.get(id(storage))
        all_in = len(plist) == len(storage.sharded_params) and len(have_grads) == len(plist)
        same_dtype = len({p.dtype for p in plist}) == 1 and len({p.grad.dtype for p in plist}) == 1
        eligible = all_in and same_dtype and self._grads_flat(plist, storage)
        if eligible and flat is None and all("step" not in self.state[p] for p in plist):
            flat = self._init_bucket_state(storage, plist)
        if eligible and flat is not None:
            step = None
            for p in plist:
                self.state[p]["step"] += 1
                step = int(self.state[p]["step"])
            nz = [p for p in plist if p.numel() > 0]
            if not nz:
                return
            itemsize = nz[0].element_size()
            pflat = storage.byte_storage.view(nz[0].dtype)
            g0 = nz[0].grad
            goff = g0.storage_offset() - nz[0]._fsb_info.byte_offset // itemsize
            n = flat["n"]
            gbase = g0.as_strided((n,), (1,), goff)
            adamw_step_(pflat, gbase, flat["m"], flat["v"], step=step, **hp)
            return
        for p in have_grads:
            self._step_param(p, hp)

    @staticmethod
    def _grads_flat(plist, storage) -> bool:
        """True when the grads are views of one buffer laid out like the bucket storage."""
        nz = [p for p in plist if p.numel() > 0]
        if not nz:
            return True
        g0 = nz[0].grad
        itemsize = nz[0].element_size()
        base_ptr = g0.untyped_storage().data_ptr()
        goff = g0.storage_offset() - nz[0]._fsb_info.byte_offset // itemsize
        if goff < 0:
            return False
        n = storage.byte_storage.numel() // itemsize
        if (g0.untyped_storage().nbytes() // g0.element_size()) < goff + n:
            return False
        for p in nz:
            g = p.grad
            if g.untyped_storage().data_ptr() != base_ptr or not g.is_contiguous():
                return False
            if g.storage_offset() - p._fsb_info.byte_offset // itemsize != goff:
                return False
        return True
