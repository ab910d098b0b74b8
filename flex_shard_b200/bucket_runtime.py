"""The bucket runtime: hooks, prefetch, streams and the autograd choreography.

Per root module one ``BucketCommContext`` (streams, learned orders, pending
reductions) and per bucket one ``BucketRuntime``. Forward: the pre-forward hook
gathers the bucket (consuming a prefetch if one is in flight), swaps the
persistent unsharded ``nn.Parameter`` objects into the module and prefetches the
next bucket; the post-forward hook registers backward hooks and reshards.
Backward: a tensor hook on the outputs re-gathers, an identity autograd function
on the inputs fires the post-backward step (take grads -> reshard -> reduce on
the reduce stream -> accumulate into the sharded ``.grad``), and an engine
callback drains the reductions at the end of backward.

Parity: behaviour of ``flex_shard/bucket_runtime.py:210-1546`` of the reference
(context, runtime, hooks, learned and explicit prefetch, persistent unsharded
parameters with storage freed on reshard, no-sync accumulation, manual
finalization, error poisoning after a raised backward).
"""
from __future__ import annotations

import weakref
from typing import Sequence

import torch
import torch.nn as nn
from torch.autograd import Variable
from torch.utils._pytree import tree_flatten, tree_unflatten

from .bucket_comm import (
    PendingReduce,
    PendingUnshard,
    StreamHandoff,
    begin_bucket_unshard,
    begin_explicit_bucket_unshard,
    begin_reduce_grad,
)
from .bucket_storage import ShardedBucketStorage
from .utils.checkpointing import outside_selective_checkpoint
from .utils.profiling import record


def _outside_inference_mode(fn):
    """Run ``fn`` as in ordinary mode when the caller is under ``torch.inference_mode()`` (an evaluation pass before
    training): the gathered parameters and the buffers behind them outlive the call, and tensors created under
    inference mode (dtype views of the byte storage among them) could neither be saved by a later backward nor be
    refilled in place outside it.  Parity: the reference's "first unshard may run under inference_mode"
    (``tests/test_flex_shard_runtime.py:409-541`` there)."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if torch.is_inference_mode_enabled():
            with torch.inference_mode(False):
                return fn(*args, **kwargs)
        return fn(*args, **kwargs)

    return wrapper


def _in_backward() -> bool:
    return torch._C._current_graph_task_id() != -1


class BucketCommContext:
    """State shared by the buckets of one root module."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        if self.cuda:
            # high priority so collectives are not starved by queued compute kernels
            self.unshard_stream = torch.cuda.Stream(device=device, priority=-1)
            self.reduce_stream = torch.cuda.Stream(device=device, priority=-1)
            # third stream: where a retired reduction's buffers are handed back (it waits for the reduction,
            # then the buffers' allocation stream is ordered behind it), so the hand-back is not queued
            # behind unrelated work of either other stream
            self.release_stream = torch.cuda.Stream(device=device, priority=-1)
        else:
            self.unshard_stream = None
            self.reduce_stream = None
            self.release_stream = None
        self.retired_reduces: list[PendingReduce] = []
        self.runtimes: list["BucketRuntime"] = []
        self.forward_order: list["BucketRuntime"] = []
        self.post_forward_order: list["BucketRuntime"] = []
        self.learned = False
        self.pending_reduces: list[PendingReduce] = []
        self.max_pending_reduce_grads = 1
        self.manual_finalization = False
        self.backward_running = False
        self.callback_queued = False
        self.poisoned = False
        self.pending_finalize_handle = None
        self.stats = {"unshards": 0, "prefetch_hits": 0, "reduces": 0}
        self._exposed: list | None = None   # (before, after) event pairs around waits on communication

    # ------------------------------------------------------------------ exposed communication time
    def measure_exposed_comm(self, enabled: bool = True) -> None:
        """Start (or stop) timing how long the compute stream sits blocked on communication: every wait
        on a gather's or a reduction's completion event is bracketed by two timing events."""
        self._exposed = [] if (enabled and self.cuda) else None

    def exposed_comm_ms(self) -> float:
        """Milliseconds the compute stream spent waiting on gathers and reductions since the last call
        (device time between the bracketing events; synchronises)."""
        if not self._exposed:
            return 0.0
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in self._exposed)
        self._exposed.clear()
        return float(total)

    def wait_comm_event(self, event) -> None:
        cur = torch.cuda.current_stream()
        if self._exposed is None:
            cur.wait_event(event)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        cur.wait_event(event)
        b.record(cur)
        self._exposed.append((a, b))

    # ------------------------------------------------------------------ learned orders
    def note_forward(self, rt: "BucketRuntime") -> None:
        if not self.learned and rt not in self.forward_order:
            self.forward_order.append(rt)

    def note_post_forward(self, rt: "BucketRuntime") -> None:
        if not self.learned:
            if rt in self.post_forward_order:
                self.post_forward_order.remove(rt)
            self.post_forward_order.append(rt)

    def next_forward_bucket(self, rt):
        if rt in self.forward_order:
            i = self.forward_order.index(rt)
            if i + 1 < len(self.forward_order):
                return self.forward_order[i + 1]
        return None

    def next_backward_bucket(self, rt):
        order = self.post_forward_order
        if rt in order:
            i = order.index(rt)
            if i - 1 >= 0:
                return order[i - 1]
        return None

    # ------------------------------------------------------------------ reductions
    def drain_reduces(self, keep: int = 0) -> None:
        """Retire pending reductions until at most ``keep`` are left; with ``keep == 0`` (end of backward,
        ``finalize_backward().wait()``) also make the current stream wait for every retired one, so the
        optimizer sees the reduced gradients.

        A reduction that holds a packed send buffer is retired by ordering the buffer's allocation stream
        behind it before the buffer is dropped: with ``max_pending_reduce_grads = 1`` the next bucket's
        send buffer reuses the block, which bounds memory like FSDP2 does.  A reduction without buffers
        (gradients were written straight into the peers' symmetric memory) has nothing to hand back and is
        retired without making the compute stream wait for it."""
        while len(self.pending_reduces) > keep:
            st = self.pending_reduces.pop(0)
            buffers = [t for t in st.keep if isinstance(t, torch.Tensor)]
            if st.event is not None and (buffers or keep == 0):
                with record("FlexShard::post_backward_reduce_grad_retire" if keep else
                            "FlexShard::post_backward_reduce_grad_wait"):
                    if keep and self.release_stream is not None:
                        alloc_stream = torch.cuda.current_stream()
                        with torch.cuda.stream(self.release_stream):
                            self.release_stream.wait_event(st.event)
                            StreamHandoff.release_after_current_stream(st.keep, alloc_stream)
                    else:
                        self.wait_comm_event(st.event)
            elif st.event is not None:
                self.retired_reduces.append(st)
            st.keep.clear()
        if keep == 0:
            for st in self.retired_reduces:
                with record("FlexShard::post_backward_reduce_grad_wait"):
                    self.wait_comm_event(st.event)
            self.retired_reduces.clear()

    # ------------------------------------------------------------------ end of backward
    def queue_final_callback(self) -> None:
        if self.callback_queued:
            return
        self.callback_queued = True
        self.backward_running = True
        Variable._execution_engine.queue_callback(self._final_callback)

    def _final_callback(self) -> None:
        try:
            if not self.manual_finalization:
                for rt in reversed(self.post_forward_order or self.runtimes):
                    rt.finish_backward()
                for rt in self.runtimes:
                    if rt not in self.post_forward_order:
                        rt.finish_backward()
                self.drain_reduces(0)
            else:
                for rt in self.runtimes:
                    rt.end_of_backward_without_finalize()
            self.fence_peer_reads()
            for rt in self.runtimes:
                rt.release_unused_prefetch()
            if self.forward_order:
                self.learned = True
        finally:
            self.callback_queued = False
            self.backward_running = False
            for rt in self.runtimes:
                rt.reset_backward_state()

    def fence_peer_reads(self) -> None:
        """Buckets whose storage the peers read in place (symmetric memory): make the current stream wait
        until every peer has finished this backward's reads, so that whatever runs next on it (an
        optimizer step) may overwrite the shards."""
        seen = set()
        for rt in self.runtimes:
            comm = rt.storage.comm
            fence = getattr(comm, "fence_resident", None)
            if fence is not None and id(comm) not in seen:
                seen.add(id(comm))
                fence()

    def check_not_poisoned(self) -> None:
        if self.backward_running and not _in_backward():
            self.poisoned = True
        if self.poisoned:
            raise RuntimeError(
                "FlexShard: a previous backward raised before its gradient reduction finished; "
                "the runtime state is not recoverable.")

    def idle(self) -> bool:
        return (not self.pending_reduces and not self.retired_reduces and not self.backward_running
                and all(rt.pending is None for rt in self.runtimes))


class _PostBackwardTrigger(torch.autograd.Function):
    """Identity on a module's inputs; its backward runs after the module's parameter grads are
    accumulated (AccumulateGrad nodes run as soon as they are ready), so it marks the end of the
    bucket's backward."""

    @staticmethod
    def forward(ctx, rt_ref, *inputs):
        ctx.rt_ref = rt_ref
        return inputs

    @staticmethod
    def backward(ctx, *grads):
        rt = ctx.rt_ref()
        if rt is not None:
            rt.on_input_grads()
        return (None, *grads)


class BucketRuntime:
    def __init__(self, storage: ShardedBucketStorage, context: BucketCommContext,
                 modules: Sequence[nn.Module], is_group: bool):
        self.storage = storage
        self.context = context
        self.modules = list(modules)
        self.is_group = is_group or len(self.modules) > 1
        storage.runtime = self
        context.runtimes.append(self)
        self.is_unsharded = False
        self.unsharded_params: list[nn.Parameter] | None = None
        self.persistent: list[torch.Tensor] | None = None
        self.pending: PendingUnshard | None = None
        self.keepalive: list = []
        self._forwards_in_pass = 0     # member-module forwards since the last reshard
        self._triggers_registered = 0
        self._triggers_fired = 0
        self._pre_backward_done = False
        self._post_backward_done = False
        self._ran_forward = False      # a member module ran forward with gradients enabled since the last backward
        self.needs_sync = False        # holds unreduced unsharded grads (no-sync accumulation)
        self._handles: list = []
        self._bucket_base = None
        self._bucket_nbytes = 0

    # ------------------------------------------------------------------ persistent unsharded params
    def _refills_in_finish(self) -> bool:
        """False when the gather itself writes the persistent buffers (they must exist beforehand)."""
        pl = self.storage.placement
        direct = getattr(pl, "gathers_into_persistent", None)
        if direct is not None and direct(self.storage.infos, self.storage.comm):
            return False
        return pl.refills_persistent_buffers_in_finish

    def _aliases_storage(self) -> bool:
        fn = getattr(self.storage.placement, "unshard_aliases_storage", None)
        return bool(fn is not None and fn(self.storage.infos, self.storage.comm.world_size))

    def _alloc_persistent(self) -> list[torch.Tensor]:
        st = self.storage
        W = st.comm.world_size
        if self._aliases_storage():
            return []
        bucket_alloc = getattr(st.placement, "alloc_unsharded_bucket", None)
        if bucket_alloc is not None:
            # one buffer for the whole bucket; the parameters are views of it
            if self.persistent is None:
                self._bucket_base, self.persistent = bucket_alloc(st)
                self._bucket_nbytes = self._bucket_base.untyped_storage().size()
            elif self._bucket_base.untyped_storage().size() != self._bucket_nbytes:
                self._bucket_base.untyped_storage().resize_(self._bucket_nbytes)
            return self.persistent
        if self.persistent is None:
            self.persistent = []
            for info in st.infos:
                n = info.placement.unsharded_buffer_numel(info, W)
                self.persistent.append(torch.empty(n, dtype=info.param_dtype, device=st.device))
        else:
            for info, buf in zip(st.infos, self.persistent):
                n = info.placement.unsharded_buffer_numel(info, W)
                nbytes = n * info.param_dtype.itemsize
                if buf.untyped_storage().size() != nbytes:
                    buf.untyped_storage().resize_(nbytes)
        return self.persistent

    def _free_persistent(self) -> None:
        if self.persistent is None or self._aliases_storage():
            return
        if getattr(self, "_bucket_base", None) is not None:
            self._bucket_base.untyped_storage().resize_(0)
            return
        for buf in self.persistent:
            buf.untyped_storage().resize_(0)

    def _create_unsharded_params(self, tensors: list[torch.Tensor]) -> None:
        self.unsharded_params = []
        for info, t, sp in zip(self.storage.infos, tensors, self.storage.sharded_params):
            up = nn.Parameter(t, requires_grad=sp.requires_grad)
            for k, v in info.param_attrs.items():
                try:
                    setattr(up, k, v)
                except Exception:
                    pass
            up._fsb_sharded = weakref.ref(sp)
            up._fsb_storage = self.storage
            self.unsharded_params.append(up)
        self._set_unsharded_grad_dtypes(defer_upcast=False)

    # ------------------------------------------------------------------ gradient accumulation dtype
    def _accumulates_after_backward(self) -> bool:
        """How gradients of the gathered parameters accumulate across backward passes without
        reduction.  ``False`` (default): through autograd, by giving each gathered parameter the wider
        ``grad_dtype``.  ``True``: like the FSDP2 of older torch releases (those whose ``FSDPParam`` has
        ``to_accumulated_grad_if_needed``), which ``fsdp2_compatible`` buckets must reproduce bit for
        bit: every backward sums in the compute dtype, a kept gradient is widened to the reduce dtype
        after the backward, and the next backward's gradient is added to it when that backward ends."""
        from .bucket_storage import installed_fsdp2_accumulates_after_backward

        return self.storage.spec.fsdp2_compatible and installed_fsdp2_accumulates_after_backward()

    def _wide_grad_params(self):
        """(info, gathered parameter, wide dtype) for parameters whose gradient accumulates in a dtype
        wider than they compute in.  A parameter with a partial-gradient group keeps autograd's cast so
        that its all-reduce runs in the wider dtype."""
        for info, up in zip(self.storage.infos, self.unsharded_params or []):
            wide, cd = info.unsharded_grad_dtype, info.param_dtype
            if (wide is None or not up.requires_grad or not wide.is_floating_point or not cd.is_floating_point
                    or wide.itemsize <= cd.itemsize):
                continue
            yield info, up, wide

    def _set_unsharded_grad_dtypes(self, *, defer_upcast: bool) -> None:
        """Defer or restore the cast of gradients that accumulate in a wider dtype.

        Deferred (``grad_dtype = None``, set before a backward that reduces, or that adds to a kept
        gradient): autograd leaves new gradients in the compute dtype, the reduce-scatter copy-in
        widens them while it packs, and additions to a kept wide gradient happen in place; one cast
        kernel per parameter and the wide full-size gradients are saved.  A backward that does not
        reduce and starts a gradient keeps the cast, so a parameter used twice sums its uses in the
        wide dtype.  Restoring widens a kept gradient once and puts ``grad_dtype`` back.
        Parity: ``flex_shard/bucket_runtime.py:1062-1108`` of the reference."""
        if self._accumulates_after_backward():
            return
        syncing = self.storage.requires_gradient_sync and not self.context.manual_finalization
        for info, up, wide in self._wide_grad_params():
            if info.partial_grad_group is not None:
                if up.grad_dtype != wide:
                    up.grad_dtype = wide
                continue
            if defer_upcast:
                if up.grad is not None or syncing:
                    up.grad_dtype = None
                continue
            g = up.grad
            if g is not None and g.dtype != wide:
                up.grad = g.to(wide)
            up.grad_dtype = wide

    def _widen_kept_grads(self) -> None:
        """Older-FSDP2 accumulation: after a backward whose gradients are kept, move each into a wide
        accumulator (adding to the one a previous backward left)."""
        if not self._accumulates_after_backward():
            return
        for info, up, wide in self._wide_grad_params():
            if not info.explicit_reduce_dtype:
                continue
            acc, g = getattr(up, "_fsb_wide_grad", None), up.grad
            if g is None:
                continue
            if acc is None:
                up._fsb_wide_grad = g.to(wide)
            else:
                acc += g
            up.grad = None

    # ------------------------------------------------------------------ unshard / reshard
    @_outside_inference_mode
    def begin_unshard(self, prefetch: bool = False) -> None:
        if self.is_unsharded or self.pending is not None:
            return
        st = self.storage
        persistent = None
        if not self._refills_in_finish():
            persistent = self._alloc_persistent()
        stream = self.context.unshard_stream
        # a gather that lands straight in the persistent buffers refills tensors autograd may have
        # saved: same values, so the version counters must not move
        guard = tuple(persistent or ())
        if self._bucket_base is not None:
            guard = guard + (self._bucket_base,)
        with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(guard):
            self.pending = begin_bucket_unshard(st, persistent, stream)
        self.context.stats["unshards"] += 1

    @_outside_inference_mode
    def finish_unshard(self) -> None:
        p = self.pending
        assert p is not None
        self.pending = None
        st = self.storage
        if p.event is not None:
            self.context.wait_comm_event(p.event)
        persistent = self._alloc_persistent()
        # Refilling the persistent buffers must not look like an in-place edit to autograd: the
        # tensors saved by the forward are these very buffers, re-gathered with the same values.
        with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(tuple(persistent)):
            res = st.placement.finish_prepared_unshard(p.prepared, st.comm, persistent)
        if self.unsharded_params is None:
            self._create_unsharded_params(res.tensors)
        else:
            # refresh requires_grad from the sharded parameters (freezing after wrap takes effect here)
            for up, sp in zip(self.unsharded_params, st.sharded_params):
                if up.requires_grad != sp.requires_grad and up.grad_fn is None:
                    up.requires_grad_(sp.requires_grad)
        keep = list(res.keepalive)
        if p.prepared.recv is not None:
            keep.append(p.prepared.recv)
        StreamHandoff.release_after_current_stream(keep, p.stream)
        self.is_unsharded = True

    def unshard(self) -> None:
        if self.is_unsharded:
            return
        if self.pending is not None:
            self.context.stats["prefetch_hits"] += 1
        else:
            self.begin_unshard()
        self.finish_unshard()

    def explicit_unshard(self, async_op: bool = False):
        if _in_backward():
            raise RuntimeError("unshard() cannot run in backward; the runtime gathers buckets itself there.")
        self.context.check_not_poisoned()
        if self.is_unsharded:
            return _UnshardHandle([])
        if self.pending is None:
            st = self.storage
            persistent = None
            if not self._refills_in_finish():
                persistent = self._alloc_persistent()
            guard = tuple(persistent or ())
            if self._bucket_base is not None:
                guard = guard + (self._bucket_base,)
            with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(guard):
                self.pending = begin_explicit_bucket_unshard(st, persistent, async_op)
            self.context.stats["unshards"] += 1
        handle = _UnshardHandle([self])
        if not async_op:
            handle.wait()
        return handle

    @_outside_inference_mode
    def swap_in_unsharded(self) -> None:
        for up, slots in zip(self.unsharded_params, self.storage.param_slots):
            for mod, attr in slots:
                mod._parameters[attr] = up

    def swap_in_sharded(self) -> None:
        for sp, slots in zip(self.storage.sharded_params, self.storage.param_slots):
            for mod, attr in slots:
                mod._parameters[attr] = sp

    def reshard(self) -> None:
        if self.pending is not None and not self.is_unsharded:
            self.release_unused_prefetch()
        if not self.is_unsharded:
            return
        self.swap_in_sharded()
        self._free_persistent()
        self.is_unsharded = False
        self._forwards_in_pass = 0
        if self.unsharded_params is not None and not _in_backward():
            self._set_unsharded_grad_dtypes(defer_upcast=False)   # a deferred cast does not outlive the gathered state

    def release_unused_prefetch(self) -> None:
        """Drop a prefetched gather that nothing consumed (its buffers return to the allocator)."""
        p = self.pending
        if p is None or self.is_unsharded:
            return
        with record("FlexShard::release_unused_prefetch"):
            self.pending = None
            if p.event is not None:
                torch.cuda.current_stream().wait_event(p.event)
            if p.prepared.work is not None:
                p.prepared.work.wait()
            self._free_persistent()

    # ------------------------------------------------------------------ prefetch
    def _prefetch(self, forward: bool) -> None:
        st = self.storage
        explicit = st.forward_prefetch if forward else st.backward_prefetch
        if explicit is not None:
            for other in explicit:
                other.runtime.begin_unshard(prefetch=True)
            return
        ctx = self.context
        if not ctx.learned:
            return
        nxt = ctx.next_forward_bucket(self) if forward else ctx.next_backward_bucket(self)
        if nxt is not None and not nxt.is_unsharded:
            nxt.begin_unshard(prefetch=True)

    # ------------------------------------------------------------------ hooks
    @outside_selective_checkpoint
    def pre_forward(self, module, args, kwargs):
        ctx = self.context
        ctx.check_not_poisoned()
        in_bwd = _in_backward()
        with record("FlexShard::pre_forward", self.storage.name):
            if not in_bwd:
                ctx.note_forward(self)
            self.unshard()
            self.swap_in_unsharded()
            if not in_bwd:
                self._prefetch(forward=True)
        self._forwards_in_pass += 1
        if torch.is_grad_enabled() and not in_bwd:
            self._ran_forward = True
        if torch.is_grad_enabled() and not (in_bwd and self._triggers_registered > 0):
            flat, spec = tree_flatten((args, kwargs))
            idx = [i for i, t in enumerate(flat) if isinstance(t, torch.Tensor) and t.requires_grad]
            if idx:
                outs = _PostBackwardTrigger.apply(weakref.ref(self), *[flat[i] for i in idx])
                for i, o in zip(idx, outs):
                    flat[i] = o
                self._triggers_registered += 1
                args, kwargs = tree_unflatten(flat, spec)
        return args, kwargs

    @outside_selective_checkpoint
    def post_forward(self, module, args, output):
        ctx = self.context
        in_bwd = _in_backward()
        if not in_bwd:
            ctx.note_post_forward(self)
        if torch.is_grad_enabled():
            flat, _ = tree_flatten(output)
            for t in flat:
                if isinstance(t, torch.Tensor) and t.requires_grad:
                    t.register_hook(self._make_pre_backward_hook())
        if in_bwd:
            return output  # recompute inside backward: stay gathered until post-backward
        all_ran = (not self.is_group) or self._forwards_in_pass >= len(self.modules)
        if self.storage.reshard_after_forward and all_ran:
            self.reshard()
        return output

    def _make_pre_backward_hook(self):
        ref = weakref.ref(self)

        def hook(grad):
            rt = ref()
            if rt is not None:
                rt.pre_backward()
            return grad

        return hook

    @outside_selective_checkpoint
    def pre_backward(self) -> None:
        ctx = self.context
        ctx.queue_final_callback()
        if self._pre_backward_done:
            return
        self._pre_backward_done = True
        self._post_backward_done = False
        with record("FlexShard::pre_backward", self.storage.name):
            self.unshard()
            self.swap_in_unsharded()
            self._set_unsharded_grad_dtypes(defer_upcast=True)
            hook = self.storage.spec.pre_backward_hook
            if hook is not None:
                hook(self._hook_args())
            elif self.storage.placement.reduces_grads_in_param_layout(self.storage.infos):
                from .utils.validation import alloc_grads_in_param_layout

                alloc_grads_in_param_layout(self.storage)
            elif getattr(self.storage.placement, "wants_grad_bucket", lambda infos: False)(self.storage.infos):
                self.storage.placement.alloc_grad_bucket(self.storage, self.unsharded_params)
            self._prefetch(forward=False)

    def _hook_args(self):
        from .bucket_storage import BucketHookArgs

        pairs = [(i.fqn, u) for i, u in zip(self.storage.infos, self.unsharded_params or ())]
        return BucketHookArgs(self.storage, pairs)

    def on_input_grads(self) -> None:
        self._triggers_fired += 1
        if self._triggers_fired >= self._triggers_registered and not self.storage.spec.defer_post_backward:
            self.post_backward()

    def finish_deferred(self, param) -> None:
        """The late gradients of a deferring bucket exist: run its post-backward now (reduce into the shards and
        reshard with gradient sync on; keep the gradients for the next syncing backward without). Calls after the
        bucket has finished do nothing, so a hook per parameter may call it.
        Parity: ``flex_shard/flex_shard.py:215-235`` of the reference."""
        if not self.storage.spec.defer_post_backward:
            raise ValueError(f"bucket {self.storage.name!r} does not defer its post-backward "
                             "(BucketSpec.defer_post_backward)")
        if self._pre_backward_done and not self._post_backward_done:
            self.post_backward()
            if not _in_backward():
                self.context.drain_reduces(0)

    # ------------------------------------------------------------------ post-backward
    def _take_grads(self) -> list[torch.Tensor] | None:
        grads = []
        any_grad = False
        for info, up in zip(self.storage.infos, self.unsharded_params):
            if not info.requires_grad or not up.requires_grad:
                continue
            g = up.grad
            acc = getattr(up, "_fsb_wide_grad", None)
            if acc is not None:     # older-FSDP2 accumulation: this backward's gradient joins the kept one
                if g is not None:
                    acc += g
                g = acc
                up._fsb_wide_grad = None
            mg = getattr(up, "main_grad", None)
            if mg is not None:
                if getattr(up, "main_grad_written", False):
                    if g is not None and not hasattr(mg, "is_contiguous"):
                        raise RuntimeError(
                            "a parameter received both an in-place peer-memory gradient and an autograd "
                            "gradient in one backward; use grad_bucket=False for this bucket")
                    if g is not None:  # autograd also produced a gradient (e.g. a second use): fold it in
                        from .ops.elementwise import cast_scale_

                        dense = g.contiguous()
                        if mg.is_contiguous():
                            cast_scale_(mg.view(-1), dense.view(-1), 1.0, accumulate=True)
                        else:
                            br = mg.shape[1]
                            for i in range(mg.shape[0]):
                                lo, hi = i * br, min((i + 1) * br, dense.shape[0])
                                if hi > lo:
                                    mg[i, : hi - lo].add_(dense[lo:hi])
                    g = mg
                up.main_grad = None
                up.main_grad_written = False
            if g is not None:
                any_grad = True
            grads.append(g)
            up.grad = None
        trainable = [(i, u, sp) for i, u, sp in zip(self.storage.infos, self.unsharded_params,
                                                    self.storage.sharded_params)
                     if i.requires_grad and u.requires_grad]
        if self.storage.spec.fsdp2_compatible:
            # like an FSDP2 group: a parameter that received no gradient in this backward takes no part
            # in the reduce-scatter and its sharded .grad stays untouched (None if it never had one)
            kept = [(t, g) for t, g in zip(trainable, grads) if g is not None]
            if not kept:
                return None
            trainable, grads = [t for t, _ in kept], [g for _, g in kept]
        out = []
        for (info, up, _), g in zip(trainable, grads):
            if g is None:
                g = torch.zeros(info.global_shape, dtype=info.param_dtype, device=self.storage.device)
            if info.partial_grad_group is not None:
                torch.distributed.all_reduce(g, group=info.partial_grad_group)
            out.append(g)
        bucket = getattr(self.storage, "_grad_bucket", None)
        if getattr(bucket, "kind", None) == "peer":
            # the bucket's ring entry is already reserved on every rank: gradients that were not
            # written in place must still travel through it
            for g in out:
                if isinstance(g, torch.Tensor):
                    g._fsb_peer_target = bucket
        self.storage.infos_for_reduce = [t[0] for t in trainable]
        self._sharded_for_reduce = [t[2] for t in trainable]
        return out

    def post_backward(self) -> None:
        if self._post_backward_done or self.unsharded_params is None:
            return
        st = self.storage
        ctx = self.context
        self._post_backward_done = True
        with record("FlexShard::post_backward_reduce", st.name):
            if not st.requires_gradient_sync or ctx.manual_finalization:
                self.needs_sync = True
                if st.reshard_after_backward:
                    self.reshard()
                self._set_unsharded_grad_dtypes(defer_upcast=False)
                self._widen_kept_grads()
                return
            self._reduce_now()

    def _reduce_now(self) -> None:
        st = self.storage
        ctx = self.context
        if not self.is_unsharded and self.unsharded_params is None:
            return
        grads = self._take_grads()
        st._grad_bucket = None
        hook = st.spec.post_reduce_hook
        if st.reshard_after_backward:
            self.reshard()
        # the gradients are taken: this only puts the gathered parameters' grad_dtype back
        self._set_unsharded_grad_dtypes(defer_upcast=False)
        self.needs_sync = False
        if grads is None or not grads:
            if hook is not None:
                hook(self._hook_args())
            return
        reduce_dtype = st.bucket_reduce_dtype
        for g in grads:
            reduce_dtype = torch.promote_types(reduce_dtype, g.dtype) if st.spec.mp_policy.reduce_dtype is None else reduce_dtype
        ctx.drain_reduces(max(ctx.max_pending_reduce_grads - 1, 0))
        stream = ctx.reduce_stream if st.reduce_comm.world_size > 1 else None
        state = begin_reduce_grad(self, grads, reduce_dtype, st.reduction, stream)
        ctx.stats["reduces"] += 1
        ctx.pending_reduces.append(state)
        if hook is not None:
            hook(self._hook_args())

    def accumulate_sharded_grads(self, result) -> None:
        st = self.storage
        with record("FlexShard::reduce_grad_accumulate", st.name):
            for sp, g in zip(self._sharded_for_reduce, result.grads):
                if g is None:
                    continue
                info = sp._fsb_info
                gd = info.grad_dtype or sp.dtype
                if sp.grad is None:
                    sp.grad = g if g.dtype == gd else g.to(gd)
                else:
                    sp.grad.add_(g.to(sp.grad.dtype) if g.dtype != sp.grad.dtype else g)

    def finish_backward(self) -> None:
        """End of backward: run the post-backward step if its trigger never fired (inputs that do not require
        grad) and the bucket took part in this backward.  A bucket whose forward ran but whose outputs this rank
        did not use (or that still holds kept gradients from a backward without sync) reduces too, with zeros for
        the gradients it does not have: its peers may have used it, and every rank must issue the same
        collectives (parity: the reference's rank-dependent unused parameters,
        ``tests/test_flex_shard_training.py:1722-1761``).  ``fsdp2_compatible`` buckets keep FSDP2's rule instead:
        a group without gradients takes no part."""
        ran, self._ran_forward = self._ran_forward, False
        if self._pre_backward_done and not self._post_backward_done:
            if self.storage.spec.defer_post_backward and self.storage.requires_gradient_sync:
                raise RuntimeError(
                    f"bucket {self.storage.name!r} has defer_post_backward=True but its backward ended "
                    "without finish_deferred_backward() for every parameter")
            self.post_backward()
        elif (not self._pre_backward_done and (ran or self.needs_sync) and self.unsharded_params is not None
              and self.storage.requires_gradient_sync and not self.storage.spec.fsdp2_compatible
              and not self.storage.spec.defer_post_backward
              and any(i.requires_grad for i in self.storage.infos)):
            self._post_backward_done = False
            self.post_backward()

    def end_of_backward_without_finalize(self) -> None:
        if self._pre_backward_done and not self._post_backward_done:
            self._post_backward_done = True
            self.needs_sync = True
            if self.storage.reshard_after_backward:
                self.reshard()
            self._set_unsharded_grad_dtypes(defer_upcast=False)
            self._widen_kept_grads()

    def reset_backward_state(self) -> None:
        self._pre_backward_done = False
        self._post_backward_done = False
        self._triggers_registered = 0
        self._triggers_fired = 0

    def finalize(self) -> None:
        """Reduce gradients accumulated by no-sync / manual-finalization backwards."""
        if not self.needs_sync or self.unsharded_params is None:
            return
        self._reduce_now()


class _UnshardHandle:
    def __init__(self, runtimes):
        self.runtimes = runtimes

    def wait(self) -> None:
        for rt in self.runtimes:
            if rt.pending is not None and not rt.is_unsharded:
                rt.finish_unshard()
                rt.swap_in_unsharded()
        self.runtimes = []


class ModuleUnshardHandle(_UnshardHandle):
    pass


class GradientReductionHandle:
    def __init__(self, context: BucketCommContext):
        self.context = context
        self.done = False

    def wait(self) -> None:
        if not self.done:
            self.context.drain_reduces(0)
            self.context.pending_finalize_handle = None
            self.done = True


# --------------------------------------------------------------------------- installation
def install_bucket_hooks(root: nn.Module, storages: list[ShardedBucketStorage],
                         hook_modules: list[tuple[list[nn.Module], bool]],
                         context: BucketCommContext | None = None) -> BucketCommContext:
    device = storages[0].device if storages else torch.device("cpu")
    ctx = context or BucketCommContext(device)
    for st, (mods, is_group) in zip(storages, hook_modules):
        rt = BucketRuntime(st, ctx, mods, is_group)
        st.modules = list(mods)
        for m in mods:
            rt._handles.append(m.register_forward_pre_hook(rt.pre_forward, with_kwargs=True, prepend=True))
            rt._handles.append(m.register_forward_hook(rt.post_forward, prepend=False))

    def root_post_forward(module, args, output):
        if _in_backward():
            return output
        for rt in ctx.runtimes:
            if rt.is_group and rt.is_unsharded and rt.storage.reshard_after_forward and rt._forwards_in_pass > 0:
                rt.reshard()
        return output

    root.register_forward_hook(root_post_forward, prepend=False)

    def state_dict_pre_hook(module, prefix, keep_vars):
        for rt in ctx.runtimes:
            rt.reshard()

    root.register_state_dict_pre_hook(state_dict_pre_hook)
    root._register_load_state_dict_pre_hook(lambda *a, **k: [rt.reshard() for rt in ctx.runtimes] and None)
    return ctx
