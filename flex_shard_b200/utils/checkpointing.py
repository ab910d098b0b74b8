"""Keeping the bucket hooks out of selective activation checkpointing's sight.

Selective activation checkpointing (``torch.utils.checkpoint`` with a ``context_fn`` made by
``create_selective_checkpoint_contexts``) records, through a pair of dispatch modes, the operators a
checkpointed region runs in forward and replays or recomputes them in backward; it requires both passes to
run the same operators.  A bucket hook inside such a region does not satisfy that: whether it gathers,
consumes a prefetch, prefetches the next bucket or releases one depends on runtime state that differs
between the forward and the recompute.  The hooks produce nothing a checkpoint should save (gathers run
without grad and refill buffers in place), so they simply run with the checkpointing modes taken off the
dispatch stack, and every other mode left on.

Parity: ``flex_shard/utils.py:85-118`` of the reference.
"""
from __future__ import annotations

import contextlib
import functools

from torch.utils._python_dispatch import _get_current_dispatch_mode_stack, _pop_mode, _push_mode


def _sac_modes() -> tuple:
    try:
        from torch.utils.checkpoint import _CachedTorchDispatchMode, _CachingTorchDispatchMode

        return (_CachingTorchDispatchMode, _CachedTorchDispatchMode)
    except ImportError:        # a torch without selective checkpointing: nothing to hide from
        return ()


@contextlib.contextmanager
def hidden_from_selective_checkpoint():
    """Run the body with selective-checkpointing dispatch modes removed from the stack."""
    kinds = _sac_modes()
    stack = _get_current_dispatch_mode_stack() if kinds else []
    first = next((i for i, m in enumerate(stack) if isinstance(m, kinds)), None)
    if first is None:
        yield
        return
    taken = [_pop_mode() for _ in range(len(stack) - first)]        # innermost first
    others = [m for m in reversed(taken) if not isinstance(m, kinds)]
    for m in others:
        _push_mode(m)
    try:
        yield
    finally:
        for _ in others:
            _pop_mode()
        for m in reversed(taken):
            _push_mode(m)


def outside_selective_checkpoint(fn):
    """Decorator form of ``hidden_from_selective_checkpoint`` for hook methods."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        with hidden_from_selective_checkpoint():
            return fn(*args, **kwargs)

    return wrapper
