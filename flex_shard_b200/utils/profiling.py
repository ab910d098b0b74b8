"""Named ranges around runtime phases: ``torch.profiler.record_function`` plus NVTX when on.

Range names follow the ``FlexShard::<phase>`` convention of the reference
(``flex_shard/utils.py:35-78``) so traces of both line up.
"""
from __future__ import annotations

import contextlib
import os

import torch

_NVTX = os.environ.get("FSB200_NVTX", "0") == "1"
_RANGES = os.environ.get("FSB200_PROFILE_RANGES", "1") == "1"


@contextlib.contextmanager
def record(name: str, bucket: str | None = None):
    if not _RANGES:
        yield
        return
    label = name if bucket is None else f"{name} ({bucket})"
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(label)
    try:
        with torch.profiler.record_function(label):
            yield
    finally:
        if _NVTX and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()


_WRAPPER_PARTS = ("_checkpoint_wrapped_module", "_orig_mod")


def strip_wrapper_path(path: str) -> str:
    """Module path without the components that activation-checkpoint / compile wrappers insert."""
    return ".".join(p for p in path.split(".") if p and p not in _WRAPPER_PARTS)


def bucket_debug_fqn(fqns) -> str | None:
    """A short name for a bucket in traces: the longest module path shared by the owners of its
    parameters (wrapper components removed); when they share none, the distinct top-level owners joined by
    ", " (``layers.3`` counts as top level for parameters under a module list); ``None`` for no parameters.
    Parity: ``flex_shard/utils.py:169-193`` of the reference."""
    owners = sorted({strip_wrapper_path(".".join(f.split(".")[:-1])) for f in fqns})
    if not owners:
        return None
    parts = [o.split(".") if o else [] for o in owners]
    common = []
    for level in zip(*parts):
        if len(set(level)) != 1:
            break
        common.append(level[0])
    if common:
        return ".".join(common)
    tops = []
    for p in parts:
        if not p:
            continue
        top = ".".join(p[:2]) if len(p) > 1 and p[1].isdigit() else p[0]
        if top not in tops:
            tops.append(top)
    return ", ".join(tops) if tops else None
