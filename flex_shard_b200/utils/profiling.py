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
