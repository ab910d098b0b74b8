"""Many small copies / casts as ONE kernel launch.

Placements move data between per-parameter tensors and packed communication rows: a few dozen strided
copies per bucket per pass.  Issued one ``copy_`` at a time they cost a launch each; here they are collected
as (destination view, source view) pairs, decomposed into contiguous runs, and executed by one launch of the
descriptor-driven segment kernel (``fsb_segment_op`` in ``csrc/elementwise.cu``: byte copy, fp32->bf16,
bf16->fp32, zero-fill; 16-byte vectors when the addresses allow).

The decomposition of a given list of shapes / strides / dtypes is computed once and cached as offsets
relative to each view's address (numpy arrays); a later call with the same geometry only adds the current
base addresses and writes the table to pinned memory, which the kernel reads in place (short tables) or
which is uploaded first (long ones).  CPU tensors take a plain ``copy_`` loop, which
is also the oracle the GPU test compares against.

Parity: the role of the reference's Triton copy kernels and their launchers
(``custom_placements/_copy_kernels.py:17-161`` kernels, ``:164-246`` descriptor tables staged through pinned
host memory, ``:362-461`` long segments split over the grid).
"""
from __future__ import annotations

import math
import threading

import numpy as np
import torch

from . import _lib
from ._lib import count_launch

MODE_COPY, MODE_F32_TO_BF16, MODE_BF16_TO_F32, MODE_ZERO = 0, 1, 2, 3
_MAX_SEGS = 65535
_DESC = np.dtype([("src", "<u8"), ("dst", "<u8"), ("n", "<i8"), ("mode", "<i4"), ("pad", "<i4")])


def _dense_tail(shape, *stride_sets) -> int:
    """Number of trailing dims over which every view is dense (so that they form one contiguous run)."""
    k, acc = 0, 1
    for d in range(len(shape) - 1, -1, -1):
        if shape[d] != 1 and any(st[d] != acc for st in stride_sets):
            break
        acc *= shape[d]
        k += 1
    return k


def _runs(shape, dst_stride, src_stride):
    """Element offsets (dst, src) of every contiguous run and the run length in elements."""
    if math.prod(shape) == 0:
        return np.zeros(0, np.int64), np.zeros(0, np.int64), 0
    sets = (dst_stride,) if src_stride is None else (dst_stride, src_stride)
    k = _dense_tail(shape, *sets)
    lead = shape[: len(shape) - k]
    run = math.prod(shape[len(shape) - k:])
    if not lead:
        return np.zeros(1, np.int64), np.zeros(1, np.int64), run
    idx = np.indices(lead, dtype=np.int64).reshape(len(lead), -1)
    doff = (idx * np.asarray(dst_stride[: len(lead)], np.int64)[:, None]).sum(0)
    soff = doff * 0 if src_stride is None else (idx * np.asarray(src_stride[: len(lead)], np.int64)[:, None]).sum(0)
    return doff, soff, run


class _Plan:
    __slots__ = ("op", "doff", "soff", "n", "mode", "blocks")

    def __init__(self, ops):
        op, doff, soff, n, mode = [], [], [], [], []
        longest = 1
        for i, (dst, src) in enumerate(ops):
            if src is None:
                m, unit = MODE_ZERO, dst.element_size()
            elif src.dtype == dst.dtype:
                m, unit = MODE_COPY, dst.element_size()
            elif src.dtype == torch.float32 and dst.dtype == torch.bfloat16:
                m, unit = MODE_F32_TO_BF16, 1
            elif src.dtype == torch.bfloat16 and dst.dtype == torch.float32:
                m, unit = MODE_BF16_TO_F32, 1
            else:
                raise TypeError(f"segment copy supports equal dtypes and fp32<->bf16, got {src.dtype} -> {dst.dtype}")
            if src is not None and tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"segment copy needs equal shapes, got {tuple(src.shape)} -> {tuple(dst.shape)}")
            d, s, run = _runs(tuple(dst.shape), dst.stride(), None if src is None else src.stride())
            if run == 0:
                continue
            op.append(np.full(d.shape, i, np.int64))
            doff.append(d * dst.element_size())
            soff.append(s * (src.element_size() if src is not None else 0))
            n.append(np.full(d.shape, run * unit, np.int64))     # bytes for copy / zero, elements for casts
            mode.append(np.full(d.shape, m, np.int32))
            longest = max(longest, run * dst.element_size())
        cat = (lambda xs, dt: np.concatenate(xs) if xs else np.zeros(0, dt))
        self.op, self.doff, self.soff = cat(op, np.int64), cat(doff, np.int64), cat(soff, np.int64)
        self.n, self.mode = cat(n, np.int64), cat(mode, np.int32)
        # CTAs per run: enough for the longest run to stream at full bandwidth (32 KB per CTA), bounded so that
        # the whole grid stays near sixteen CTAs per SM
        self.blocks = int(max(1, min(longest // (32 * 1024), (148 * 16) // max(1, self.op.size))))


def _key(ops):
    return tuple((tuple(d.shape), d.stride(), d.dtype, None if s is None else (s.stride(), s.dtype)) for d, s in ops)


_plans: dict = {}


def _check_table(ops, plan, table) -> None:
    """Debug check of a descriptor table on the host (``FSB200_CHECK_SEGMENTS=1``): every run must lie inside the
    storage of the tensor it belongs to, and no two destination runs may overlap. The kernel trusts its table, so
    this is where a wrong offset is caught before it becomes a stray device write."""
    unit = {MODE_COPY: (1, 1), MODE_ZERO: (1, 0), MODE_F32_TO_BF16: (2, 4), MODE_BF16_TO_F32: (4, 2)}
    spans = []
    for k in range(plan.op.size):
        d, s = ops[int(plan.op[k])]
        db, sb = unit[int(table["mode"][k])]
        n = int(table["n"][k])
        for what, t, start, nbytes in (("destination", d, int(table["dst"][k]), n * db),
                                       ("source", s, int(table["src"][k]), n * sb)):
            if t is None or nbytes == 0:
                continue
            st = t.untyped_storage()
            lo, hi = st.data_ptr(), st.data_ptr() + st.nbytes()
            if start < lo or start + nbytes > hi:
                raise RuntimeError(f"segment table: {what} run {k} [{start:#x}, +{nbytes}) leaves its tensor's storage "
                                   f"[{lo:#x}, {hi:#x})")
        spans.append((int(table["dst"][k]), int(table["dst"][k]) + n * db, k))
    spans.sort()
    for (a0, a1, ka), (b0, b1, kb) in zip(spans, spans[1:]):
        if b0 < a1:
            raise RuntimeError(f"segment table: destination runs {ka} and {kb} overlap ([{a0:#x}, {a1:#x}) and "
                               f"[{b0:#x}, {b1:#x}))")


def _checking() -> bool:
    import os

    return os.environ.get("FSB200_CHECK_SEGMENTS", "0") == "1"


def run_segment_ops(ops, cache: dict | None = None) -> int:
    """Execute ``ops`` = [(dst view, src view or None)]: copy (casting fp32<->bf16 when the dtypes differ) or
    zero-fill.  Destinations must not overlap.  On CUDA this is one launch (per 65 535 runs); returns the
    number of launches.  ``cache``: where the decomposition is remembered (default: a module-level table)."""
    ops = [(d, s) for d, s in ops if d.numel()]
    if not ops:
        return 0
    if not ops[0][0].is_cuda or torch.cuda.is_current_stream_capturing():
        # CPU tensors, or a stream capture (descriptor upload and the event bookkeeping are not capturable):
        # plain copies, which capture fine
        for d, s in ops:
            if s is None:
                d.zero_()
            else:
                d.copy_(s)
        return 0
    cache = _plans if cache is None else cache
    key = _key(ops)
    plan = cache.get(key)
    if plan is None:
        plan = _Plan(ops)
        if len(cache) < 8192:
            cache[key] = plan
    nseg = plan.op.size
    if nseg == 0:
        return 0
    dbase = np.asarray([d.data_ptr() for d, _ in ops], np.uint64)
    sbase = np.asarray([0 if s is None else s.data_ptr() for _, s in ops], np.uint64)
    table = np.empty(nseg, _DESC)
    table["dst"] = dbase[plan.op] + plan.doff.astype(np.uint64)
    table["src"] = sbase[plan.op] + plan.soff.astype(np.uint64)
    table["n"], table["mode"], table["pad"] = plan.n, plan.mode, 0
    if _checking():
        _check_table(ops, plan, table)
    dev = ops[0][0].device
    host = torch.from_numpy(table.view(np.uint8)).pin_memory()
    lib, stream, launches = _lib.load(), _lib.stream_ptr(dev), 0
    descs = None
    global _host_tables
    if _host_tables and nseg <= _HOST_TABLE_MAX:
        # short table: the kernel reads it where it is (page-locked host memory), no copy in the stream
        rc = lib.fsb_segment_op_host(host.data_ptr(), nseg, plan.blocks, stream)
        if rc == 1:
            _host_tables = False     # not device-accessible on this system: upload tables from now on
        else:
            _lib.check(rc, "fsb_segment_op_host")
            launches = 1
    if not launches:
        descs = host.to(dev, non_blocking=True)
        for lo in range(0, nseg, _MAX_SEGS):
            cnt = min(_MAX_SEGS, nseg - lo)
            rc = lib.fsb_segment_op(descs.data_ptr() + lo * _DESC.itemsize, cnt, plan.blocks, stream)
            _lib.check(rc, "fsb_segment_op")
            launches += 1
    count_launch(launches)
    # the pinned table must outlive the asynchronous upload: park it until the stream has passed this point
    _park(host, descs, dev)
    return launches


_parked: list = []
_parked_lock = threading.Lock()      # forward (caller's thread) and backward hooks (autograd's thread) both park tables
_host_tables = True
_HOST_TABLE_MAX = 512


def _park(host, descs, dev) -> None:
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(dev))
    with _parked_lock:
        _parked.append((ev, host, descs))
        while _parked and _parked[0][0].query():
            _parked.pop(0)
