"""The decomposition behind the one-launch segment copies, checked without a GPU: the descriptor table of
a mixed list of strided copies, casts and zero-fills is replayed by a tiny interpreter over CPU memory and
must equal a plain ``copy_`` loop.  (The CUDA kernel that executes the same table is compared against the
same loop in ``test_segments_gpu.py``.)"""
import ctypes

import numpy as np
import torch

from flex_shard_b200.ops import segments as sg


def _replay(ops):
    plan = sg._Plan(ops)
    for i in range(plan.op.size):
        d, s = ops[plan.op[i]]
        dptr = d.data_ptr() + int(plan.doff[i])
        sptr = (s.data_ptr() + int(plan.soff[i])) if s is not None else 0
        n, mode = int(plan.n[i]), int(plan.mode[i])
        if mode == sg.MODE_COPY:
            ctypes.memmove(dptr, sptr, n)
        elif mode == sg.MODE_ZERO:
            ctypes.memset(dptr, 0, n)
        elif mode == sg.MODE_F32_TO_BF16:
            src = torch.from_numpy(np.ctypeslib.as_array((ctypes.c_float * n).from_address(sptr)))
            out = src.to(torch.bfloat16).view(torch.int16).numpy()
            ctypes.memmove(dptr, out.ctypes.data, 2 * n)
        else:
            raw = np.ctypeslib.as_array((ctypes.c_int16 * n).from_address(sptr))
            out = torch.from_numpy(raw.copy()).view(torch.bfloat16).float().numpy()
            ctypes.memmove(dptr, out.ctypes.data, 4 * n)
    return plan


def _cases():
    torch.manual_seed(0)
    a = torch.randn(6, 10)
    b = torch.randn(6, 10).bfloat16()
    row = torch.zeros(400)
    rowb = torch.zeros(400, dtype=torch.bfloat16)
    wide = torch.full((5, 12), 7.0)
    return [
        (row[0:60].view(6, 10), a),                                  # dense copy: one run
        (row[100:130].view(6, 5), a[:, 2:7]),                        # column slice: one run per row
        (rowb[0:60].view(6, 10), a),                                 # fp32 -> bf16
        (row[200:260].view(6, 10), b),                               # bf16 -> fp32
        (rowb[100:124].view(6, 4), b[:, 6:10]),                      # bf16 column slice
        (wide[:, 3:9], None),                                        # strided zero-fill
        (row[300:300], a[0:0].reshape(0)),                           # empty: skipped
        (row[320:340].view(2, 10), a[4:6]),                          # row slice of a dense tensor
    ]


def test_descriptor_table_equals_copy_loop():
    ops = _cases()
    want = []
    for d, s in _cases():           # the same geometry on fresh tensors, executed by copy_
        if s is None:
            d.zero_()
        else:
            d.copy_(s)
        want.append(d.clone())
    plan = _replay(ops)
    for (d, _), w in zip(ops, want):
        assert torch.equal(d, w)
    # run counts: 1 + 6 + 1 + 1 + 6 + 5 + 0 + 1
    assert plan.op.size == 21
    assert plan.mode.tolist().count(sg.MODE_ZERO) == 5


def test_cpu_path_and_cache_key():
    ops = _cases()
    assert sg.run_segment_ops(ops) == 0          # CPU tensors: plain loop, no launch
    assert torch.equal(ops[1][0], ops[1][1])
    k1, k2 = sg._key(_cases()), sg._key(_cases())
    assert k1 == k2                              # geometry only: addresses are not part of the key


def _table_of(ops):
    ops = [(d, s) for d, s in ops if d.numel()]
    plan = sg._Plan(ops)
    table = np.empty(plan.op.size, sg._DESC)
    dbase = np.asarray([d.data_ptr() for d, _ in ops], np.uint64)
    sbase = np.asarray([0 if s is None else s.data_ptr() for _, s in ops], np.uint64)
    table["dst"] = dbase[plan.op] + plan.doff.astype(np.uint64)
    table["src"] = sbase[plan.op] + plan.soff.astype(np.uint64)
    table["n"], table["mode"], table["pad"] = plan.n, plan.mode, 0
    return ops, plan, table


def test_debug_check_catches_stray_and_overlapping_runs():
    """The host-side check of a descriptor table (the debug mode that stands in for a device sanitizer): a valid
    table passes, a run moved outside its tensor's storage and two overlapping destinations are refused."""
    import pytest

    ops, plan, table = _table_of(_cases())
    sg._check_table(ops, plan, table)                       # the valid table
    bad = table.copy()
    bad["dst"][0] += np.uint64(400 * 4)                     # 60 floats starting at the end of a 400-float row
    with pytest.raises(RuntimeError, match="leaves its tensor's storage"):
        sg._check_table(ops, plan, bad)
    bad = table.copy()
    bad["src"][1] -= np.uint64(4096)
    with pytest.raises(RuntimeError, match="source run"):
        sg._check_table(ops, plan, bad)
    row = torch.zeros(64)
    a = torch.randn(4, 8)
    ops2, plan2, table2 = _table_of([(row[0:32].view(4, 8), a), (row[24:56].view(4, 8), a)])
    with pytest.raises(RuntimeError, match="overlap"):
        sg._check_table(ops2, plan2, table2)
