"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some callers of this library run where device memory may not be allocated (inside another runtime's
execution callback, with all memory handed out up front). For them ``fsb_rmsnorm_bwd_noalloc`` keeps
its weight-gradient partial sums in a fixed array inside the library instead of a caller-allocated
buffer. This test checks it against the ordinary entry point (which takes the scratch buffer as an
argument) on two calls in a row with different sizes, since the array is shared between calls and
keeps the previous call's contents, and checks that an oversized problem is refused.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from flex_shard_b200.ops import _lib as L

    lib = L.load()
    c = ctypes
    vp, i32, i64 = c.c_void_p, c.c_int, c.c_longlong
    lib.fsb_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i64, i32, vp]
    lib.fsb_rmsnorm_bwd_noalloc.restype = c.c_int
    lib.fsb_rmsnorm_bwd_noalloc_capacity.argtypes = []
    lib.fsb_rmsnorm_bwd_noalloc_capacity.restype = c.c_longlong
    return lib, L


def _case(T, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return dy, x, w, rstd


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    lib, L = _lib()
    stream = L.stream_ptr(torch.device("cuda"))
    for T, D, seed in [(1000, 1024, 1), (333, 4096, 2)]:   # two calls in a row, second one smaller in rows
        dy, x, w, rstd = _case(T, D, seed)
        # ordinary entry point: scratch allocated by the caller
        dx_ref = torch.empty_like(x)
        dw_ref = torch.empty(D, device="cuda", dtype=torch.float32)
        scratch = torch.empty((T + 31) // 32, D, device="cuda", dtype=torch.float32)
        rc = lib.fsb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx_ref.data_ptr(),
                                 scratch.data_ptr(), dw_ref.data_ptr(), 1, 0, T, D, stream)
        assert rc == 0
        # allocation-free entry point: outputs provided by the caller, nothing else
        dx = torch.empty_like(x)
        dw = torch.empty(D, device="cuda", dtype=torch.float32)
        # the plain-PyTorch fp32 formula, evaluated before the memory measurement
        xf, dyf, wf, r = x.float(), dy.float(), w.float(), rstd.unsqueeze(-1)
        xhat = xf * r
        dyw = dyf * wf
        dx_formula = r * (dyw - xhat * (dyw * xhat).mean(-1, keepdim=True))
        dw_formula = (dyf * xhat).sum(0)
        del xf, dyf, wf, dyw
        torch.cuda.synchronize()
        before_torch = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()      # the driver's view: sees allocations the caching allocator does not
        rc = lib.fsb_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                         dx.data_ptr(), dw.data_ptr(), 1, 0, T, D, stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before_torch
        if (T, D) != (1000, 1024):       # the very first call on a device may load the kernels' module lazily
            assert free_after == free_before, (free_before, free_after)
        # against the fp32 formula (bf16 outputs: one rounding of values of order 1) and the ordinary entry point
        torch.testing.assert_close(dx.float(), dx_formula, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_formula, rtol=2e-3, atol=2e-3 * (T ** 0.5))
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_ref, rtol=2e-2, atol=2e-2)


def test_noalloc_entry_point_rejects_oversized_problem():
    lib, L = _lib()
    cap = lib.fsb_rmsnorm_bwd_noalloc_capacity()
    D = 4096
    T = (cap // D + 1) * 32          # one block row too many
    rc = lib.fsb_rmsnorm_bwd_noalloc(None, None, None, None, None, None, None, 1, 0, T, D,
                                     L.stream_ptr(torch.device("cuda")))
    assert rc == 64


def test_noalloc_entry_point_refuses_null_and_misaligned_pointers():
    lib, L = _lib()
    stream = L.stream_ptr(torch.device("cuda"))
    T, D = 64, 256
    dy, x, w, rstd = _case(T, D, 3)
    dx = torch.empty_like(x)
    dw = torch.empty(D, device="cuda", dtype=torch.float32)
    good = [dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr()]
    assert lib.fsb_rmsnorm_bwd_noalloc(*good, 1, 0, T, D, stream) == 0
    for i in (0, 1, 2, 3, 5, 6):                      # every required pointer, null
        args = list(good)
        args[i] = None
        assert lib.fsb_rmsnorm_bwd_noalloc(*args, 1, 0, T, D, stream) == 1, i
    for i in (0, 1, 2, 5):                            # bf16 tensors two bytes off a 16-byte boundary
        args = list(good)
        args[i] = good[i] + 2
        assert lib.fsb_rmsnorm_bwd_noalloc(*args, 1, 0, T, D, stream) == 1, i
    args = list(good)
    args[4] = dy.data_ptr() + 2                       # optional residual gradient, misaligned
    assert lib.fsb_rmsnorm_bwd_noalloc(*args, 1, 0, T, D, stream) == 1
    args = list(good)
    args[6] = dw.data_ptr() + 2                       # fp32 output on a 2-byte boundary
    assert lib.fsb_rmsnorm_bwd_noalloc(*args, 1, 0, T, D, stream) == 1
    torch.cuda.synchronize()
    from flex_shard_b200 import ops

    ops.check_status()
