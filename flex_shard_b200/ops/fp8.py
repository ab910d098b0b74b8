"""Blockwise FP8 (e4m3) quantisers and the block-scaled tcgen05 GEMM, with a linear autograd fn.

Quantisation contract (bit-exact spec, parity with the reference's quantiser test
``tests/test_flex_shard_fp8_allgather.py:45-90``): tiles are padded with zeros; per tile
``amax = max|x|`` clamped at 1e-12; ``scale = 448/amax`` in fp32; ``q = clamp(x*scale, +-448)``
rounded to e4m3; the stored scale is ``1/scale`` (fp32). Weights use 128x128 tiles, activations
1x128 groups. CPU tensors take a PyTorch restatement of the same arithmetic.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import count_launch
from .gemm import gemm

FP8 = torch.float8_e4m3fn
_declared = False


def _ensure():
    global _declared
    if not _declared:
        c = ctypes
        vp, i32, i64 = c.c_void_p, c.c_int, c.c_longlong
        _lib.declare("fsb_fp8_quant_weight", [vp, vp, vp, i32, i32, i64, i64, vp])
        _lib.declare("fsb_fp8_quant_act", [vp, vp, vp, i64, i32, i64, i64, vp])
        _lib.declare("fsb_gemm_fp8", [vp, vp, vp, vp, i64, i64, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp])
        _declared = True


# --------------------------------------------------------------------------- quantisers
def quantize_blockwise_ref(w: torch.Tensor, block: int = 128):
    rows, cols = w.shape
    pr, pc = -(-rows // block) * block, -(-cols // block) * block
    wf = torch.zeros(pr, pc, dtype=torch.float32, device=w.device)
    wf[:rows, :cols] = w.to(torch.bfloat16).float()
    t = wf.view(pr // block, block, pc // block, block)
    amax = t.abs().amax(dim=(1, 3)).double().clamp_min(1e-12)
    scale = (448.0 / amax).float()   # correctly rounded quotient (fp64 divide, then fp32)
    q = (t * scale[:, None, :, None]).clamp(-448.0, 448.0).to(FP8)
    return q.view(pr, pc)[:rows, :cols].contiguous(), (1.0 / scale.double()).float()


def quantize_blockwise(w: torch.Tensor, out_q: torch.Tensor | None = None, out_scale: torch.Tensor | None = None):
    """bf16 ``[rows, cols]`` -> (e4m3 ``[rows, cols]``, fp32 reciprocal scales ``[ceil(r/128), ceil(c/128)]``)."""
    rows, cols = w.shape
    if not w.is_cuda:
        q, s = quantize_blockwise_ref(w)
        if out_q is not None:
            out_q.view(torch.uint8).copy_(q.view(torch.uint8))
            out_scale.copy_(s)
            return out_q, out_scale
        return q, s
    _ensure()
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1
    q = out_q if out_q is not None else torch.empty(rows, cols, dtype=FP8, device=w.device)
    s = out_scale if out_scale is not None else torch.empty(-(-rows // 128), -(-cols // 128), dtype=torch.float32,
                                                            device=w.device)
    rc = _lib.load().fsb_fp8_quant_weight(w.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols, w.stride(0),
                                          q.stride(0), _lib.stream_ptr(w.device))
    _lib.check(rc, "fsb_fp8_quant_weight")
    count_launch()
    return q, s


def dequantize_blockwise(q: torch.Tensor, inv_scale: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    rows, cols = q.shape
    s = inv_scale.repeat_interleave(128, 0)[:rows].repeat_interleave(128, 1)[:, :cols]
    return (q.float() * s).to(dtype)


def quantize_act_ref(x: torch.Tensor):
    T, K = x.shape
    g = x.to(torch.bfloat16).float().view(T, K // 128, 128)
    amax = g.abs().amax(-1).double().clamp_min(1e-12)
    scale = (448.0 / amax).float()
    q = (g * scale[..., None]).clamp(-448.0, 448.0).to(FP8).view(T, K)
    return q, (1.0 / scale.double()).float().t().contiguous()


def quantize_act(x: torch.Tensor):
    """bf16 ``[T, K]`` -> (e4m3 ``[T, K]``, fp32 reciprocal scales ``[K/128, T]``)."""
    T, K = x.shape
    if not x.is_cuda:
        return quantize_act_ref(x)
    _ensure()
    x = x if x.stride(1) == 1 else x.contiguous()
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.empty(K // 128, T, dtype=torch.float32, device=x.device)
    rc = _lib.load().fsb_fp8_quant_act(x.data_ptr(), q.data_ptr(), s.data_ptr(), T, K, x.stride(0), q.stride(0),
                                       _lib.stream_ptr(x.device))
    _lib.check(rc, "fsb_fp8_quant_act")
    count_launch()
    return q, s


# --------------------------------------------------------------------------- GEMM
def gemm_fp8(aq, sa, bq, sb, *, b_t: bool = False) -> torch.Tensor:
    """``out[M,N] = sum_kb sa[kb,m] * sb[..] * Aq[m,kb] . Bq[n,kb]`` in bf16.

    ``bq`` is the quantised weight ``[N, K]`` (``b_t=False``) or the same weight used transposed:
    stored ``[K, N]`` (``b_t=True``), with ``sb`` its 128x128 scales in storage orientation."""
    M, K = aq.shape
    N = bq.shape[1] if b_t else bq.shape[0]
    if not aq.is_cuda:
        a = aq.float().view(M, K // 128, 128) * sa.t()[..., None]
        w = dequantize_blockwise(bq, sb)
        w = w.t() if b_t else w
        return (a.view(M, K) @ w.t()).to(torch.bfloat16)
    _ensure()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    sc = sb.shape[1]
    stride_n, stride_k = (1, sc) if b_t else (sc, 1)
    status = _lib.status_word(aq.device)
    rc = _lib.load().fsb_gemm_fp8(aq.data_ptr(), sa.data_ptr(), bq.data_ptr(), sb.data_ptr(), stride_n, stride_k,
                                  out.data_ptr(), M, N, K, aq.stride(0), bq.stride(0), out.stride(0), int(b_t),
                                  status.data_ptr(), _lib.stream_ptr(aq.device))
    _lib.check(rc, "fsb_gemm_fp8")
    count_launch()
    return out


def fp8_linear_forward(x2: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    xq, sx = quantize_act(x2)
    return gemm_fp8(xq, sx, wq, ws)


class _Fp8Linear(torch.autograd.Function):
    """y = x W^T with W given as (e4m3 data, 128x128 reciprocal scales); the ``weight`` argument is
    the logical high-precision parameter that receives the (bf16-GEMM) weight gradient."""

    @staticmethod
    def forward(ctx, x, weight, wq, ws):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, wq, ws)
        ctx.xshape = x.shape
        ctx.weight = weight
        y = fp8_linear_forward(x2, wq, ws)
        return y.view(*x.shape[:-1], wq.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wq, ws = ctx.saved_tensors
        weight = ctx.weight
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = quantize_act(dy2)
            dx = gemm_fp8(dyq, sdy, wq, ws, b_t=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None and main.dtype in (torch.float32, torch.bfloat16):
                gemm(dy2, x2, a_t=True, b_t=True, out=main,
                     accumulate=bool(getattr(weight, "main_grad_written", False)))
                weight.main_grad_written = True
            else:
                gd = getattr(weight, "grad_dtype", None) or torch.bfloat16
                dw = gemm(dy2, x2, a_t=True, b_t=True,
                          out_dtype=gd if gd in (torch.bfloat16, torch.float32) else torch.bfloat16)
        return dx, dw, None, None


def fp8_linear(x, weight, wq, ws):
    return _Fp8Linear.apply(x, weight, wq, ws)
