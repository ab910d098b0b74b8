"""MXFP8: e4m3 data with one power-of-two (e8m0) scale per 32 elements, quantisers and the
block-scaled tcgen05 GEMM (``kind::mxf8f6f4.block_scale``), with a linear autograd function.

Contract (the "round up" scaling mode, parity with ``scaling_mode="rceil"`` of
``custom_placements/mxfp8_bucketed_block_shard.py:7-31`` in the reference): the scale of a group is
the smallest power of two ``s`` with ``amax / s <= 448``, stored as the byte ``log2(s) + 127``
(0 for an all-zero group); ``q = e4m3(x / s)``. Weights use 32x32 tiles, so one set of tile
exponents serves the forward product (contraction over the columns) and the input-gradient product
(contraction over the rows); activations use 1x32 groups.

Scale tensors handed to the GEMM are in the tensor core's block layout: rows in blocks of 128,
groups in blocks of 4, every (row block, group block) being 512 contiguous bytes with the byte of
(row r, group g) at ``(r % 32) * 16 + (r // 32) * 4 + g``. CPU tensors take a PyTorch restatement.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import count_launch
from .gemm import gemm

FP8 = torch.float8_e4m3fn
GROUP = 32
MX_WGRAD = True   # weight gradients of the MXFP8 linear as a third block-scaled product (when dims allow)
_declared = False


def _ensure():
    global _declared
    if not _declared:
        c = ctypes
        vp, i32, i64 = c.c_void_p, c.c_int, c.c_longlong
        _lib.declare("fsb_mx_quant_weight", [vp, vp, vp, i32, i32, i64, i64, vp])
        _lib.declare("fsb_mx_expand_scales", [vp, vp, i32, i32, i32, vp])
        _lib.declare("fsb_mx_quant_act", [vp, vp, vp, i64, i32, i64, i64, vp])
        _lib.declare("fsb_mx_quant_rows", [vp, vp, vp, i64, i32, i64, i64, vp])
        _lib.declare("fsb_gemm_mxfp8", [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, i32, vp, vp])
        _declared = True


# --------------------------------------------------------------------------- layout helpers
def blocked_scale_numel(rows: int, cols: int) -> int:
    """Bytes of the blocked scale tensor of an operand ``[rows, cols]`` (groups along the columns)."""
    return (-(-rows // 128) * 128) * (-(-(-(-cols // GROUP)) // 4) * 4)


def _blocked_index(rows_p: int, groups_p: int, device) -> torch.Tensor:
    r = torch.arange(rows_p, device=device)[:, None]
    g = torch.arange(groups_p, device=device)[None, :]
    return ((r // 128) * (groups_p // 4) + g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4


def to_blocked(scales: torch.Tensor) -> torch.Tensor:
    """Logical ``[rows, groups]`` uint8 exponents -> blocked bytes (padding = 127, i.e. scale 1)."""
    rows, groups = scales.shape
    rp, gp = -(-rows // 128) * 128, -(-groups // 4) * 4
    full = torch.full((rp, gp), 127, dtype=torch.uint8, device=scales.device)
    full[:rows, :groups] = scales
    out = torch.empty(rp * gp, dtype=torch.uint8, device=scales.device)
    out[_blocked_index(rp, gp, scales.device).reshape(-1)] = full.reshape(-1)
    return out


def from_blocked(blocked: torch.Tensor, rows: int, groups: int) -> torch.Tensor:
    rp, gp = -(-rows // 128) * 128, -(-groups // 4) * 4
    return blocked.view(torch.uint8).reshape(-1)[_blocked_index(rp, gp, blocked.device)][:rows, :groups]


def _round_up_exponent(amax: torch.Tensor) -> torch.Tensor:
    v = (amax.float() * (1.0 / 448.0)).contiguous()
    bits = v.view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = torch.where(((bits & 0x7FFFFF) != 0) & (e < 254), e + 1, e).clamp(max=254)
    return torch.where(amax > 0, e, torch.zeros_like(e)).to(torch.uint8)


def _inv_scale(e: torch.Tensor) -> torch.Tensor:
    return torch.exp2(127.0 - e.float())


# --------------------------------------------------------------------------- quantisers
def mx_quantize_weight_ref(w: torch.Tensor):
    rows, cols = w.shape
    pr, pc = -(-rows // GROUP) * GROUP, -(-cols // GROUP) * GROUP
    wf = torch.zeros(pr, pc, dtype=torch.float32, device=w.device)
    wf[:rows, :cols] = w.to(torch.bfloat16).float()
    t = wf.view(pr // GROUP, GROUP, pc // GROUP, GROUP)
    e = _round_up_exponent(t.abs().amax(dim=(1, 3)))
    q = (t * _inv_scale(e)[:, None, :, None]).clamp(-448.0, 448.0).to(FP8)
    return q.view(pr, pc)[:rows, :cols].contiguous(), e


def mx_quantize_weight(w: torch.Tensor, out_q: torch.Tensor | None = None, out_e: torch.Tensor | None = None):
    """bf16 ``[rows, cols]`` -> (e4m3 ``[rows, cols]``, uint8 tile exponents ``[ceil(r/32), ceil(c/32)]``)."""
    rows, cols = w.shape
    if not w.is_cuda:
        q, e = mx_quantize_weight_ref(w)
        if out_q is not None:
            out_q.view(torch.uint8).copy_(q.view(torch.uint8))
            out_e.copy_(e)
            return out_q, out_e
        return q, e
    _ensure()
    w = w if (w.dtype == torch.bfloat16 and w.stride(1) == 1) else w.to(torch.bfloat16).contiguous()
    q = out_q if out_q is not None else torch.empty(rows, cols, dtype=FP8, device=w.device)
    e = out_e if out_e is not None else torch.empty(-(-rows // GROUP), -(-cols // GROUP), dtype=torch.uint8,
                                                    device=w.device)
    rc = _lib.load().fsb_mx_quant_weight(w.data_ptr(), q.data_ptr(), e.data_ptr(), rows, cols, w.stride(0),
                                         q.stride(0), _lib.stream_ptr(w.device))
    _lib.check(rc, "fsb_mx_quant_weight")
    count_launch()
    return q, e


def mx_expand_scales(tile_exp: torch.Tensor, rows: int, cols: int, transpose: bool = False) -> torch.Tensor:
    """Blocked scales of the weight ``[rows, cols]`` (``transpose=False``: the forward operand) or of
    its transpose ``[cols, rows]`` (the input-gradient operand) from the 32x32 tile exponents."""
    if not tile_exp.is_cuda:
        if transpose:
            logical = tile_exp.t().repeat_interleave(GROUP, 0)[:cols]
        else:
            logical = tile_exp.repeat_interleave(GROUP, 0)[:rows]
        return to_blocked(logical.contiguous())
    _ensure()
    n = blocked_scale_numel(cols, rows) if transpose else blocked_scale_numel(rows, cols)
    out = torch.empty(n, dtype=torch.uint8, device=tile_exp.device)
    rc = _lib.load().fsb_mx_expand_scales(tile_exp.data_ptr(), out.data_ptr(), rows, cols, int(transpose),
                                          _lib.stream_ptr(tile_exp.device))
    _lib.check(rc, "fsb_mx_expand_scales")
    count_launch()
    return out


def mx_quantize_act_ref(x: torch.Tensor):
    T, K = x.shape
    g = x.to(torch.bfloat16).float().view(T, K // GROUP, GROUP)
    e = _round_up_exponent(g.abs().amax(-1))
    q = (g * _inv_scale(e)[..., None]).clamp(-448.0, 448.0).to(FP8).view(T, K)
    return q, to_blocked(e)


def mx_quantize_act(x: torch.Tensor):
    """bf16 ``[T, K]`` (K a multiple of 128) -> (e4m3 ``[T, K]``, blocked uint8 scales)."""
    T, K = x.shape
    if K % 128:
        raise ValueError("the contraction length must be a multiple of 128")
    if not x.is_cuda:
        return mx_quantize_act_ref(x)
    _ensure()
    x = x if (x.dtype == torch.bfloat16 and x.stride(1) == 1) else x.to(torch.bfloat16).contiguous()
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.full((blocked_scale_numel(T, K),), 127, dtype=torch.uint8, device=x.device) if T % 128 else \
        torch.empty(blocked_scale_numel(T, K), dtype=torch.uint8, device=x.device)
    rc = _lib.load().fsb_mx_quant_act(x.data_ptr(), q.data_ptr(), s.data_ptr(), T, K, x.stride(0), q.stride(0),
                                      _lib.stream_ptr(x.device))
    _lib.check(rc, "fsb_mx_quant_act")
    count_launch()
    return q, s


def mx_quantize_rows(x: torch.Tensor):
    """bf16 ``[T, K]`` (T and K multiples of 128) quantised in 32x1 groups (32 consecutive rows of a
    column share a scale), for products that contract over the rows. Returns (e4m3 ``[T, K]`` in the
    same layout, blocked scales of the operand ``x^T``: ``[K rows, T/32 groups]``)."""
    T, K = x.shape
    if T % 128 or K % 128:
        raise ValueError("both dims must be multiples of 128")
    if not x.is_cuda:
        q, s = mx_quantize_act_ref(x.t().contiguous())
        return q.t().contiguous(), s
    _ensure()
    x = x if (x.dtype == torch.bfloat16 and x.stride(1) == 1) else x.to(torch.bfloat16).contiguous()
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.empty(blocked_scale_numel(K, T), dtype=torch.uint8, device=x.device)
    rc = _lib.load().fsb_mx_quant_rows(x.data_ptr(), q.data_ptr(), s.data_ptr(), T, K, x.stride(0), q.stride(0),
                                       _lib.stream_ptr(x.device))
    _lib.check(rc, "fsb_mx_quant_rows")
    count_launch()
    return q, s


def mx_dequantize(q: torch.Tensor, blocked: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Row-major e4m3 ``[rows, cols]`` with blocked scales whose groups run along the columns."""
    rows, cols = q.shape
    e = from_blocked(blocked, rows, -(-cols // GROUP))
    s = torch.exp2(e.float() - 127.0).repeat_interleave(GROUP, 1)[:, :cols]
    return (q.float() * s).to(dtype)


# --------------------------------------------------------------------------- GEMM
def gemm_mxfp8(aq, sfa, bq, sfb, *, a_t: bool = False, b_t: bool = False, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``out[M, N] = (Aq * 2^sfa) . (Bq * 2^sfb)^T``. ``aq``: e4m3 ``[M, K]`` or, with ``a_t``, stored
    ``[K, M]``; ``bq``: e4m3 ``[N, K]`` or, with ``b_t``, stored ``[K, N]``. ``sfa`` / ``sfb``: blocked
    scales of the operands as the product sees them (``[M, K]`` and ``[N, K]``, groups along K)."""
    M, K = (aq.shape[1], aq.shape[0]) if a_t else aq.shape
    N = bq.shape[1] if b_t else bq.shape[0]
    if not aq.is_cuda:
        al = aq.float().t() if a_t else aq.float()
        ea = from_blocked(sfa, M, K // GROUP)
        a = al * torch.exp2(ea.float() - 127.0).repeat_interleave(GROUP, 1)[:, :K]
        bl = bq.float().t() if b_t else bq.float()
        e = from_blocked(sfb, N, K // GROUP)
        b = bl * torch.exp2(e.float() - 127.0).repeat_interleave(GROUP, 1)[:, :K]
        return (a @ b.t()).to(out_dtype)
    _ensure()
    out = torch.empty(M, N, dtype=out_dtype, device=aq.device)
    status = _lib.status_word(aq.device)
    rc = _lib.load().fsb_gemm_mxfp8(aq.data_ptr(), sfa.data_ptr(), bq.data_ptr(), sfb.data_ptr(), out.data_ptr(),
                                    M, N, K, aq.stride(0), bq.stride(0), out.stride(0), int(a_t), int(b_t),
                                    int(out_dtype == torch.float32), status.data_ptr(), _lib.stream_ptr(aq.device))
    _lib.check(rc, "fsb_gemm_mxfp8")
    count_launch()
    return out


class _Mxfp8Linear(torch.autograd.Function):
    """y = x W^T with W given as (e4m3 data, forward-orientation scales, input-gradient-orientation
    scales); ``weight`` is the logical high-precision parameter that receives the weight gradient
    (a bf16 tcgen05 GEMM written in the parameter's gradient dtype)."""

    @staticmethod
    def forward(ctx, x, weight, wq, fwd_scale, dgrad_scale):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, wq, dgrad_scale)
        ctx.xshape = x.shape
        ctx.weight = weight
        xq, sx = mx_quantize_act(x2)
        y = gemm_mxfp8(xq, sx, wq, fwd_scale)
        return y.view(*x.shape[:-1], wq.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wq, dgrad_scale = ctx.saved_tensors
        weight = ctx.weight
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = mx_quantize_act(dy2)
            dx = gemm_mxfp8(dyq, sdy, wq, dgrad_scale, b_t=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            gd = getattr(weight, "grad_dtype", None) or torch.bfloat16
            gd = gd if gd in (torch.bfloat16, torch.float32) else torch.bfloat16
            if main is not None and main.dtype in (torch.float32, torch.bfloat16):
                gemm(dy2, x2, a_t=True, b_t=True, out=main,
                     accumulate=bool(getattr(weight, "main_grad_written", False)))
                weight.main_grad_written = True
            elif MX_WGRAD and dy2.shape[0] % 128 == 0 and dy2.shape[1] % 128 == 0 and x2.shape[1] % 128 == 0:
                # third block-scaled product: dW = dy^T x, both operands quantised in 32x1 groups along
                # the tokens (the contraction) and read transposed by the tensor core
                dq, sd = mx_quantize_rows(dy2)
                xq, sx = mx_quantize_rows(x2)
                dw = gemm_mxfp8(dq, sd, xq, sx, a_t=True, b_t=True, out_dtype=gd)
            else:
                dw = gemm(dy2, x2, a_t=True, b_t=True, out_dtype=gd)
        return dx, dw, None, None, None


def mxfp8_linear(x, weight, wq, fwd_scale, dgrad_scale):
    return _Mxfp8Linear.apply(x, weight, wq, fwd_scale, dgrad_scale)
