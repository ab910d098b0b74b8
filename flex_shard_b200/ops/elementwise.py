"""RMSNorm, RoPE, SwiGLU, fused cross-entropy, AdamW and cast kernels with autograd wrappers.

CUDA tensors run the sm_100a kernels of ``csrc/elementwise.cu``; CPU tensors take
a PyTorch reference path with the same numerics contract (fp32 math, bf16
storage), which the CPU test-suite and the GPU numerics tests both use.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from ._lib import count_launch


def _s(dev):
    return _lib.stream_ptr(dev)


# --------------------------------------------------------------------------- RMSNorm
def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype), rstd.squeeze(-1)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        T = x2.shape[0]
        if x.is_cuda:
            x2 = x2.contiguous()
            y = torch.empty_like(x2)
            rstd = torch.empty(T, dtype=torch.float32, device=x.device)
            w = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
            if residual is not None:
                r2 = residual.reshape(-1, D).contiguous()
                s = torch.empty_like(x2)
            else:
                r2, s = None, None
            rc = _lib.load().fsb_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr() if r2 is not None else None,
                                             w.data_ptr(), y.data_ptr(),
                                             s.data_ptr() if s is not None else None, rstd.data_ptr(),
                                             T, D, eps, _s(x.device))
            _lib.check(rc, "fsb_rmsnorm_fwd")
            count_launch()
            normed_in = s if s is not None else x2
        else:
            normed_in = x2 if residual is None else (x2.float() + residual.reshape(-1, D).float()).to(x.dtype)
            y, rstd = _rmsnorm_ref(normed_in, weight, eps)
            s = normed_in if residual is not None else None
        ctx.save_for_backward(normed_in, weight, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is not None:
            ctx.mark_non_differentiable()
            return y.view(x.shape), s.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dsum):
        xin, weight, rstd = ctx.saved_tensors
        D = xin.shape[-1]
        T = xin.shape[0]
        dy2 = dy.reshape(-1, D)
        dres = dsum.reshape(-1, D) if (ctx.has_res and dsum is not None) else None
        if xin.is_cuda:
            dy2 = dy2.contiguous()
            dres = dres.contiguous() if dres is not None else None
            dx = torch.empty_like(xin)
            nblk = (T + 31) // 32
            partial = torch.empty(nblk, D, dtype=torch.float32, device=xin.device)
            w = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
            main = getattr(weight, "main_grad", None)
            use_main = main is not None and main.dtype == torch.float32 and main.dim() == 1 and main.is_contiguous()
            if use_main:
                dw_buf, dw_fp32, acc = main, 1, int(bool(getattr(weight, "main_grad_written", False)))
            else:
                dw_buf = torch.empty(D, dtype=torch.float32, device=xin.device)
                dw_fp32, acc = 1, 0
            rc = _lib.load().fsb_rmsnorm_bwd(dy2.data_ptr(), xin.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                             dres.data_ptr() if dres is not None else None, dx.data_ptr(),
                                             partial.data_ptr(), dw_buf.data_ptr(), dw_fp32, acc, T, D,
                                             _s(xin.device))
            _lib.check(rc, "fsb_rmsnorm_bwd")
            count_launch(2)
            if use_main:
                weight.main_grad_written = True
                dw = None
            else:
                dw = dw_buf.to(weight.dtype)
        else:
            xf, dyf, wf = xin.float(), dy2.float(), weight.float()
            r = rstd.unsqueeze(-1)
            xhat = xf * r
            dyw = dyf * wf
            dxf = r * (dyw - xhat * (dyw * xhat).mean(-1, keepdim=True))
            if dres is not None:
                dxf = dxf + dres.float()
            dx = dxf.to(xin.dtype)
            dw = (dyf * xhat).sum(0).to(weight.dtype)
        dx = dx.view(ctx.shape)
        return dx, dw, None, (dx if ctx.has_res else None)


def rmsnorm(x, weight, eps: float = 1e-5):
    return _RMSNorm.apply(x, weight, eps, None)[0]


def add_rmsnorm(x, residual, weight, eps: float = 1e-5):
    """Returns ``(rmsnorm(x + residual), x + residual)`` from one pass over the data."""
    y, s = _RMSNorm.apply(x, weight, eps, residual)
    return y, s


# --------------------------------------------------------------------------- RoPE
def rope_table(seq_len: int, head_dim: int, theta: float, device, yarn: dict | None = None) -> torch.Tensor:
    """[S, hd/2, 2] fp32 table of (cos, sin) for interleaved-pair rotation.

    ``yarn`` = ``dict(factor, original_seq_len, beta_fast=32, beta_slow=1)`` stretches the context the
    YaRN way: pairs that complete fewer than ``beta_slow`` turns over the original context have their
    frequency divided by ``factor`` (interpolation), pairs with more than ``beta_fast`` turns keep it,
    and a linear ramp over the pair index blends the two in between (parity: the rotary cache of the
    reference's DeepSeek-V3 example, ``examples/deepseek_v3/model.py:88-109``)."""
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv = 1.0 / (theta ** (idx / head_dim))
    if yarn is not None and float(yarn.get("factor", 1.0)) != 1.0:
        factor, orig = float(yarn["factor"]), float(yarn["original_seq_len"])

        def pair_with_turns(turns: float) -> float:   # pair index whose wavelength gives `turns` turns over `orig`
            return head_dim * math.log(orig / (turns * 2 * math.pi)) / (2 * math.log(theta))

        lo = max(math.floor(pair_with_turns(float(yarn.get("beta_fast", 32.0)))), 0)
        hi = min(math.ceil(pair_with_turns(float(yarn.get("beta_slow", 1.0)))), head_dim - 1)
        span = (hi - lo) if hi != lo else 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float32, device=device) - lo) / span).clamp(0, 1)
        inv = inv / factor * ramp + inv * (1 - ramp)
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()


def yarn_attention_scale(head_dim: int, factor: float, mscale: float = 0.70) -> float:
    """Softmax scale that goes with a YaRN-stretched context: ``head_dim**-0.5 * m**2`` with
    ``m = 0.1 * mscale * ln(factor) + 1``."""
    m = 0.1 * mscale * math.log(factor) + 1.0 if factor > 1.0 else 1.0
    return head_dim ** -0.5 * m * m


def _rope_ref(x, table, inverse):
    # x: [B, S, H, hd]
    S = x.shape[1]
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c = table[:S, :, 0].view(1, S, 1, -1)
    s = table[:S, :, 1].view(1, S, 1, -1)
    if inverse:
        s = -s
    o = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c], dim=-1)
    return o.reshape(x.shape).to(x.dtype)


def _rope_inplace(x, table, inverse: bool):
    """x: [B, S, H, hd] view whose last two dims are dense; rotates in place on CUDA."""
    B, S, H, hd = x.shape
    assert x.stride(3) == 1 and x.stride(2) == hd and x.stride(0) == S * x.stride(1)
    rc = _lib.load().fsb_rope(x.data_ptr(), table.data_ptr(), B * S, S, H, hd, x.stride(1), int(inverse),
                              _s(x.device))
    _lib.check(rc, "fsb_rope")
    count_launch()
    return x


class _RoPE(torch.autograd.Function):
    """Rotates in place (the input is a fresh projection output that nothing else reads)."""

    @staticmethod
    def forward(ctx, x, table):
        ctx.save_for_backward(table)
        if x.is_cuda:
            ctx.mark_dirty(x)
            return _rope_inplace(x, table, False)
        return _rope_ref(x, table, False)

    @staticmethod
    def backward(ctx, dy):
        (table,) = ctx.saved_tensors
        if dy.is_cuda:
            # Rotate a private copy: the incoming gradient may be shared with other consumers.
            return _rope_inplace(dy.contiguous().clone(), table, True), None
        return _rope_ref(dy, table, True), None


def rope(x, table):
    """Apply rotary embedding to ``x`` of shape [B, S, H, hd] (in place on CUDA)."""
    return _RoPE.apply(x, table)


# --------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        F = F2 // 2
        g2 = gu.reshape(-1, F2)
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        if gu.is_cuda:
            g2 = g2.contiguous()
            h = torch.empty(g2.shape[0], F, dtype=gu.dtype, device=gu.device)
            rc = _lib.load().fsb_swiglu_fwd(g2.data_ptr(), h.data_ptr(), g2.shape[0], F, _s(gu.device))
            _lib.check(rc, "fsb_swiglu_fwd")
            count_launch()
        else:
            gf = g2.float()
            h = (torch.nn.functional.silu(gf[:, :F]) * gf[:, F:]).to(gu.dtype)
        return h.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dh):
        (g2,) = ctx.saved_tensors
        F = g2.shape[1] // 2
        dh2 = dh.reshape(-1, F)
        if g2.is_cuda:
            dh2 = dh2.contiguous()
            dgu = torch.empty_like(g2)
            rc = _lib.load().fsb_swiglu_bwd(g2.data_ptr(), dh2.data_ptr(), dgu.data_ptr(), g2.shape[0], F,
                                            _s(g2.device))
            _lib.check(rc, "fsb_swiglu_bwd")
            count_launch()
        else:
            gf, d = g2.float(), dh2.float()
            g, u = gf[:, :F], gf[:, F:]
            sg = torch.sigmoid(g)
            silu = g * sg
            dgu = torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], dim=1).to(g2.dtype)
        return dgu.view(ctx.shape)


def swiglu(gate_up):
    """``silu(gate) * up`` for ``gate_up = [..., 2F]`` with gate in the first half."""
    return _SwiGLU.apply(gate_up)


# --------------------------------------------------------------------------- cross entropy
class _CrossEntropy(torch.autograd.Function):
    """Mean (or scaled-sum) token cross-entropy; the backward pass is produced by the forward
    kernel in place of the logits, so the fp32 softmax never exists in memory."""

    @staticmethod
    def forward(ctx, logits, target, scale, ignore_index, unit_grad):
        ctx.unit_grad = unit_grad
        T, V = logits.shape
        if logits.is_cuda:
            assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
            loss = torch.empty(T, dtype=torch.float32, device=logits.device)
            rc = _lib.load().fsb_cross_entropy(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), T, V,
                                               logits.stride(0), scale, ignore_index, _s(logits.device))
            _lib.check(rc, "fsb_cross_entropy")
            count_launch()
            ctx.save_for_backward(logits)
            return loss.sum() * scale
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = target != ignore_index
        tsafe = target.clamp_min(0)
        loss = (lse - lf.gather(1, tsafe[:, None]).squeeze(1)) * valid
        p = torch.softmax(lf, dim=-1)
        p[torch.arange(T), tsafe] -= 1.0
        p = p * valid[:, None] * scale
        ctx.save_for_backward(p.to(logits.dtype))
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        if ctx.unit_grad:
            return dlogits, None, None, None, None
        return dlogits * dloss.to(dlogits.dtype), None, None, None, None


def cross_entropy(logits, target, scale: float | None = None, ignore_index: int = -100,
                  unit_grad: bool = False):
    """``sum(token losses) * scale`` (default scale ``1/T``). Overwrites ``logits`` on CUDA.
    ``unit_grad=True`` promises that the gradient flowing into the loss is exactly 1 (the loss
    is the root of ``backward()``), which skips one multiply pass over the logits."""
    if scale is None:
        scale = 1.0 / logits.shape[0]
    return _CrossEntropy.apply(logits, target, float(scale), ignore_index, bool(unit_grad))


# --------------------------------------------------------------------------- AdamW / casts
def adamw_step_(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, lowp_out=None):
    """One AdamW update over flat tensors (``p`` fp32 or bf16, ``g`` fp32 or bf16, ``m``/``v`` fp32)."""
    n = p.numel()
    if n == 0:
        return
    if m.dtype != torch.float32 or v.dtype != torch.float32 or m.numel() < n or v.numel() < n or g.numel() < n:
        raise ValueError(f"AdamW moments must be fp32 with at least {n} elements (got {m.dtype}[{m.numel()}], "
                         f"{v.dtype}[{v.numel()}]; gradient has {g.numel()})")
    if p.is_cuda:
        assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
        rc = _lib.load().fsb_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                   lowp_out.data_ptr() if lowp_out is not None else None, n,
                                   int(p.dtype == torch.float32), int(g.dtype == torch.float32),
                                   lr, beta1, beta2, eps, weight_decay, step, grad_scale, _s(p.device))
        _lib.check(rc, "fsb_adamw")
        count_launch()
        return
    gf = g.float() * grad_scale
    pf = p.float() * (1 - lr * weight_decay)
    m.lerp_(gf, 1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    b1 = 1 - beta1 ** step
    b2s = math.sqrt(1 - beta2 ** step)
    pf = pf - (lr / b1) * (m / (v.sqrt() / b2s + eps))
    p.copy_(pf)
    if lowp_out is not None:
        lowp_out.copy_(pf)


_CAST_MODES = {(torch.float32, torch.bfloat16): 1, (torch.bfloat16, torch.float32): 2,
               (torch.float32, torch.float32): 4, (torch.bfloat16, torch.bfloat16): 5}


def cast_scale_(dst, src, scale: float = 1.0, accumulate: bool = False):
    """``dst = (dst +) src * scale`` across fp32/bf16, flat and contiguous."""
    if src.is_cuda and (src.dtype, dst.dtype) in _CAST_MODES and src.is_contiguous() and dst.is_contiguous():
        rc = _lib.load().fsb_cast_scale(src.data_ptr(), dst.data_ptr(), src.numel(),
                                        _CAST_MODES[(src.dtype, dst.dtype)], scale, int(accumulate),
                                        _s(src.device))
        _lib.check(rc, "fsb_cast_scale")
        count_launch()
        return dst
    r = src.float() * scale
    if accumulate:
        r = r + dst.float()
    dst.copy_(r)
    return dst
