"""Causal flash attention (head_dim 128, GQA) on the tcgen05 kernels, with RoPE folded in.

``qkv_attention(qkv, rope_table, Hq, Hkv)`` takes the fused projection output
``[B, S, (Hq + 2*Hkv) * 128]``, rotates the q and k slices in place, runs the
attention kernel on the three column slices and returns ``[B, S, Hq * 128]``.
Its backward writes dq/dk/dv straight into one ``dqkv`` buffer of the same fused
layout (no concatenation) and un-rotates dq/dk in place.

CPU tensors take an fp32 PyTorch reference path.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .elementwise import _rope_inplace, _rope_ref
from ._lib import count_launch

HD = 128


def _declare():
    import ctypes as c

    vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    _lib.declare("fsb_attn_fwd", [vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, f32, vp, vp])
    _lib.declare("fsb_attn_bwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32,
                                  i64, i64, i64, i64, i64, i64, i64, f32, vp, vp])
    _lib.declare("fsb_cast2d_f32_bf16", [vp, vp, i64, i32, i64, i64, vp])


_declared = False
_deterministic: bool | None = None


def set_deterministic(enabled: bool | None) -> None:
    """Ordered accumulation of dQ in the backward kernel (the same bits on every run) on / off; ``None``
    returns to the default: on when ``torch.use_deterministic_algorithms(True)`` is set or the environment
    variable ``FSB200_DETERMINISTIC`` is ``1``."""
    global _deterministic
    _deterministic = enabled


def _heads_inner(ordered: bool) -> int:
    """Walk order of the backward kernel's (query tile, head) pairs: query tiles from the last one down with the
    heads of a group inside. The ordered mode needs it (each CTA then stays one hand-over behind its predecessor:
    1.21 ms against 1.65 ms head by head at S 8192, 16q/4kv) and the unordered kernel is no slower with it
    (0.863 against 0.870 ms: the CTAs of a kv head read the same query tiles at about the same time).
    ``FSB200_ATTN_BWD_WALK`` = ``tiles`` / ``heads`` overrides it for measurements."""
    import os

    walk = os.environ.get("FSB200_ATTN_BWD_WALK", "")
    if walk in ("tiles", "heads"):
        return int(walk == "tiles")
    return 1


def is_deterministic() -> bool:
    if _deterministic is not None:
        return _deterministic
    import os

    return os.environ.get("FSB200_DETERMINISTIC", "0") == "1" or torch.are_deterministic_algorithms_enabled()


def _ensure():
    global _declared
    if not _declared:
        _declare()
        _declared = True


def attention_ref(q, k, v, scale=None):
    """fp32 reference: q [B,S,Hq,D], k/v [B,S,Hkv,D] -> [B,S,Hq,D]."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale or 1.0 / math.sqrt(D)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    att = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    att = att.masked_fill(~mask, float("-inf")).softmax(-1)
    return (att @ vf).transpose(1, 2)


def attn_fwd_raw(q, k, v, o, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale):
    _ensure()
    status = _lib.status_word(o.device)
    rc = _lib.load().fsb_attn_fwd(q, k, v, o.data_ptr(), lse.data_ptr(), B, S, Hq, Hkv, ldq, ldk, ldv, ldo,
                                  scale, status.data_ptr(), _lib.stream_ptr(o.device))
    _lib.check(rc, "fsb_attn_fwd")
    count_launch()


class _QKVAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, rope_table, Hq, Hkv):
        B, S, C = qkv.shape
        assert C == (Hq + 2 * Hkv) * HD
        scale = 1.0 / math.sqrt(HD)
        if not qkv.is_cuda:
            q = qkv[..., : Hq * HD].reshape(B, S, Hq, HD)
            k = qkv[..., Hq * HD: (Hq + Hkv) * HD].reshape(B, S, Hkv, HD)
            v = qkv[..., (Hq + Hkv) * HD:].reshape(B, S, Hkv, HD)
            if rope_table is not None:
                q, k = _rope_ref(q, rope_table, False), _rope_ref(k, rope_table, False)
            with torch.enable_grad():
                qd, kd, vd = (t.detach().float().requires_grad_() for t in (q, k, v))
                o = attention_ref(qd, kd, vd, scale)
            ctx.cpu = (qd, kd, vd, o)
            ctx.save_for_backward(rope_table)
            ctx.dims = (B, S, Hq, Hkv)
            return o.detach().to(qkv.dtype).reshape(B, S, Hq * HD)
        assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous()
        q = qkv[..., : Hq * HD].view(B, S, Hq, HD)
        k = qkv[..., Hq * HD: (Hq + Hkv) * HD].view(B, S, Hkv, HD)
        if rope_table is not None:
            _rope_inplace(q, rope_table, False)
            _rope_inplace(k, rope_table, False)
        o = torch.empty(B, S, Hq * HD, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
        base = qkv.data_ptr()
        attn_fwd_raw(base, base + Hq * HD * 2, base + (Hq + Hkv) * HD * 2, o, lse, B, S, Hq, Hkv,
                     C, C, C, Hq * HD, scale)
        ctx.save_for_backward(qkv, o, lse, rope_table)
        ctx.dims = (B, S, Hq, Hkv)
        ctx.cpu = None
        return o

    @staticmethod
    def backward(ctx, d_o):
        B, S, Hq, Hkv = ctx.dims
        scale = 1.0 / math.sqrt(HD)
        if ctx.cpu is not None:
            (rope_table,) = ctx.saved_tensors
            qd, kd, vd, o = ctx.cpu
            dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), d_o.float().reshape(B, S, Hq, HD))
            if rope_table is not None:
                dq, dk = _rope_ref(dq, rope_table, True), _rope_ref(dk, rope_table, True)
            dqkv = torch.cat([dq.reshape(B, S, -1), dk.reshape(B, S, -1), dv.reshape(B, S, -1)], dim=-1)
            return dqkv.to(d_o.dtype), None, None, None
        _ensure()
        qkv, o, lse, rope_table = ctx.saved_tensors
        C = qkv.shape[-1]
        d_o = d_o.contiguous()
        dev = qkv.device
        dqkv = torch.empty_like(qkv)
        # the fp32 dQ accumulator and, in ordered mode, the turn counters behind it: one zero-fill
        n_acc = B * S * Hq * HD
        n_turns = B * Hq * (S // 64) + 1 if is_deterministic() else 0
        zeroed = torch.zeros(n_acc + n_turns, dtype=torch.float32, device=dev)
        dq_acc = zeroed[:n_acc]
        turns = zeroed.data_ptr() + n_acc * 4 if n_turns else None
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device=dev)
        base, dbase = qkv.data_ptr(), dqkv.data_ptr()
        status = _lib.status_word(dev)
        lib = _lib.load()
        rc = lib.fsb_attn_bwd(base, base + Hq * HD * 2, base + (Hq + Hkv) * HD * 2, o.data_ptr(),
                              d_o.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), turns, _heads_inner(n_turns > 0),
                              dbase + Hq * HD * 2, dbase + (Hq + Hkv) * HD * 2, B, S, Hq, Hkv,
                              C, C, C, Hq * HD, Hq * HD, C, C, scale, status.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "fsb_attn_bwd")
        rc = lib.fsb_cast2d_f32_bf16(dq_acc.data_ptr(), dbase, B * S, Hq * HD, Hq * HD, C, _lib.stream_ptr(dev))
        _lib.check(rc, "fsb_cast2d_f32_bf16")
        count_launch(4)
        if rope_table is not None:
            _rope_inplace(dqkv[..., : Hq * HD].view(B, S, Hq, HD), rope_table, True)
            _rope_inplace(dqkv[..., Hq * HD: (Hq + Hkv) * HD].view(B, S, Hkv, HD), rope_table, True)
        return dqkv, None, None, None


def qkv_attention(qkv, rope_table, n_heads: int, n_kv_heads: int):
    """Fused RoPE + causal GQA attention over a fused QKV projection (modified in place on CUDA)."""
    return _QKVAttention.apply(qkv, rope_table, n_heads, n_kv_heads)
