"""Mixture-of-experts building blocks: routing plan on the device, row dispatch/combine kernels and
grouped tcgen05 GEMMs over an expert-major, 128-row-aligned token layout.

Nothing here synchronises with the host: the per-expert counts, padded offsets and the tile ->
expert table all stay in device memory and the grouped GEMM reads them there (the reference's
dispatcher copies split sizes to the CPU, ``examples/deepseek_v3/expert_parallel.py:82-89``).
CPU tensors take PyTorch reference paths with the same layout.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import count_launch

ALIGN = 128
_declared = False


def _ensure():
    global _declared
    if not _declared:
        c = ctypes
        vp, i32, i64 = c.c_void_p, c.c_int, c.c_longlong
        _lib.declare("fsb_moe_gather_rows", [vp, vp, vp, vp, i64, i32, i64, i64, vp])
        _lib.declare("fsb_moe_combine_rows", [vp, vp, vp, vp, i64, i32, i32, i64, i64, vp])
        _lib.declare("fsb_moe_combine_bwd_w", [vp, vp, vp, vp, i64, i32, i32, i64, i64, vp])
        _lib.declare("fsb_gemm_bf16_grouped", [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, i32, i32,
                                               vp, vp, vp, i32, vp, vp])
        _lib.declare("fsb_route_topk", [vp, vp, i64, i32, i32, i32, i32, c.c_float, vp, vp, vp, vp])
        _lib.declare("fsb_moe_plan_routes", [vp, i32, i64, i32, i32, i64, vp, vp, vp, vp, vp, vp, vp])
        _declared = True


@dataclass
class RoutePlan:
    """Device-resident description of one routing decision.

    ``pos[t, k]``: row of (token t, choice k) in the expert-major layout; ``src[r]``: token of row r
    (-1 for padding rows); ``offs[e]``: first row of expert e (multiple of 128, ``offs[E]`` = rows in
    use); ``tile_expert[m]``: expert of m-tile m; ``num_mtiles``: valid m-tiles; ``max_rows``: static
    upper bound the buffers are sized for."""

    pos: torch.Tensor
    src: torch.Tensor
    offs: torch.Tensor
    tile_expert: torch.Tensor
    num_mtiles: torch.Tensor
    max_rows: int
    num_experts: int
    counts: torch.Tensor | None = None     # pairs per expert (int32 [E]); filled by the planning kernel


def max_rows_for(num_pairs: int, num_experts: int) -> int:
    """Rows of the padded expert-major layout in the worst case (every expert's block rounded up to 128)."""
    return (num_pairs + num_experts * (ALIGN - 1) + ALIGN - 1) // ALIGN * ALIGN


def plan_routes_reference(expert_idx: torch.Tensor, num_experts: int) -> RoutePlan:
    """The same plan computed with PyTorch operators (CPU path and oracle of the kernel)."""
    if expert_idx.is_cuda:
        cpu = plan_routes(expert_idx.cpu(), num_experts)
        dev = expert_idx.device
        return RoutePlan(cpu.pos.to(dev), cpu.src.to(dev), cpu.offs.to(dev), cpu.tile_expert.to(dev),
                         cpu.num_mtiles.to(dev), cpu.max_rows, cpu.num_experts)
    return plan_routes(expert_idx, num_experts)


def plan_routes(expert_idx: torch.Tensor, num_experts: int) -> RoutePlan:
    """Stable expert-major ordering of the (token, choice) pairs, every expert's block padded to 128 rows."""
    T, k = expert_idx.shape
    dev = expert_idx.device
    n = expert_idx.numel()
    max_rows = (n + num_experts * (ALIGN - 1) + ALIGN - 1) // ALIGN * ALIGN
    if expert_idx.is_cuda and num_experts <= 256 and expert_idx.dtype in (torch.int64, torch.int32):
        # one launch: histogram, padded prefix sums, tile table and the row of every pair (stable within an expert)
        _ensure()
        idx = expert_idx.contiguous()
        pos = torch.empty(T, k, dtype=torch.int32, device=dev)
        src = torch.empty(max_rows, dtype=torch.int32, device=dev)
        offs = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(max_rows // ALIGN, dtype=torch.int32, device=dev)
        num_mtiles = torch.empty(1, dtype=torch.int32, device=dev)
        counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
        rc = _lib.load().fsb_moe_plan_routes(idx.data_ptr(), int(idx.dtype == torch.int64), n, k, num_experts, max_rows,
                                             pos.data_ptr(), src.data_ptr(), offs.data_ptr(), tile_expert.data_ptr(),
                                             num_mtiles.data_ptr(), counts.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "fsb_moe_plan_routes")
        count_launch()
        return RoutePlan(pos, src, offs, tile_expert, num_mtiles, max_rows, num_experts, counts)
    flat = expert_idx.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + ALIGN - 1) // ALIGN * ALIGN
    offs = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    offs[1:] = torch.cumsum(padded, 0)
    starts = torch.cumsum(counts, 0) - counts
    sorted_e = flat[order]
    rank_in = torch.arange(n, device=dev) - starts[sorted_e]
    rows = offs[sorted_e] + rank_in
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    pos[order] = rows.to(torch.int32)
    src = torch.full((max_rows,), -1, dtype=torch.int32, device=dev)
    src[rows] = (order // k).to(torch.int32)
    tiles = torch.arange(max_rows // ALIGN, device=dev)
    tile_expert = torch.searchsorted(offs[1:] // ALIGN, tiles, right=True).clamp_max(num_experts - 1).to(torch.int32)
    num_mtiles = (offs[-1:] // ALIGN).to(torch.int32)
    return RoutePlan(pos.view(T, k), src, offs.to(torch.int32), tile_expert, num_mtiles, max_rows, num_experts,
                     counts.to(torch.int32))


# --------------------------------------------------------------------------- row movement
def _gather(src, index, scale, n, D):
    if not src.is_cuda:
        out = torch.zeros(n, D, dtype=src.dtype)
        valid = index >= 0
        rows = src[index[valid].long()].float()
        if scale is not None:
            rows = rows * scale[valid, None]
        out[valid] = rows.to(src.dtype)
        return out
    _ensure()
    out = torch.empty(n, D, dtype=src.dtype, device=src.device)
    rc = _lib.load().fsb_moe_gather_rows(src.data_ptr(), index.data_ptr(), scale.data_ptr() if scale is not None else None,
                                         out.data_ptr(), n, D, src.stride(0), out.stride(0), _lib.stream_ptr(src.device))
    _lib.check(rc, "fsb_moe_gather_rows")
    count_launch()
    return out


def _combine(rows, pos, w, T, k, D):
    if not rows.is_cuda:
        g = rows[pos.reshape(-1).long()].float().view(T, k, D)
        if w is not None:
            g = g * w[..., None]
        return g.sum(1).to(rows.dtype)
    _ensure()
    out = torch.empty(T, D, dtype=rows.dtype, device=rows.device)
    rc = _lib.load().fsb_moe_combine_rows(rows.data_ptr(), pos.data_ptr(), w.data_ptr() if w is not None else None,
                                          out.data_ptr(), T, k, D, rows.stride(0), out.stride(0),
                                          _lib.stream_ptr(rows.device))
    _lib.check(rc, "fsb_moe_combine_rows")
    count_launch()
    return out


class _Dispatch(torch.autograd.Function):
    """x [T, D] -> expert-major rows [max_rows, D] (padding rows are zero)."""

    @staticmethod
    def forward(ctx, x, plan: RoutePlan):
        ctx.plan = plan
        ctx.T = x.shape[0]
        return _gather(x.contiguous(), plan.src, None, plan.max_rows, x.shape[1])

    @staticmethod
    def backward(ctx, dxp):
        plan = ctx.plan
        T, k = plan.pos.shape
        return _combine(dxp.contiguous(), plan.pos, None, T, k, dxp.shape[1]), None


class _Combine(torch.autograd.Function):
    """y[t] = sum_k w[t, k] * rows[pos[t, k]]"""

    @staticmethod
    def forward(ctx, rows, w, plan: RoutePlan):
        T, k = plan.pos.shape
        rows = rows.contiguous()
        w = w.float().contiguous()
        ctx.save_for_backward(rows, w)
        ctx.plan = plan
        return _combine(rows, plan.pos, w, T, k, rows.shape[1])

    @staticmethod
    def backward(ctx, dy):
        rows, w = ctx.saved_tensors
        plan = ctx.plan
        T, k = plan.pos.shape
        D = rows.shape[1]
        dy = dy.contiguous()
        # row r = (t, k): scale[r] = w[t, k]; rows of padding get index -1
        scale = torch.zeros(plan.max_rows, dtype=torch.float32, device=dy.device)
        scale[plan.pos.reshape(-1).long()] = w.reshape(-1)
        drows = _gather(dy, plan.src, scale, plan.max_rows, D)
        if dy.is_cuda:
            _ensure()
            dw = torch.empty(T, k, dtype=torch.float32, device=dy.device)
            rc = _lib.load().fsb_moe_combine_bwd_w(dy.data_ptr(), rows.data_ptr(), plan.pos.data_ptr(), dw.data_ptr(),
                                                   T, k, D, dy.stride(0), rows.stride(0), _lib.stream_ptr(dy.device))
            _lib.check(rc, "fsb_moe_combine_bwd_w")
            count_launch()
        else:
            dw = (rows[plan.pos.reshape(-1).long()].float().view(T, k, D) * dy.float()[:, None, :]).sum(-1)
        return drows, dw, None


def moe_dispatch(x, plan):
    return _Dispatch.apply(x, plan)


def moe_combine(rows, weights, plan):
    return _Combine.apply(rows, weights, plan)


# --------------------------------------------------------------------------- grouped GEMMs
def _grouped(mode, a, b, out, plan: RoutePlan, E, M, N, K, b_mn, accumulate=False):
    _ensure()
    status = _lib.status_word(a.device)
    rc = _lib.load().fsb_gemm_bf16_grouped(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), mode, E, M, N, K, a.stride(0), b.stride(-2), out.stride(-2),
        int(b_mn), int(out.dtype == torch.float32), int(accumulate), plan.tile_expert.data_ptr(),
        plan.num_mtiles.data_ptr(), plan.offs.data_ptr(), plan.max_rows, status.data_ptr(),
        _lib.stream_ptr(a.device))
    _lib.check(rc, "fsb_gemm_bf16_grouped")
    count_launch()
    return out


class _GroupedLinear(torch.autograd.Function):
    """rows [R, K] x stacked weights [E, N, K] -> [R, N], each 128-row tile using its expert's slice."""

    @staticmethod
    def forward(ctx, x, weight, plan: RoutePlan):
        E, N, K = weight.shape
        ctx.save_for_backward(x, weight)
        ctx.plan = plan
        if not x.is_cuda:
            out = torch.zeros(plan.max_rows, N, dtype=x.dtype)
            offs = plan.offs.tolist()
            for e in range(E):
                a, b_ = offs[e], offs[e + 1]
                if b_ > a:
                    out[a:b_] = (x[a:b_].float() @ weight[e].float().t()).to(x.dtype)
            return out
        out = torch.empty(plan.max_rows, N, dtype=x.dtype, device=x.device)
        return _grouped(1, x, weight.view(E * N, K), out, plan, E, plan.max_rows, N, K, b_mn=False)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        plan = ctx.plan
        E, N, K = weight.shape
        dy = dy.contiguous()
        dx = dw = None
        if not x.is_cuda:
            offs = plan.offs.tolist()
            dx = torch.zeros_like(x)
            dw = torch.zeros_like(weight, dtype=torch.float32)
            for e in range(E):
                a, b_ = offs[e], offs[e + 1]
                if b_ > a:
                    dx[a:b_] = (dy[a:b_].float() @ weight[e].float()).to(x.dtype)
                    dw[e] = dy[a:b_].float().t() @ x[a:b_].float()
            return dx, dw.to(weight.dtype), None
        if ctx.needs_input_grad[0]:
            # dx[R, K] = dy[R, N] . W_e[N, K]: B read MN-major from the stacked [E*N, K] weight
            dx = torch.empty(plan.max_rows, K, dtype=x.dtype, device=x.device)
            _grouped(1, dy, weight.view(E * N, K), dx, plan, E, plan.max_rows, K, N, b_mn=True)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None and isinstance(main, torch.Tensor) and main.is_contiguous() \
                    and main.dtype in (torch.float32, torch.bfloat16) and main.shape == weight.shape:
                _grouped(2, dy, x, main.view(E * N, K), plan, E, N, K, plan.max_rows, b_mn=True,
                         accumulate=bool(getattr(weight, "main_grad_written", False)))
                weight.main_grad_written = True
            else:
                dw = torch.empty(E, N, K, dtype=weight.dtype, device=x.device)
                _grouped(2, dy, x, dw.view(E * N, K), plan, E, N, K, plan.max_rows, b_mn=True)
        return dx, dw, None


def grouped_linear(x_rows, weight, plan):
    """``x_rows`` in the expert-major layout of ``plan`` times the stacked ``weight [E, N, K]``."""
    return _GroupedLinear.apply(x_rows, weight, plan)


def _route_scores(logits, mode):
    return torch.sigmoid(logits) if mode == "sigmoid" else torch.softmax(logits, dim=-1)


class _RouteTopK(torch.autograd.Function):
    """Fused router: activation, biased top-k, weight normalisation, token histogram (one kernel on
    CUDA); the backward pass is a handful of [T, k] / [T, E] elementwise ops."""

    @staticmethod
    def forward(ctx, logits, bias, k, mode, scale, normalize, counts):
        T, E = logits.shape
        lg = logits.float().contiguous()
        if lg.is_cuda:
            _ensure()
            idx = torch.empty(T, k, dtype=torch.int64, device=lg.device)
            w = torch.empty(T, k, dtype=torch.float32, device=lg.device)
            b = bias.float().contiguous() if bias is not None else None
            if counts is not None and not (counts.dtype == torch.float32 and counts.is_contiguous()):
                raise ValueError("counts must be a contiguous fp32 tensor")
            rc = _lib.load().fsb_route_topk(lg.data_ptr(), b.data_ptr() if b is not None else None, T, E, k,
                                            int(mode == "softmax"), int(normalize), float(scale), idx.data_ptr(),
                                            w.data_ptr(), counts.data_ptr() if counts is not None else None,
                                            _lib.stream_ptr(lg.device))
            _lib.check(rc, "fsb_route_topk")
            count_launch(1)
        else:
            s = _route_scores(lg, mode)
            _, idx = (s + bias.float() if bias is not None else s).topk(k, dim=-1)
            sel = s.gather(1, idx)
            w = sel / (sel.sum(-1, keepdim=True) + 1e-20) * scale if normalize else sel * scale
            if counts is not None:
                counts += torch.bincount(idx.reshape(-1), minlength=E).to(counts.dtype)
        ctx.save_for_backward(lg, idx)
        ctx.cfg = (mode, float(scale), bool(normalize), logits.dtype)
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _didx, dw):
        lg, idx = ctx.saved_tensors
        mode, scale, normalize, in_dtype = ctx.cfg
        s = _route_scores(lg, mode)
        sel = s.gather(1, idx)
        dw = dw.float()
        if normalize:
            denom = sel.sum(-1, keepdim=True) + 1e-20
            dsel = scale * (dw / denom - (dw * sel).sum(-1, keepdim=True) / (denom * denom))
        else:
            dsel = scale * dw
        ds = torch.zeros_like(s).scatter_(1, idx, dsel)
        if mode == "sigmoid":
            dlogits = ds * s * (1 - s)
        else:
            dlogits = s * (ds - (ds * s).sum(-1, keepdim=True))
        return dlogits.to(in_dtype), None, None, None, None, None, None


def route_topk(logits, k, bias=None, mode="sigmoid", scale=1.0, normalize=True, counts=None):
    """Router decision for [T, E] logits: ``(idx [T, k] int64, weights [T, k] fp32)``.

    ``mode``: "sigmoid" (DeepSeek-V3 style; ``bias`` steers the selection only) or "softmax".
    ``normalize`` divides the selected scores by their sum; ``counts`` (fp32 [E]) is incremented
    by the number of tokens sent to each expert."""
    if mode not in ("sigmoid", "softmax"):
        raise ValueError(f"unknown router mode {mode!r}")
    return _RouteTopK.apply(logits, bias, k, mode, scale, normalize, counts)
