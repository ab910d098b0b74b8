"""Newton-Schulz orthogonalisation on the tcgen05 GEMM, with the polynomial fused in epilogues.

Per step (coefficients a, b, c), for ``X`` of shape ``[s, l]`` with ``s <= l``::

    A = X X^T                      one GEMM
    B = b*A + c*A@A                one GEMM, epilogue  c*acc + b*A
    X = a*X + B@X                  one GEMM, epilogue  acc + a*X

Tall matrices use ``A = X^T X`` and ``X = a*X + X@B`` instead, through the GEMM's transposed
operand modes, so no transpose copy is ever made. ``A`` and ``B`` are symmetric: their GEMMs compute the
tiles on or above the diagonal only and mirror them (28 % fewer FLOPs per iteration for a 4096 x 14336 matrix). Math parity with the reference's
``_zeropower_via_newtonschulz`` (``dist_muon/optimizer.py:2120-2151``): bf16 operands, fp32
accumulation, Frobenius normalisation first.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import count_launch
from .gemm import gemm

NS_COEFFS = (3.4445, -4.7750, 2.0315)
_declared = False


def _ensure():
    global _declared
    if not _declared:
        c = ctypes
        vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        _lib.declare("fsb_muon_prepare", [vp, vp, i32, vp, vp, i64, f32, i32, vp])
        _lib.declare("fsb_muon_scale", [vp, vp, i64, f32, vp])
        _lib.declare("fsb_muon_update", [vp, i32, vp, i64, f32, f32, vp])
        _lib.declare("fsb_muon_workspace_floats", [])
        _declared = True


def _workspace(device) -> torch.Tensor:
    """Zeroed scratch of the prepare kernel: [0] receives the sum of squares, the rest holds the per-block
    partial sums, which the last block adds in index order (the same bits on every run)."""
    return torch.zeros(_lib.load().fsb_muon_workspace_floats(), dtype=torch.float32, device=device)


def ns_iterations(x: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS) -> torch.Tensor:
    """Run the iteration on an already normalised bf16 matrix ``x`` (any aspect ratio)."""
    a, b, c = coeffs
    rows, cols = x.shape
    wide = rows <= cols
    s = min(rows, cols)
    A = torch.empty(s, s, dtype=x.dtype, device=x.device)
    B = torch.empty(s, s, dtype=x.dtype, device=x.device)
    nxt = torch.empty_like(x)
    for _ in range(steps):
        if wide:
            gemm(x, x, out=A, symmetric=True)                   # A = X X^T
            gemm(A, A, out=B, c=A, alpha=c, beta=b, symmetric=True)   # B = b A + c A A   (A symmetric)
            gemm(B, x, b_t=True, out=nxt, c=x, alpha=1.0, beta=a)  # X = a X + B X
        else:
            gemm(x, x, a_t=True, b_t=True, out=A, symmetric=True)     # A = X^T X
            gemm(A, A, out=B, c=A, alpha=c, beta=b, symmetric=True)
            gemm(x, B, out=nxt, c=x, alpha=1.0, beta=a)         # X = a X + X B     (B symmetric)
        x, nxt = nxt, x
    return x


_batch_tables: dict = {}


def _tables(E: int, rows: int, device):
    """Grouped-GEMM tables of ``E`` equal groups of ``rows`` rows (``rows`` a multiple of 128): the group of every
    128-row tile, the tile count and the group offsets, as device tensors."""
    key = (E, rows, device)
    t = _batch_tables.get(key)
    if t is None:
        tile_group = torch.arange(E, dtype=torch.int32).repeat_interleave(rows // 128).to(device)
        count = torch.tensor([E * rows // 128], dtype=torch.int32, device=device)
        offs = (torch.arange(E + 1, dtype=torch.int64) * rows).to(torch.int32).to(device)
        t = _batch_tables[key] = (tile_group, count, offs)
        if len(_batch_tables) > 256:
            _batch_tables.pop(next(iter(_batch_tables)))
    return t


def _grouped(mode, a, b, out, E, M, N, K, b_mn, tables, max_rows, c=None, alpha=1.0, beta=0.0):
    lib = _lib.load()
    fn = lib.fsb_gemm_bf16_grouped_ex
    if not getattr(fn, "_fsb_declared", False):
        cc = ctypes
        vp, i32, i64, f32 = cc.c_void_p, cc.c_int, cc.c_longlong, cc.c_float
        fn.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, i32, i32, vp, vp, vp, i32,
                       vp, i64, i32, f32, f32, vp, vp]
        fn.restype = cc.c_int
        fn._fsb_declared = True
    tile_group, count, offs = tables
    rc = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), mode, E, M, N, K, a.stride(0), b.stride(0), out.stride(-2),
            int(b_mn), 0, 0, tile_group.data_ptr(), count.data_ptr(), offs.data_ptr(), max_rows,
            c.data_ptr() if c is not None else None, c.stride(-2) if c is not None else 0, 0, alpha, beta,
            _lib.status_word(a.device).data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "fsb_gemm_bf16_grouped_ex")
    count_launch()


def batched_ns_supported(x: torch.Tensor) -> bool:
    """Stacks of equal matrices whose dimensions are multiples of 128 run every product of an iteration as one
    grouped launch over the whole stack."""
    return (x.is_cuda and x.dim() == 3 and x.shape[0] > 1 and x.shape[1] % 128 == 0 and x.shape[2] % 128 == 0)


def ns_iterations_batched(x: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS) -> torch.Tensor:
    """The iteration on a stack ``[E, rows, cols]`` of normalised bf16 matrices: three grouped GEMM launches per
    step for all ``E`` matrices (per-head and per-expert matrices are small; one launch each would leave most of
    the GPU idle and pay 15 launches per matrix).  Same arithmetic per matrix as ``ns_iterations``."""
    a, b, c = coeffs
    E, rows, cols = x.shape
    wide = rows <= cols
    s = min(rows, cols)
    x = x.contiguous()
    dev = x.device
    A = torch.empty(E, s, s, dtype=x.dtype, device=dev)
    B = torch.empty(E, s, s, dtype=x.dtype, device=dev)
    nxt = torch.empty_like(x)
    t_s, t_rows = _tables(E, s, dev), _tables(E, rows, dev)
    A2, B2 = A.view(E * s, s), B.view(E * s, s)
    for _ in range(steps):
        x2, n2 = x.view(E * rows, cols), nxt.view(E * rows, cols)
        if wide:
            _grouped(1, x2, x2, A2, E, E * s, s, cols, False, t_s, E * s)                      # A = X X^T
            _grouped(1, A2, A2, B2, E, E * s, s, s, False, t_s, E * s, c=A2, alpha=c, beta=b)  # B = b A + c A A
            _grouped(1, B2, x2, n2, E, E * s, cols, s, True, t_s, E * s, c=x2, alpha=1.0, beta=a)   # X = a X + B X
        else:
            _grouped(2, x2, x2, A, E, s, s, E * rows, True, t_rows, E * rows)                   # A = X^T X
            _grouped(1, A2, A2, B2, E, E * s, s, s, False, t_s, E * s, c=A2, alpha=c, beta=b)
            _grouped(1, x2, B2, n2, E, E * rows, s, s, False, t_rows, E * rows, c=x2, alpha=1.0, beta=a)  # X = a X + X B
        x, nxt = nxt, x
    return x


def _newton_schulz_cpu(g: torch.Tensor, steps: int, coeffs, eps: float) -> torch.Tensor:
    """The CPU statement of the iteration, in the very operations ``torch.optim.Muon`` uses (bf16 norm and division,
    bf16 ``matmul`` / ``addmm``), so that on CPU an owner-stored matrix steps bitwise like that optimizer."""
    a, b, c = coeffs
    x = g.to(torch.bfloat16)
    tall = g.size(0) > g.size(1)
    if tall:
        x = x.T
    x = x / x.norm().clamp(min=eps)
    for _ in range(steps):
        gram = x @ x.T
        x = torch.addmm(x, torch.addmm(gram, gram, gram, beta=b, alpha=c), x, beta=a)
    return x.T if tall else x


def newton_schulz_kernel_reference(g: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS, eps: float = 1e-7) -> torch.Tensor:
    """CPU restatement of the arithmetic of the GPU kernels for one matrix (norm in fp32, the scaled matrix rounded to
    bf16 once, every product accumulated in fp32 and rounded once): the oracle the GPU tests compare against."""
    x = g.detach().cpu().to(torch.bfloat16)
    x = x / x.float().norm().clamp_min(eps).to(torch.bfloat16)
    return ns_iterations(x.contiguous(), steps, coeffs)


def newton_schulz(g: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS, eps: float = 1e-7) -> torch.Tensor:
    """Approximate polar factor of ``g`` ([rows, cols] or batched [n, rows, cols]); returns bf16."""
    if g.dim() == 2 and not g.is_cuda:
        return _newton_schulz_cpu(g, steps, coeffs, eps)
    if g.dim() == 3:
        if batched_ns_supported(g):
            x = g.to(torch.bfloat16)
            norm = x.float().square().sum((1, 2), keepdim=True).sqrt().clamp_min(eps)
            return ns_iterations_batched((x.float() / norm).to(torch.bfloat16), steps, coeffs)
        return torch.stack([newton_schulz(m, steps, coeffs, eps) for m in g])
    x = g.to(torch.bfloat16)
    x = x / x.float().norm().clamp_min(eps).to(torch.bfloat16) if not x.is_cuda else _normalise_cuda(x, eps)
    return ns_iterations(x.contiguous(), steps, coeffs)


def _normalise_cuda(x: torch.Tensor, eps: float) -> torch.Tensor:
    _ensure()
    x = x.contiguous().clone()
    ss = (x.float() ** 2).sum().reshape(1)
    rc = _lib.load().fsb_muon_scale(x.data_ptr(), ss.data_ptr(), x.numel(), eps, _lib.stream_ptr(x.device))
    _lib.check(rc, "fsb_muon_scale")
    count_launch()
    return x


def muon_direction_(momentum: torch.Tensor, grad: torch.Tensor, mu: float, nesterov: bool, steps: int,
                    coeffs=NS_COEFFS, eps: float = 1e-7) -> torch.Tensor:
    """Momentum update (in place, fp32) + Nesterov + normalise + Newton-Schulz; returns the bf16
    direction with the shape of ``grad`` (2-D)."""
    assert grad.dim() == 2 and momentum.shape == grad.shape
    if not grad.is_cuda:
        momentum.lerp_(grad.float(), 1 - mu)
        u = grad.float().lerp(momentum, mu) if nesterov else momentum
        return _newton_schulz_cpu(u, steps, coeffs, eps)
    _ensure()
    lib = _lib.load()
    g = grad.contiguous()
    assert momentum.is_contiguous() and momentum.dtype == torch.float32
    u = torch.empty(g.shape, dtype=torch.bfloat16, device=g.device)
    ss = _workspace(g.device)
    s = _lib.stream_ptr(g.device)
    rc = lib.fsb_muon_prepare(momentum.data_ptr(), g.data_ptr(), int(g.dtype == torch.float32), u.data_ptr(),
                              ss.data_ptr(), g.numel(), mu, int(nesterov), s)
    _lib.check(rc, "fsb_muon_prepare")
    rc = lib.fsb_muon_scale(u.data_ptr(), ss.data_ptr(), u.numel(), eps, s)
    _lib.check(rc, "fsb_muon_scale")
    count_launch(2)
    return ns_iterations(u, steps, coeffs)


def muon_momentum_direction_(momentum: torch.Tensor, grad: torch.Tensor, mu: float, nesterov: bool) -> torch.Tensor:
    """``M <- lerp(M, g, 1-mu)`` in place (fp32) and return ``u = lerp(g, M, mu)`` (Nesterov) or ``M`` as bf16,
    in the shape of ``grad``: the elementwise half of a Muon step, for rows that are orthogonalised elsewhere."""
    assert momentum.shape == grad.shape and momentum.dtype == torch.float32
    if not grad.is_cuda:
        momentum.lerp_(grad.float(), 1 - mu)
        u = grad.float().lerp(momentum, mu) if nesterov else momentum
        return u.to(torch.bfloat16)
    _ensure()
    g = grad.contiguous()
    assert momentum.is_contiguous()
    u = torch.empty(g.shape, dtype=torch.bfloat16, device=g.device)
    ss = _workspace(g.device)
    rc = _lib.load().fsb_muon_prepare(momentum.data_ptr(), g.data_ptr(), int(g.dtype == torch.float32), u.data_ptr(),
                                      ss.data_ptr(), g.numel(), mu, int(nesterov), _lib.stream_ptr(g.device))
    _lib.check(rc, "fsb_muon_prepare")
    count_launch()
    return u


def muon_apply_(param: torch.Tensor, direction: torch.Tensor, lr: float, weight_decay: float, ratio: float):
    """``p <- p (1 - lr*wd) - lr*ratio*direction`` in place."""
    if not param.is_cuda:
        param.mul_(1 - lr * weight_decay).add_(direction.to(param.dtype), alpha=-lr * ratio)
        return
    _ensure()
    assert param.is_contiguous() and direction.is_contiguous() and direction.dtype == torch.bfloat16
    rc = _lib.load().fsb_muon_update(param.data_ptr(), int(param.dtype == torch.float32), direction.data_ptr(),
                                     param.numel(), 1.0 - lr * weight_decay, lr * ratio,
                                     _lib.stream_ptr(param.device))
    _lib.check(rc, "fsb_muon_update")
    count_launch()
