"""bf16 tcgen05 GEMM and the linear-layer autograd function built on it.

``gemm`` computes ``D = alpha * A @ B^T + beta * C (+ D)`` where A is
``[M, K]`` and B is ``[N, K]`` logically; each may be handed over transposed
in memory (``a_t`` / ``b_t``: the tensor passed is ``[K, M]`` / ``[K, N]``),
which the kernel reads as an MN-major operand, so a linear layer's forward,
dgrad and wgrad all run without a transpose copy.

CPU tensors take a PyTorch fp32 reference path (used by the CPU test-suite).
"""
from __future__ import annotations

import torch

from . import _lib

from ._lib import count_launch


class PeerBlocked:
    """A ``[rows, cols]`` gradient destination cut into ``len(addrs)`` row blocks of ``block_rows``
    rows, block ``i`` living at address ``addrs[i]`` (peer GPU ``i``'s incoming slot, row stride
    ``cols``). Handing it to ``gemm(out=...)`` makes the epilogue store each block straight into the
    owner's memory over NVLink."""

    def __init__(self, addrs, block_rows: int, rows: int, cols: int, dtype: torch.dtype, device, local: bool = False):
        import ctypes

        self.local = local   # every block is in this GPU's own memory: ordinary vector stores are best

        self.addrs = (ctypes.c_ulonglong * len(addrs))(*addrs)
        self.n = len(addrs)
        self.block_rows, self.rows, self.cols = block_rows, rows, cols
        self.dtype, self.device = dtype, device
        self.shape = (rows, cols)

    def dim(self):
        return 2


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.stride(-1) != 1 or (t.dim() == 2 and t.stride(0) % 8 != 0) or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         c: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 1.0,
         accumulate: bool = False, max_ctas: int = 0, symmetric: bool = False) -> torch.Tensor:
    """``out = alpha * A @ B^T + beta * c (+ out)`` with bf16 operands, fp32 accumulation.

    ``symmetric=True`` promises that the result is a symmetric matrix (``X X^T``, or a symmetric matrix times
    itself, with a symmetric ``c``): for square bf16 outputs the kernel then computes only the tiles on or above
    the diagonal and mirrors them, which halves the work of a large product."""
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_t else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_t else b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    block_rows = block_stride = 0
    peer = None
    if isinstance(out, PeerBlocked):
        assert a.is_cuda and out.shape == (M, N) and c is None
        peer, block_rows, ldd = out, out.block_rows, out.cols
    elif out.dim() == 3:
        # [blocks, rows_per_block, N] view of a reduce-scatter send buffer: rows of block i
        # start at out[i]; rows past M (padding of the last block) are never written.
        assert out.shape[2] == N and out.stride(2) == 1 and out.shape[0] * out.shape[1] >= M
        block_rows, block_stride = out.shape[1], out.stride(0)
        ldd = out.stride(1)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
        ldd = out.stride(0)
    if not a.is_cuda:
        af = (a.t() if a_t else a).float()
        bf = (b.t() if b_t else b).float()
        r = alpha * (af @ bf.t())
        if c is not None:
            r = r + beta * c.float()
        dst = out if out.dim() == 2 else out.reshape(-1, N)[:M] if out.is_contiguous() else None
        if dst is None:  # strided block view: write block by block
            br = out.shape[1]
            for i in range(out.shape[0]):
                lo, hi = i * br, min((i + 1) * br, M)
                if hi > lo:
                    blk = out[i, : hi - lo]
                    blk.copy_(r[lo:hi] + (blk.float() if accumulate else 0))
            return out
        if accumulate:
            r = r + dst.float()
        dst.copy_(r)
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert out.dtype in (torch.bfloat16, torch.float32)
    if peer is None:
        out_ptr, peer_ptrs, peer_n = out.data_ptr(), None, 0
    else:
        out_ptr, peer_ptrs, peer_n = None, peer.addrs, (-peer.n if peer.local else peer.n)
    a = _rowmajor(a)
    b = _rowmajor(b)
    if c is not None:
        assert c.shape == (M, N) and c.stride(1) == 1 and c.dtype in (torch.bfloat16, torch.float32)
    if K % 8 != 0 or (a_t and M % 8 != 0) or (b_t and N % 8 != 0):
        raise ValueError("gemm: K (and the contiguous dim of transposed operands) must be a multiple of 8")
    lib = _lib.load()
    status = _lib.status_word(a.device)
    rc = lib.fsb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out_ptr, c.data_ptr() if c is not None else None,
        M, N, K, a.stride(0), b.stride(0), ldd, c.stride(0) if c is not None else 0,
        int(a_t), int(b_t), int(out.dtype == torch.float32),
        int(c is not None and c.dtype == torch.float32), alpha, beta, int(accumulate) | (2 if symmetric else 0),
        block_rows, block_stride, peer_ptrs, peer_n, status.data_ptr(), max_ctas, _lib.stream_ptr(a.device))
    _lib.check(rc, "fsb_gemm_bf16")
    count_launch()
    return out


class _Linear(torch.autograd.Function):
    """y = x W^T on the tcgen05 GEMM; wgrad may accumulate straight into an fp32 buffer."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, weight)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_t=True).view(x.shape)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None and (isinstance(main, PeerBlocked) or main.dtype in (torch.float32, torch.bfloat16)):
                # The weight gradient goes straight into this parameter's rows of the bucket's
                # reduce-scatter send buffer (cast to the reduce dtype in the GEMM epilogue);
                # autograd gets nothing to cast, pack or add.
                gemm(dy2, x2, a_t=True, b_t=True, out=main,
                     accumulate=bool(getattr(weight, "main_grad_written", False)))
                weight.main_grad_written = True
                dw = None
            else:
                dw = gemm(dy2, x2, a_t=True, b_t=True, out_dtype=weight.dtype
                          if weight.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)
        return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T``. A weight handed out by a quantised-gather placement (FP8 128x128 blocks or
    MXFP8) runs the matching block-scaled products; its gradient still goes to the logical parameter."""
    if type(weight) is not torch.Tensor and type(weight) is not torch.nn.Parameter:
        from ..quant.weight import BlockwiseFp8Weight, BlockwiseMxfp8Weight

        if isinstance(weight, BlockwiseMxfp8Weight):
            from .mxfp8 import mxfp8_linear

            return mxfp8_linear(x, weight, weight.qdata, weight.scale, weight.dgrad_scale)
        if isinstance(weight, BlockwiseFp8Weight):
            from .fp8 import fp8_linear

            return fp8_linear(x, weight, weight.qdata, weight.scale)
    return _Linear.apply(x, weight)


def split_into_bf16_pieces(t: torch.Tensor):
    """fp32 tensor -> three bf16 tensors (high, middle, low part) whose sum reproduces it to ~24 bits."""
    hi = t.to(torch.bfloat16)
    rest = t - hi.float()
    mid = rest.to(torch.bfloat16)
    lo = (rest - mid.float()).to(torch.bfloat16)
    return hi, mid, lo


class _Fp32OutputLinear(torch.autograd.Function):
    """``x @ weight.T`` from bf16 operands, accumulated and returned in fp32 (router logits). The
    backward pass keeps close to fp32 accuracy on bf16 tensor cores: the fp32 output gradient is cut
    into three bf16 pieces that sum to it, and each product is three tcgen05 GEMMs accumulated in an
    fp32 output (parity: ``_Fp32OutputLinear`` of the reference's DeepSeek-V3 example,
    ``examples/deepseek_v3/model.py:368-422``)."""

    @staticmethod
    def forward(ctx, x, weight):
        x2 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16)
        w = weight.to(torch.bfloat16)
        ctx.save_for_backward(x2, w)
        ctx.xshape, ctx.xdtype, ctx.wdtype = x.shape, x.dtype, weight.dtype
        return gemm(x2, w, out_dtype=torch.float32).view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, w = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1]).float().contiguous()
        pieces = split_into_bf16_pieces(g2)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            acc = torch.empty(g2.shape[0], w.shape[1], dtype=torch.float32, device=g2.device)
            for i, p in enumerate(pieces):
                gemm(p, w, b_t=True, out=acc, accumulate=i > 0)
            dx = acc.to(ctx.xdtype).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            acc = torch.empty(w.shape, dtype=torch.float32, device=g2.device)
            for i, p in enumerate(pieces):
                gemm(p, x2, a_t=True, b_t=True, out=acc, accumulate=i > 0)
            dw = acc.to(ctx.wdtype)
        return dx, dw


def fp32_output_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _Fp32OutputLinear.apply(x, weight)
