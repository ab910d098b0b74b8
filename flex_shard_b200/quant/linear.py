"""Linear layers that consume prequantised (FP8 blockwise) weights.

``FlexShardFloat8BlockwiseLinear`` keeps a bf16 master ``weight``. Under ``flex_shard`` with
``Fp8BucketedBlockShard`` the runtime swaps in a ``BlockwiseFp8Weight`` whose payload was
quantised on the owning ranks and gathered as FP8; the forward and dgrad GEMMs run block-scaled
FP8 on tcgen05, the weight gradient is a bf16 GEMM in the parameter's gradient dtype. Without
sharding the master is quantised on the fly (same kernels, same numerics).

Parity: ``blockwise_quant/linear.py:20-184`` and ``blockwise_fp8/fp8_blockwise_linear.py:42-211``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.fp8 import fp8_linear, quantize_blockwise
from ..ops.mxfp8 import mx_expand_scales, mx_quantize_weight, mxfp8_linear
from .weight import BlockwiseFp8Weight, BlockwiseMxfp8Weight


class FlexShardPrequantizedLinear(nn.Module):
    """Base: ``weight`` is ``[out, in]`` (stacked weights multiply as the flattened matrix)."""

    def __init__(self, in_features: int, out_features: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))

    def payload(self, w):
        raise NotImplementedError

    def forward(self, x):
        raise NotImplementedError


class FlexShardFloat8BlockwiseLinear(FlexShardPrequantizedLinear):
    def payload(self, w):
        if isinstance(w, BlockwiseFp8Weight):
            return w.qdata, w.scale
        wq, ws = quantize_blockwise(w.detach().to(torch.bfloat16))
        return wq, ws

    def forward(self, x):
        w = self.weight
        wq, ws = self.payload(w)
        return fp8_linear(x, w, wq, ws)


class _Fp8StackedLinear(torch.autograd.Function):
    """y[e] = x[e] W[e]^T for a stacked weight ``[E, out, in]`` given as the FP8 payload of the matrices laid one
    under the other; ``weight`` is the logical parameter that receives the stacked bf16-GEMM weight gradient."""

    @staticmethod
    def forward(ctx, x, weight, wq, ws):
        from ..ops.fp8 import gemm_fp8, quantize_act

        E, out = x.shape[0], wq.shape[0] // x.shape[0]
        ctx.save_for_backward(x, wq, ws)
        ctx.weight_ref, ctx.out = weight, out
        ys = []
        for e in range(E):
            xq, sx = quantize_act(x[e].reshape(-1, x.shape[-1]))
            ys.append(gemm_fp8(xq, sx, wq[e * out:(e + 1) * out], ws[e * out // 128:(e + 1) * out // 128]))
        return torch.stack(ys).view(E, *x.shape[1:-1], out)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.fp8 import gemm_fp8, quantize_act
        from ..ops.gemm import gemm

        x, wq, ws = ctx.saved_tensors
        E, out, cin = x.shape[0], ctx.out, x.shape[-1]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dxs = []
            for e in range(E):
                dyq, sdy = quantize_act(dy[e].reshape(-1, out).contiguous())
                dxs.append(gemm_fp8(dyq, sdy, wq[e * out:(e + 1) * out], ws[e * out // 128:(e + 1) * out // 128], b_t=True))
            dx = torch.stack(dxs).view(x.shape)
        if ctx.needs_input_grad[1]:
            gd = getattr(ctx.weight_ref, "grad_dtype", None)
            gd = gd if gd in (torch.bfloat16, torch.float32) else torch.bfloat16
            dw = torch.empty(E, out, cin, dtype=gd, device=x.device)
            for e in range(E):
                gemm(dy[e].reshape(-1, out).contiguous(), x[e].reshape(-1, cin).contiguous(), a_t=True, b_t=True, out=dw[e])
        return dx, dw, None, None


class FlexShardFloat8BlockwiseStackedLinear(nn.Module):
    """``n`` independent linears held as one stacked weight ``[n, out, in]`` (MoE experts): ``forward(x)`` maps
    ``x[e]`` through matrix ``e``. Under ``Fp8BucketedBlockShard`` the gathered weight is one FP8 payload of the
    matrices laid one under the other (``out`` a multiple of 128, so every matrix keeps its own tiles)."""

    def __init__(self, n: int, in_features: int, out_features: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.n, self.in_features, self.out_features = n, in_features, out_features
        self.weight = nn.Parameter(torch.empty(n, out_features, in_features, dtype=dtype, device=device))

    def forward(self, x):
        w = self.weight
        if isinstance(w, BlockwiseFp8Weight):
            wq, ws = w.qdata, w.scale
        else:
            wq, ws = quantize_blockwise(w.detach().to(torch.bfloat16).reshape(-1, self.in_features))
        return _Fp8StackedLinear.apply(x, w, wq, ws)


class FlexShardMxfp8BlockwiseLinear(FlexShardPrequantizedLinear):
    """Linear on MXFP8 operands: forward and input-gradient products run on the block-scaled tensor
    core path (``kind::mxf8f6f4``), activations and output gradients are quantised 1x32 on the fly,
    the weight gradient is a bf16 GEMM emitted in the parameter's gradient dtype.
    Parity: ``blockwise_mxfp8/mxfp8_blockwise_linear.py:58-196`` of the reference."""

    def payload(self, w):
        if isinstance(w, BlockwiseMxfp8Weight):
            return w.qdata, w.scale, w.dgrad_scale
        rows, cols = w.shape
        q, e = mx_quantize_weight(w.detach().to(torch.bfloat16))
        return q, mx_expand_scales(e, rows, cols, False), mx_expand_scales(e, rows, cols, True)

    def forward(self, x):
        w = self.weight
        q, fwd, dgrad = self.payload(w)
        return mxfp8_linear(x, w, q, fwd, dgrad)


def _convert(module: nn.Module, cls, filter_fn) -> nn.Module:
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear) and child.bias is None and child.in_features % 128 == 0 \
                and child.out_features % 128 == 0 and (filter_fn is None or filter_fn(name, child)):
            new = cls(child.in_features, child.out_features, child.weight.dtype, child.weight.device)
            new.weight = child.weight
            setattr(module, name, new)
        else:
            _convert(child, cls, filter_fn)
    return module


def convert_to_flex_shard_mxfp8_blockwise_linear(module: nn.Module, filter_fn=None) -> nn.Module:
    """Replace bias-free ``nn.Linear`` layers whose dims are multiples of 128 by the MXFP8 linear."""
    return _convert(module, FlexShardMxfp8BlockwiseLinear, filter_fn)


def convert_to_flex_shard_float8_blockwise_linear(module: nn.Module, filter_fn=None) -> nn.Module:
    """Replace ``nn.Linear`` layers (without bias, dims multiples of 128) by the FP8 blockwise linear,
    keeping the weights. ``filter_fn(name, linear) -> bool`` selects layers."""
    for name, child in list(module.named_children()):
        if isinstance(child, nn.Linear) and child.bias is None and child.in_features % 128 == 0 \
                and child.out_features % 128 == 0 and (filter_fn is None or filter_fn(name, child)):
            new = FlexShardFloat8BlockwiseLinear(child.in_features, child.out_features, child.weight.dtype,
                                                 child.weight.device)
            new.weight = child.weight
            setattr(module, name, new)
        else:
            convert_to_flex_shard_float8_blockwise_linear(child, filter_fn)
    return module


convert_to_flex_shard_prequantized_linear = convert_to_flex_shard_float8_blockwise_linear
