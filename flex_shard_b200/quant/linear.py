"""Linear layers that consume prequantised (FP8 blockwise) weights.

``FlexShardFloat8BlockwiseLinear`` keeps a bf16 master ``weight``. Under ``flex_shard`` with
``Fp8BucketedBlockShard`` the runtime swaps in a ``BlockwiseFp8Weight`` whose payload was
quantised on the owning ranks and gathered as FP8; the forward and dgrad GEMMs run block-scaled
FP8 on tcgen05, the weight gradient is a bf16 GEMM in the parameter's gradient dtype. Without
sharding the master is quantised on the fly (same kernels, same numerics).

Parity: ``blockwise_quant/linear.py:20-184`` and ``blockwise_fp8/fp8_blockwise_linear.py:42-211``.
"""
from __future__ import annotations

import math
from typing import Callable, Protocol

import torch
import torch.nn as nn

from ..ops.fp8 import fp8_linear, quantize_blockwise
from ..ops.mxfp8 import mx_expand_scales, mx_quantize_weight, mxfp8_linear
from .weight import BlockwiseFp8Weight, BlockwiseMxfp8Weight, BlockwiseQuantWeight


class PrequantizedLinearGemms(Protocol):
    """The products of a linear layer for one quantised weight format: what another format has to supply to run
    under ``FlexShardPrequantizedLinear``.  A stacked ``[*stack, out, in]`` weight multiplies as its flattened
    ``[prod(stack) * out, in]`` matrix.  Parity: ``blockwise_quant/linear.py:20-47`` of the reference."""

    def forward(self, x_2d: torch.Tensor, weight: BlockwiseQuantWeight) -> torch.Tensor:
        """``x_2d @ matrix(weight).T``, shape ``[tokens, rows]``."""
        ...

    def backward(self, grad_output_2d: torch.Tensor, x_2d: torch.Tensor, weight: BlockwiseQuantWeight,
                 needs_x_grad: bool, needs_weight_grad: bool) -> tuple[torch.Tensor | None, torch.Tensor | None]:
        """``(grad_x_2d, grad_weight)``; ``grad_weight`` is contiguous and has the weight's shape."""
        ...


class _GemmsLinear(torch.autograd.Function):
    """``y = x W^T (+ bias)`` through a format's ``PrequantizedLinearGemms``."""

    @staticmethod
    def forward(ctx, x, weight, bias, gemms):
        if x.shape[-1] != weight.shape[-1]:
            raise ValueError(f"input last dim {x.shape[-1]} does not match the weight's input dim {weight.shape[-1]}")
        out = gemms.forward(x.reshape(-1, x.shape[-1]), weight).reshape(*x.shape[:-1], *weight.shape[:-1])
        if bias is not None:
            out = out + bias
        ctx.save_for_backward(x, weight)
        ctx.gemms, ctx.has_bias = gemms, bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        g2 = grad_output.reshape(-1, math.prod(weight.shape[:-1])).contiguous()
        need_x, need_w, need_b = ctx.needs_input_grad[:3]
        dx, dw = ctx.gemms.backward(g2, x.reshape(-1, x.shape[-1]), weight, need_x, need_w)
        db = g2.sum(0).view(weight.shape[:-1]) if ctx.has_bias and need_b else None
        return (None if dx is None else dx.reshape(x.shape)), dw, db, None


class FlexShardPrequantizedLinear(nn.Module):
    """Base: ``weight`` is ``[out, in]`` (stacked weights multiply as the flattened matrix).

    The FP8 and MXFP8 layers below override ``forward`` with this library's kernels.  Another format plugs in by
    setting ``weight_type`` (its ``BlockwiseQuantWeight`` subclass, produced by its placement's
    ``weight_factory``) and returning its products from ``_prequantized_gemms``; the inherited ``forward`` then
    requires a weight of that type and runs ``y = x W^T (+ bias)`` through them."""

    weight_type: type = BlockwiseQuantWeight

    def __init__(self, in_features: int, out_features: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))

    @classmethod
    def from_float(cls, linear: nn.Linear, **kwargs):
        """The replacement of ``linear`` (bias-free), sharing its weight."""
        if linear.bias is not None:
            raise ValueError(f"{cls.__name__} replaces bias-free linear layers")
        new = cls(linear.in_features, linear.out_features, linear.weight.dtype, linear.weight.device, **kwargs)
        new.weight = linear.weight
        return new

    def payload(self, w):
        raise NotImplementedError

    def _prequantized_gemms(self) -> PrequantizedLinearGemms | None:
        return None

    def forward(self, x):
        gemms = self._prequantized_gemms()
        if gemms is None:
            raise NotImplementedError(f"{type(self).__name__} defines neither forward nor _prequantized_gemms")
        w = self.weight
        if not isinstance(w, self.weight_type):
            raise TypeError(f"{type(self).__name__} needs a {self.weight_type.__name__} produced by a quantised "
                            f"all-gather, got {type(w).__name__}")
        return _GemmsLinear.apply(x, w, getattr(self, "bias", None), gemms)


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


def _eligible(child) -> bool:
    return (isinstance(child, nn.Linear) and child.bias is None and child.in_features % 128 == 0
            and child.out_features % 128 == 0)


def convert_to_flex_shard_prequantized_linear(module: nn.Module, linear_cls: type | None = None,
                                              filter_fn: Callable[[str, nn.Linear], bool] | None = None,
                                              **from_float_kwargs) -> nn.Module:
    """Replace the ``nn.Linear`` children that ``filter_fn(dotted name, linear)`` selects (default: all) by
    ``linear_cls.from_float(linear, **from_float_kwargs)``, keeping the weights.  ``linear_cls`` defaults to the FP8
    blockwise layer; this library's two layers only take bias-free layers whose dims are multiples of 128 and skip
    the others.  Parity: ``blockwise_quant/linear.py:158-184`` of the reference."""
    linear_cls = linear_cls or FlexShardFloat8BlockwiseLinear
    own = linear_cls in (FlexShardFloat8BlockwiseLinear, FlexShardMxfp8BlockwiseLinear)

    def walk(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            fqn = f"{prefix}.{name}" if prefix else name
            if isinstance(child, FlexShardPrequantizedLinear):
                continue
            if (isinstance(child, nn.Linear) and (not own or _eligible(child))
                    and (filter_fn is None or filter_fn(fqn, child))):
                setattr(parent, name, linear_cls.from_float(child, **from_float_kwargs))
            else:
                walk(child, fqn)

    walk(module, "")
    return module


def convert_to_flex_shard_mxfp8_blockwise_linear(module: nn.Module, filter_fn=None) -> nn.Module:
    """Replace bias-free ``nn.Linear`` layers whose dims are multiples of 128 by the MXFP8 linear."""
    return convert_to_flex_shard_prequantized_linear(module, FlexShardMxfp8BlockwiseLinear, filter_fn)


def convert_to_flex_shard_float8_blockwise_linear(module: nn.Module, filter_fn=None) -> nn.Module:
    """Replace ``nn.Linear`` layers (without bias, dims multiples of 128) by the FP8 blockwise linear,
    keeping the weights. ``filter_fn(dotted name, linear) -> bool`` selects layers."""
    return convert_to_flex_shard_prequantized_linear(module, FlexShardFloat8BlockwiseLinear, filter_fn)
