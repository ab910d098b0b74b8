"""``BlockwiseQuantWeight``: a wrapper tensor whose logical shape/dtype are the high-precision
weight's while its payload is quantised data + scales living in a bucket's persistent buffer.

Only ``detach`` / ``alias`` dispatch (what ``nn.Parameter`` construction and autograd bookkeeping
need); any real math must go through a linear module that understands the payload.
Parity: ``blockwise_quant/weight.py:17-110`` of the reference.
"""
from __future__ import annotations

import torch


class BlockwiseQuantWeight(torch.Tensor):
    __slots__ = ()
    inner_names = ("qdata", "scale")

    @staticmethod
    def __new__(cls, qdata: torch.Tensor, scale: torch.Tensor, shape, dtype=torch.bfloat16, **extra):
        r = torch.Tensor._make_wrapper_subclass(cls, tuple(shape), dtype=dtype, device=qdata.device,
                                                requires_grad=False)
        r.qdata = qdata
        r.scale = scale
        r.extra = dict(extra)
        return r

    def __tensor_flatten__(self):
        return list(self.inner_names), {"shape": tuple(self.shape), "dtype": self.dtype, "extra": self.extra}

    @classmethod
    def __tensor_unflatten__(cls, inner, meta, outer_size=None, outer_stride=None):
        return cls(inner["qdata"], inner["scale"], meta["shape"], meta["dtype"], **meta.get("extra", {}))

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        name = getattr(func, "_schema", None)
        fname = str(func)
        if "detach" in fname or "alias" in fname:
            return args[0]._rebuild()
        raise NotImplementedError(
            f"{cls.__name__} only supports detach/alias; use it through a prequantised linear module ({fname})")

    def _rebuild(self):
        return type(self)(self.qdata, self.scale, self.shape, self.dtype, **self.extra)

    def __repr__(self):
        return f"{type(self).__name__}(shape={tuple(self.shape)}, dtype={self.dtype}, qdata={tuple(self.qdata.shape)})"

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        raise NotImplementedError


class BlockwiseFp8Weight(BlockwiseQuantWeight):
    """e4m3 data ``[out, in]`` + one fp32 reciprocal scale per 128x128 tile.
    Parity: ``blockwise_fp8/blockwise_fp8_weight.py:25-145`` of the reference."""

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        from ..ops.fp8 import dequantize_blockwise

        return dequantize_blockwise(self.qdata, self.scale, dtype).reshape(self.shape)

    def matrix(self, *index: int) -> "BlockwiseFp8Weight":
        """Matrix ``index`` of a stacked weight ``[*stack, out, in]`` as a 2-D quantised weight (views of the same
        payload: the stack's matrices lie one under the other and ``out`` is a multiple of 128)."""
        *stack, out, cin = self.shape
        flat = 0
        for i, n in zip(index, stack):
            flat = flat * n + i
        return BlockwiseFp8Weight(self.qdata[flat * out:(flat + 1) * out],
                                  self.scale[flat * out // 128:(flat + 1) * out // 128], (out, cin), self.dtype)


class BlockwiseMxfp8Weight(BlockwiseQuantWeight):
    """MXFP8 weight handed out by the all-gather: row-major e4m3 data ``[out, in]`` with 32x32 tile
    scales, kept as the tile exponents plus the two scale tensors the tensor core reads
    (``fwd_scale``: groups along ``in`` for y = x W^T; ``dgrad_scale``: groups along ``out`` for
    dx = dy W), both in the blocked 128x4 layout.
    Parity: ``blockwise_mxfp8/blockwise_mxfp8_weight.py:41-135`` of the reference."""

    inner_names = ("qdata", "scale", "dgrad_scale")

    @staticmethod
    def __new__(cls, qdata, scale, shape, dtype=torch.bfloat16, dgrad_scale=None, **extra):
        r = BlockwiseQuantWeight.__new__(cls, qdata, scale, shape, dtype, **extra)
        r.dgrad_scale = dgrad_scale
        return r

    @classmethod
    def from_tile_exponents(cls, qdata, tile_exp, shape, dtype=torch.bfloat16):
        from ..ops.mxfp8 import mx_expand_scales

        rows, cols = qdata.shape
        return cls(qdata, mx_expand_scales(tile_exp, rows, cols, False), shape, dtype,
                   dgrad_scale=mx_expand_scales(tile_exp, rows, cols, True), tile_exp=tile_exp)

    @classmethod
    def __tensor_unflatten__(cls, inner, meta, outer_size=None, outer_stride=None):
        return cls(inner["qdata"], inner["scale"], meta["shape"], meta["dtype"], dgrad_scale=inner["dgrad_scale"],
                   **meta.get("extra", {}))

    def _rebuild(self):
        return type(self)(self.qdata, self.scale, self.shape, self.dtype, dgrad_scale=self.dgrad_scale, **self.extra)

    @property
    def fp8_data(self):
        return self.qdata

    @property
    def fwd_scale(self):
        return self.scale

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        return blockwise_mxfp8_dequant_weight(self.qdata, self.scale).reshape(self.shape).to(dtype)

    def matrix(self, *index: int) -> "BlockwiseMxfp8Weight":
        """Matrix ``index`` of a stacked weight as a 2-D MXFP8 weight (its blocked scale tensors are rebuilt from
        the matrix's tile exponents)."""
        *stack, out, cin = self.shape
        flat = 0
        for i, n in zip(index, stack):
            flat = flat * n + i
        te = self.extra["tile_exp"]
        return BlockwiseMxfp8Weight.from_tile_exponents(self.qdata[flat * out:(flat + 1) * out],
                                                        te[flat * out // 32:(flat + 1) * out // 32], (out, cin), self.dtype)


def blockwise_mxfp8_dequant_weight(fp8_data: torch.Tensor, fwd_scale: torch.Tensor) -> torch.Tensor:
    """Row-major e4m3 data with its forward-orientation blocked scales -> fp32."""
    from ..ops.mxfp8 import mx_dequantize

    return mx_dequantize(fp8_data, fwd_scale)


def blockwise_dequant_weight(w: BlockwiseQuantWeight, dtype=torch.float32) -> torch.Tensor:
    return w.dequantize(dtype)
