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
            self = args[0]
            return type(self)(self.qdata, self.scale, self.shape, self.dtype, **self.extra)
        raise NotImplementedError(
            f"{cls.__name__} only supports detach/alias; use it through a prequantised linear module ({fname})")

    def __repr__(self):
        return f"{type(self).__name__}(shape={tuple(self.shape)}, dtype={self.dtype}, qdata={tuple(self.qdata.shape)})"

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        raise NotImplementedError


class BlockwiseFp8Weight(BlockwiseQuantWeight):
    """e4m3 data ``[out, in]`` + one fp32 reciprocal scale per 128x128 tile.
    Parity: ``blockwise_fp8/blockwise_fp8_weight.py:25-145`` of the reference."""

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        from ..ops.fp8 import dequantize_blockwise

        return dequantize_blockwise(self.qdata, self.scale, dtype)


def blockwise_dequant_weight(w: BlockwiseQuantWeight, dtype=torch.float32) -> torch.Tensor:
    return w.dequantize(dtype)
