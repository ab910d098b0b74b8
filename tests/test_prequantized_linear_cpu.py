"""The format-agnostic part of the prequantised linear layers: another quantised format plugs in with its weight
class and its products (``PrequantizedLinearGemms``), and the converter hands ``filter_fn`` dotted names.
Parity: ``blockwise_quant/linear.py:20-184`` of the reference."""
import pytest
import torch
import torch.nn as nn

from flex_shard_b200.quant import (BlockwiseQuantWeight, FlexShardFloat8BlockwiseLinear, FlexShardMxfp8BlockwiseLinear,
                                   FlexShardPrequantizedLinear, convert_to_flex_shard_float8_blockwise_linear,
                                   convert_to_flex_shard_prequantized_linear)


class RowScaledInt8Weight(BlockwiseQuantWeight):
    """int8 data with one fp32 scale per row: a stand-in for a third format."""

    def dequantize(self, dtype=torch.float32):
        return (self.qdata.float() * self.scale[:, None]).to(dtype).reshape(self.shape)

    @classmethod
    def quantise(cls, w):
        m = w.reshape(-1, w.shape[-1]).float()
        scale = m.abs().amax(1).clamp_min(1e-12) / 127
        return cls((m / scale[:, None]).round().to(torch.int8), scale, w.shape, w.dtype)


class Int8Gemms:
    calls = []

    def forward(self, x_2d, weight):
        self.calls.append(("fwd", tuple(x_2d.shape)))
        return x_2d @ weight.dequantize(x_2d.dtype).reshape(-1, weight.shape[-1]).t()

    def backward(self, grad_output_2d, x_2d, weight, needs_x_grad, needs_weight_grad):
        self.calls.append(("bwd", needs_x_grad, needs_weight_grad))
        m = weight.dequantize(x_2d.dtype).reshape(-1, weight.shape[-1])
        dx = grad_output_2d @ m if needs_x_grad else None
        dw = (grad_output_2d.t() @ x_2d).reshape(weight.shape).contiguous() if needs_weight_grad else None
        return dx, dw


class Int8Linear(FlexShardPrequantizedLinear):
    weight_type = RowScaledInt8Weight

    def _prequantized_gemms(self):
        return Int8Gemms()


def test_another_format_plugs_in_with_its_weight_class_and_products():
    torch.manual_seed(0)
    dense = nn.Linear(16, 24, bias=False)
    layer = Int8Linear.from_float(dense)
    assert layer.weight is dense.weight
    x = torch.randn(3, 5, 16, requires_grad=True)
    with pytest.raises(TypeError, match="RowScaledInt8Weight"):
        layer(x)                                            # the plain master weight is not the format's payload
    quantised = RowScaledInt8Weight.quantise(dense.weight.detach())
    layer.weight = nn.Parameter(quantised, requires_grad=False)
    y = layer(x)
    ref_w = quantised.dequantize()
    assert y.shape == (3, 5, 24) and torch.allclose(y, x.detach() @ ref_w.t(), atol=1e-5)
    y.square().sum().backward()
    want = (2 * y.detach()) @ ref_w
    assert torch.allclose(x.grad, want, atol=1e-4)
    assert Int8Gemms.calls[-1] == ("bwd", True, False)      # a frozen payload asks for no weight gradient

    # a stacked weight [2, 24, 16] multiplies as its flattened matrix and returns [..., 2, 24]
    stacked = RowScaledInt8Weight.quantise(torch.randn(2, 24, 16))
    layer.weight = nn.Parameter(stacked, requires_grad=False)
    assert layer(torch.randn(7, 16)).shape == (7, 2, 24)
    with pytest.raises(ValueError, match="input last dim"):
        layer(torch.randn(7, 8))
    with pytest.raises(NotImplementedError):
        FlexShardPrequantizedLinear(16, 16)(torch.randn(1, 16))


def test_converter_passes_dotted_names_and_skips_what_the_kernels_cannot_take():
    def net():
        m = nn.Module()
        m.block = nn.Sequential(nn.Linear(128, 256, bias=False), nn.Linear(256, 128, bias=False))
        m.head = nn.Linear(128, 128, bias=False)
        m.odd = nn.Linear(128, 100, bias=False)            # not a multiple of 128
        m.biased = nn.Linear(128, 128)
        return m

    seen = []
    m = convert_to_flex_shard_float8_blockwise_linear(net(), lambda fqn, lin: seen.append(fqn) or fqn != "head")
    assert sorted(seen) == ["block.0", "block.1", "head"]
    assert isinstance(m.block[0], FlexShardFloat8BlockwiseLinear) and isinstance(m.block[1], FlexShardFloat8BlockwiseLinear)
    assert type(m.head) is nn.Linear and type(m.odd) is nn.Linear and type(m.biased) is nn.Linear
    m2 = convert_to_flex_shard_prequantized_linear(net(), FlexShardMxfp8BlockwiseLinear)
    assert isinstance(m2.head, FlexShardMxfp8BlockwiseLinear) and type(m2.odd) is nn.Linear
    # a foreign layer class decides for itself what it can replace
    m3 = convert_to_flex_shard_prequantized_linear(net(), Int8Linear, lambda fqn, lin: lin.bias is None)
    assert isinstance(m3.odd, Int8Linear) and type(m3.biased) is nn.Linear
    again = convert_to_flex_shard_prequantized_linear(m3, Int8Linear, lambda fqn, lin: lin.bias is None)
    assert again.odd is m3.odd                              # already converted layers are left alone
