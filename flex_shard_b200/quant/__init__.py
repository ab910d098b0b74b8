"""Quantised weight wrappers and the linear layers that consume them."""
from .linear import (
    FlexShardFloat8BlockwiseLinear,
    FlexShardFloat8BlockwiseStackedLinear,
    FlexShardMxfp8BlockwiseLinear,
    FlexShardPrequantizedLinear,
    PrequantizedLinearGemms,
    convert_to_flex_shard_float8_blockwise_linear,
    convert_to_flex_shard_mxfp8_blockwise_linear,
    convert_to_flex_shard_prequantized_linear,
)
from .weight import (
    BlockwiseFp8Weight,
    BlockwiseMxfp8Weight,
    BlockwiseQuantWeight,
    blockwise_dequant_weight,
    blockwise_mxfp8_dequant_weight,
)


def __getattr__(name):
    # the comparison arm of the reference's FP8 tests is torchao's own layer, re-exported under this name
    # (``blockwise_fp8/fp8_blockwise_linear.py:25-28`` of the reference); torchao is not a dependency of this library
    if name == "TorchAOFloat8BlockwiseLinear":
        try:
            from torchao.prototype.blockwise_fp8_training.linear import Float8BlockwiseLinear
        except ImportError as e:
            raise AttributeError("TorchAOFloat8BlockwiseLinear needs the torchao package (not installed); "
                                 "FlexShardFloat8BlockwiseLinear on an unsharded module is the quantise-after-gather "
                                 "arm of this library") from e
        return Float8BlockwiseLinear
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
