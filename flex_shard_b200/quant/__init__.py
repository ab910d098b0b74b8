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
