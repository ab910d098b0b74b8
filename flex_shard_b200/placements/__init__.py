"""Built-in placements (storage schemes) and their ``placement_fn`` factories."""
from .block_shard import BlockShard, make_block_shard_placement_fn
from .blockwise_quant import (
    BlockwiseQuantBucketedBlockShard,
    Fp8BucketedBlockShard,
    Mxfp8BucketedBlockShard,
    BlockwiseFp8WeightFactory,
    BlockwiseMxfp8WeightFactory,
    make_mxfp8_bucketed_block_shard_placement_fn,
    make_fp8_bucketed_block_shard_placement_fn,
    partition_min_max,
    plan_row_ranges,
)
from .bucketed_block_shard import BucketedBlockShard, FlatBucketPlan, make_bucketed_block_shard_placement_fn
from .mixed_bucket import MixedBucketPlacement, ShardSlice, make_mixed_placement_fn
from .owned import (
    BucketedOwned,
    BucketedOwnedSegmentSpec,
    make_bucketed_owned_expert_block_placement_fn,
    make_bucketed_owned_expert_block_segments,
    make_bucketed_owned_full_param_segments,
    make_bucketed_owned_full_param_placement_fn,
    newton_schulz_cost,
)
from .shard import Shard, shard_placement_fn

# the names these factories have in the reference package (``custom_placements/__init__.py``)
make_shard_placement_fn = shard_placement_fn
make_bucketed_block_placement_fn = make_bucketed_block_shard_placement_fn
make_fp8_bucketed_block_placement_fn = make_fp8_bucketed_block_shard_placement_fn
make_mxfp8_bucketed_block_placement_fn = make_mxfp8_bucketed_block_shard_placement_fn


def per_param_placements(named_params, mesh):
    """``Shard(0)`` for every parameter (FSDP2-style)."""
    return shard_placement_fn(0)(named_params, mesh)


__all__ = [
    "BlockShard", "BlockwiseQuantBucketedBlockShard", "Fp8BucketedBlockShard", "make_fp8_bucketed_block_shard_placement_fn",
    "Mxfp8BucketedBlockShard", "make_mxfp8_bucketed_block_shard_placement_fn",
    "partition_min_max", "plan_row_ranges", "BucketedBlockShard", "BucketedOwned", "BucketedOwnedSegmentSpec",
    "make_bucketed_owned_expert_block_segments", "make_bucketed_owned_full_param_segments", "FlatBucketPlan", "make_bucketed_block_shard_placement_fn", "MixedBucketPlacement", "Shard", "ShardSlice",
    "make_block_shard_placement_fn", "make_bucketed_owned_expert_block_placement_fn",
    "make_bucketed_owned_full_param_placement_fn", "make_mixed_placement_fn", "newton_schulz_cost",
    "shard_placement_fn", "make_shard_placement_fn", "per_param_placements", "make_bucketed_block_placement_fn",
    "make_fp8_bucketed_block_placement_fn", "make_mxfp8_bucketed_block_placement_fn",
    "BlockwiseFp8WeightFactory", "BlockwiseMxfp8WeightFactory",
]
