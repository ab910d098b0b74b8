"""Built-in placements (storage schemes) and their ``placement_fn`` factories."""
from .block_shard import BlockShard, make_block_shard_placement_fn
from .bucketed_block_shard import BucketedBlockShard, FlatBucketPlan, make_bucketed_block_shard_placement_fn
from .mixed_bucket import MixedBucketPlacement, ShardSlice, make_mixed_placement_fn
from .owned import (
    BucketedOwned,
    make_bucketed_owned_expert_block_placement_fn,
    make_bucketed_owned_full_param_placement_fn,
    newton_schulz_cost,
)
from .shard import Shard, shard_placement_fn

__all__ = [
    "BlockShard", "BucketedBlockShard", "BucketedOwned", "FlatBucketPlan", "make_bucketed_block_shard_placement_fn", "MixedBucketPlacement", "Shard", "ShardSlice",
    "make_block_shard_placement_fn", "make_bucketed_owned_expert_block_placement_fn",
    "make_bucketed_owned_full_param_placement_fn", "make_mixed_placement_fn", "newton_schulz_cost",
    "shard_placement_fn",
]
