"""flex_shard_b200: a Blackwell-native data-parallel sharding library.

Public API (same names as the reference's ``flex_shard`` package,
``src/flex_shard/__init__.py:7-62``).
"""
import os as _os

# Kernels of this library wait for flags that peers set from their own kernels. With CUDA's lazy kernel loading
# the first launch of any kernel may have to wait for the context to go idle, which it does not while a wait
# kernel spins; two ranks can then hold each other up until the waits run out. Eager loading (read by CUDA when
# it initialises, so this must run before the first CUDA call of the process) removes the window.
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")

from .bucket_storage import BucketSpec, MixedPrecisionPolicy, OffloadPolicy, PlacementFn, ShardedBucketStorage
from .checkpoint import (
    get_flex_shard_global_layouts,
    register_optimizer_checkpoint_hook,
    set_state_dict_global_layouts,
)
from .flex_shard import FlexShardModule, flex_shard, relayout_bucket
from .param_init import init_from_full
from .placement_contract import (
    BucketParamStorageLayout,
    BucketStorageLayout,
    GlobalLayout,
    GradientReduction,
    LocalStorageLayout,
    Placement,
    compose_global_layouts,
    get_global_layout,
    get_partial_grad_group,
    set_global_layout,
    set_partial_grad_group,
)
from .sharded_param import get_global_shape, get_mesh, get_outer_layout, get_placements, is_flex_shard_param

__all__ = [
    "BucketParamStorageLayout", "BucketSpec", "BucketStorageLayout", "FlexShardModule", "GlobalLayout",
    "GradientReduction", "LocalStorageLayout", "MixedPrecisionPolicy", "OffloadPolicy", "Placement",
    "PlacementFn", "ShardedBucketStorage", "compose_global_layouts", "flex_shard",
    "get_flex_shard_global_layouts", "get_global_layout", "get_global_shape", "get_mesh", "get_outer_layout",
    "get_partial_grad_group", "get_placements", "init_from_full", "is_flex_shard_param",
    "register_optimizer_checkpoint_hook", "relayout_bucket", "set_global_layout", "set_partial_grad_group",
    "set_state_dict_global_layouts",
]
