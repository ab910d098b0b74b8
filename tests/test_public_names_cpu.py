"""Every public name of the reference's packages (their ``__all__`` lists, restated here) resolves under the package
mapping of the README, except one that describes an internal this design does not have."""
import importlib

import pytest

NAMES = {
    "flex_shard_b200": """BucketParamStorageLayout BucketSpec BucketStorageLayout GlobalLayout GradientReduction
        flex_shard get_flex_shard_global_layouts get_global_layout get_global_shape get_mesh get_outer_layout
        get_partial_grad_group get_placements init_from_full is_flex_shard_param LocalStorageLayout
        MixedPrecisionPolicy OffloadPolicy Placement PlacementFn register_optimizer_checkpoint_hook relayout_bucket
        set_global_layout set_partial_grad_group set_state_dict_global_layouts""",
    "flex_shard_b200.quant": """blockwise_dequant_weight BlockwiseFp8Weight convert_to_flex_shard_float8_blockwise_linear
        FlexShardFloat8BlockwiseLinear blockwise_mxfp8_dequant_weight BlockwiseMxfp8Weight
        convert_to_flex_shard_mxfp8_blockwise_linear FlexShardMxfp8BlockwiseLinear BlockwiseQuantWeight
        convert_to_flex_shard_prequantized_linear FlexShardPrequantizedLinear PrequantizedLinearGemms""",
    "flex_shard_b200.placements": """BucketedOwned BucketedOwnedSegmentSpec make_bucketed_owned_expert_block_placement_fn
        make_bucketed_owned_expert_block_segments make_bucketed_owned_full_param_placement_fn
        make_bucketed_owned_full_param_segments make_shard_placement_fn MixedBucketPlacement BlockwiseFp8WeightFactory
        BlockwiseMxfp8WeightFactory make_mxfp8_bucketed_block_placement_fn Mxfp8BucketedBlockShard
        BlockwiseQuantBucketedBlockShard Fp8BucketedBlockShard BucketedBlockShard make_fp8_bucketed_block_placement_fn
        make_bucketed_block_placement_fn per_param_placements BlockShard Shard""",
    "flex_shard_b200.dist_muon": """assign_matrices AssignmentGroup BlockShard BlockShardPlan BucketConfig
        build_local_dist_muon capture_flex_shard_muon_canonical_shards ComputeLayout DistMuon
        get_flex_shard_muon_compute_layouts LocalDistMuonBinding LocalMuonComputeLayout materialize_dist_muon_buckets
        MatrixAssignment MatrixAssignmentFn MatrixBlockGroupSpec Owned PackedParameterPlan ParameterBucketPlan
        WholeMatrixSpec""",
    "flex_shard_b200.layout_adapters": "dtensor_to_global_layout",
}
NOT_PROVIDED = {"flex_shard_b200.dist_muon": ["LocalMuonStateShard"]}


@pytest.mark.parametrize("package", sorted(NAMES))
def test_reference_names_resolve(package):
    mod = importlib.import_module(package)
    missing = [n for n in NAMES[package].split() if not hasattr(mod, n)]
    assert not missing, missing
    listed = getattr(mod, "__all__", None)
    if listed is not None:
        assert not [n for n in listed if not hasattr(mod, n)]
    for n in NOT_PROVIDED.get(package, []):
        assert not hasattr(mod, n)          # if one of these appears, the README's note on it is out of date


def test_torchao_layer_is_a_lazy_re_export():
    import flex_shard_b200.quant as q

    try:
        import torchao  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError):
            from flex_shard_b200.quant import TorchAOFloat8BlockwiseLinear  # noqa: F401
    else:
        # the real package, or the import placeholder that the reference arm's compatibility shims install in this
        # process: either way the name resolves through the lazy re-export
        assert q.TorchAOFloat8BlockwiseLinear is not None
