"""Muon for sharded models: owner-local Newton-Schulz on tcgen05, planners and adapters."""
from .bucket_planner import (AssignmentGroup, MatrixAssignment, MatrixAssignmentFn, MatrixBlockGroupSpec, MatrixSpec,
                             PackedParameterPlan, ParameterBucketPlan, WholeMatrixSpec, assign_matrices, materialize_dist_muon_buckets, validate_assignment)
from .comm_free_adapter import build_local_dist_muon, load_muon_checkpoint_state, muon_checkpoint_state
from .optimizer import DistMuon, LocalMuonComputeLayout, lr_ratio

# what build_local_dist_muon returns: the optimizer itself (it steps the real local tensors; no proxy parameters)
LocalDistMuonBinding = DistMuon
from .optimizer_reshard import BlockShard, BucketConfig, ComputeLayout, Owned
from .placement import BlockShardPlan
from .storage_layout import capture_flex_shard_muon_canonical_shards, get_flex_shard_muon_compute_layouts

__all__ = ["AssignmentGroup", "MatrixAssignment", "MatrixAssignmentFn", "MatrixBlockGroupSpec", "PackedParameterPlan", "ParameterBucketPlan", "WholeMatrixSpec",
           "BlockShard", "BlockShardPlan", "BucketConfig", "ComputeLayout", "DistMuon", "LocalDistMuonBinding", "LocalMuonComputeLayout", "MatrixSpec", "Owned",
           "assign_matrices", "build_local_dist_muon", "capture_flex_shard_muon_canonical_shards",
           "get_flex_shard_muon_compute_layouts", "lr_ratio", "load_muon_checkpoint_state", "materialize_dist_muon_buckets", "muon_checkpoint_state", "validate_assignment"]
