"""Placement helpers for DistMuon recipes: rank groups of a 2-D (efsdp x ep) layout, block partitions over a
mesh, and the ``placement_fn`` that stores a matrix in whole head blocks (so that each rank orthogonalises its
own heads with no exchange). Parity: ``dist_muon/placement.py:26-222`` of the reference."""
from __future__ import annotations

from dataclasses import dataclass

from ..placements.block_shard import BlockShard
from ..placements.mixed_bucket import make_mixed_placement_fn
from ..placements.shard import shard_placement_fn


@dataclass(frozen=True)
class BlockShardPlan:
    """Equal matrices packed one under the other along dim 0 of a 2-D parameter (attention heads, say):
    ``num_matrices`` of them.  The checks name the parameter.  Parity: ``dist_muon/placement.py:26-66`` of the
    reference."""

    num_matrices: int

    def __post_init__(self):
        if isinstance(self.num_matrices, bool) or not isinstance(self.num_matrices, int) or self.num_matrices <= 0:
            raise ValueError("num_matrices must be a positive integer")

    def validate_parameter(self, fqn: str, param) -> None:
        if param.ndim != 2:
            raise ValueError(f"matrix-sharded parameter {fqn!r} must be 2-D, but has shape {tuple(param.shape)}")
        if param.shape[0] % self.num_matrices:
            raise ValueError(f"matrix-sharded parameter {fqn!r} must have a dim 0 divisible by its "
                             f"{self.num_matrices} matrices, but has shape {tuple(param.shape)}")

    def matrix_rows(self, fqn: str, param) -> int:
        self.validate_parameter(fqn, param)
        return param.shape[0] // self.num_matrices

    def validate_matrix_extent(self, fqn: str, param, expected_matrix_extent: int) -> None:
        rows = self.matrix_rows(fqn, param)
        if rows != expected_matrix_extent:
            raise ValueError(f"matrix-sharded parameter {fqn!r} has matrices of {rows} rows, expected "
                             f"{expected_matrix_extent}")

    def blocks_per_rank(self, world_size: int) -> tuple[int, ...]:
        """Whole matrices per rank when they are dealt out as evenly as possible."""
        return get_dim0_block_partitions(self.num_matrices, world_size)


def get_mesh_rank_groups(world_size, group_size, *, rank_axis_name: str | None = None,
                         partition_axis_name: str | None = None):
    """``get_mesh_rank_groups(world_size, group_size)``: consecutive groups of ``group_size`` ranks (e.g. the
    expert-parallel groups of a job).

    ``get_mesh_rank_groups(flat_mesh, partitioned_mesh, rank_axis_name=..., partition_axis_name=...)``, the reference's
    form (``dist_muon/placement.py:69-104`` there): for every partition (index along ``partition_axis_name`` of the
    2-D mesh) the ranks that share it, as positions in the flat mesh, ordered along ``rank_axis_name``."""
    if not isinstance(world_size, int):
        flat_mesh, grid_mesh = world_size, group_size
        names = grid_mesh.mesh_dim_names
        if names is None or len(names) != 2 or set(names) != {rank_axis_name, partition_axis_name}:
            raise ValueError(f"the partition mesh must have exactly the axes {rank_axis_name!r} and "
                             f"{partition_axis_name!r}, got {names}")
        flat = [int(r) for r in flat_mesh.mesh.flatten().tolist()]
        grid = grid_mesh.mesh
        if sorted(int(r) for r in grid.flatten().tolist()) != sorted(flat):
            raise ValueError("the flat mesh and the partition mesh must hold the same ranks")
        position = {g: i for i, g in enumerate(flat)}
        by_axis = grid.permute(names.index(rank_axis_name), names.index(partition_axis_name))
        return tuple(tuple(position[int(g)] for g in by_axis[:, part].tolist()) for part in range(by_axis.shape[1]))
    if group_size <= 0 or world_size % group_size:
        raise ValueError(f"group size {group_size} does not divide the world size {world_size}")
    return [list(range(i, i + group_size)) for i in range(0, world_size, group_size)]


def get_strided_rank_groups(world_size: int, group_size: int) -> list[list[int]]:
    """The complementary groups: ranks at the same position of every consecutive group (e.g. the ranks that
    hold the same experts under expert parallelism and shard them among themselves)."""
    get_mesh_rank_groups(world_size, group_size)
    return [list(range(o, world_size, group_size)) for o in range(group_size)]


def get_dim0_block_partitions(num_blocks, world_size: int | None = None, *, num_partitions: int | None = None,
                              partition_index: int | None = None):
    """``get_dim0_block_partitions(num_blocks, world_size)``: blocks per rank when ``num_blocks`` whole blocks are
    dealt to ``world_size`` ranks as evenly as possible (the first ``num_blocks % world_size`` ranks hold one more).

    ``get_dim0_block_partitions(named_params, num_partitions=..., partition_index=...)``, the reference's form
    (``dist_muon/placement.py:107-161`` there): for stacked weights ``[blocks, ...]`` that an outer mesh axis cuts evenly
    along dim 0, ``((blocks of one partition, elements of one block over all the parameters),) * num_partitions``; with
    more than one partition every parameter must declare that layout (``set_global_layout``), this rank holding
    partition ``partition_index``."""
    if isinstance(num_blocks, int):
        base, rem = divmod(num_blocks, world_size)
        return tuple(base + (1 if r < rem else 0) for r in range(world_size))
    import math

    from ..placement_contract import GlobalLayout, get_global_layout

    fqn_params = list(num_blocks)
    if num_partitions is None or partition_index is None:
        raise TypeError("the parameter form needs num_partitions and partition_index")
    shapes = [tuple(p.shape) for _, p in fqn_params]
    if any(len(s) < 3 for s in shapes):
        raise ValueError("dimension-0 block parameters must have at least 3 dims ([blocks, rows, cols])")
    n = shapes[0][0]
    if n <= 0 or any(s[0] != n for s in shapes):
        raise ValueError("dimension-0 block parameters of one plan must hold the same, positive number of blocks")
    if num_partitions > 1:
        for (fqn, p), shape in zip(fqn_params, shapes):
            want = GlobalLayout((n * num_partitions, *shape[1:]), ((partition_index * n, *(0,) * (len(shape) - 1)),),
                                ((0,) * len(shape),), (shape,))
            if get_global_layout(p) != want:
                raise ValueError(f"partitioned block parameter {fqn!r} must declare a global layout that cuts dim 0 "
                                 f"evenly into {num_partitions} partitions, this rank holding partition "
                                 f"{partition_index} (set_global_layout)")
    return ((n, sum(math.prod(s[1:]) for s in shapes)),) * num_partitions


def make_bucketed_block_placement_fn(num_blocks_of):
    """``placement_fn`` storing every parameter as ``BlockShard`` over dim 0 in whole blocks;
    ``num_blocks_of(fqn, param)`` gives the number of blocks (attention heads, experts) of a parameter."""

    def fn(named_params, mesh):
        from ..parallel.comm import mesh_group

        _, _, W, _ = mesh_group(mesh)
        return {n: BlockShard(get_dim0_block_partitions(num_blocks_of(n, p), W), 0) for n, p in named_params}

    return fn


shard0_placement_fn = shard_placement_fn(0)
__all__ = ["BlockShardPlan", "get_mesh_rank_groups", "get_strided_rank_groups", "get_dim0_block_partitions", "make_mixed_placement_fn",
           "shard0_placement_fn", "make_bucketed_block_placement_fn"]
