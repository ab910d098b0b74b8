"""Owner assignment for Muon matrices: hosts before ranks, alternating positions on ties, loads carried from
bucket to bucket, block groups, fixed owners.  Pure planning, no process group.
Parity: the behaviours pinned by the reference's ``tests/test_matrix_assignment.py:72-361``."""
import pytest


def test_mesh_rank_hosts(monkeypatch):
    from flex_shard_b200.utils.validation import mesh_rank_hosts

    assert mesh_rank_hosts(8, 4) == (0, 0, 0, 0, 1, 1, 1, 1)
    assert mesh_rank_hosts(6, 4) == (0, 0, 0, 0, 1, 1)               # the last host may be smaller
    assert mesh_rank_hosts(4, 16) == (0, 0, 0, 0)                    # more slots than ranks: one host
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")
    assert mesh_rank_hosts(4) == (0, 0, 1, 1)                        # torchrun's value when nothing is given
    monkeypatch.delenv("LOCAL_WORLD_SIZE")
    assert mesh_rank_hosts(4) == (0, 0, 0, 0)


def test_one_host_alternates_ranks_and_equal_items_fill_even_positions_first():
    from flex_shard_b200.utils.validation import assign_to_hosts_then_ranks

    # 8 equal items on one host of 8 ranks: ranks are taken in the order 0, 2, 4, 6, 1, 3, 5, 7
    assert assign_to_hosts_then_ranks([1.0] * 8, [0] * 8) == [0, 2, 4, 6, 1, 3, 5, 7]
    # the ninth item lands on the first rank again
    assert assign_to_hosts_then_ranks([1.0] * 9, [0] * 8)[-1] == 0


def test_heavy_and_light_items_alternate_over_hosts():
    from flex_shard_b200.utils.validation import assign_to_hosts_then_ranks

    hosts = [0, 0, 1, 1, 2, 2, 3, 3]
    owners = assign_to_hosts_then_ranks([8.0, 8.0, 8.0, 8.0, 1.0, 1.0, 1.0, 1.0], hosts)
    heavy_hosts = [hosts[r] for r in owners[:4]]
    light_hosts = [hosts[r] for r in owners[4:]]
    assert sorted(heavy_hosts) == [0, 1, 2, 3] and sorted(light_hosts) == [0, 1, 2, 3]   # one of each per host
    assert heavy_hosts == [0, 2, 1, 3]                                                    # even hosts first on ties
    # a light item never shares a rank with a heavy one while a free rank exists on that host
    assert not set(owners[:4]) & set(owners[4:])


def test_loads_are_updated_in_place_and_steer_the_next_call():
    from flex_shard_b200.utils.validation import assign_to_hosts_then_ranks

    loads = [0.0, 0.0, 0.0, 0.0]
    first = assign_to_hosts_then_ranks([5.0], [0, 0, 1, 1], loads)
    assert first == [0] and loads == [5.0, 0.0, 0.0, 0.0]
    second = assign_to_hosts_then_ranks([5.0], [0, 0, 1, 1], loads)
    assert second == [2] and loads == [5.0, 0.0, 5.0, 0.0]        # the lighter host first, then its first rank
    third = assign_to_hosts_then_ranks([1.0, 1.0], [0, 0, 1, 1], loads)
    assert sorted(third) == [1, 3]


def test_groups_balance_separately_unless_loads_are_carried():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    big, small = (256, 256), (64, 64)
    groups = [[MatrixSpec(f"l{i}.big", big), MatrixSpec(f"l{i}.small", small)] for i in range(4)]
    apart = assign_matrices(groups, 4, ranks_per_host=4, carry_loads=False)
    # every group starts from empty loads: all big matrices land on the same rank
    assert len({apart[f"l{i}.big"] for i in range(4)}) == 1
    carried = assign_matrices(groups, 4, ranks_per_host=4, carry_loads=True)
    assert len({carried[f"l{i}.big"] for i in range(4)}) == 4       # spread over the mesh
    # the order of the groups decides who gets what when loads are carried
    flipped = assign_matrices(list(reversed(groups)), 4, ranks_per_host=4, carry_loads=True)
    assert flipped["l3.big"] == carried["l0.big"]


def test_block_groups_use_the_accumulated_load():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    whole = MatrixSpec("dense", (512, 512))
    heads = MatrixSpec("wq", (8 * 64, 512), num_blocks=8)
    out = assign_matrices([[whole, heads]], 4, ranks_per_host=4)
    counts = out["wq"]
    assert sum(counts) == 8 and len(counts) == 4
    assert counts[out["dense"]] == min(counts)                       # the rank that owns the dense matrix gets fewest heads


def test_fixed_owners_are_kept_and_counted():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    ms = [MatrixSpec(f"m{i}", (128, 128)) for i in range(4)]
    out = assign_matrices([ms], 2, fixed_owners={"m0": 1, "m1": 1})
    assert out["m0"] == 1 and out["m1"] == 1
    assert out["m2"] == 0 and out["m3"] == 0                          # the free ones fill the lighter rank
    with pytest.raises(ValueError, match="not a rank"):
        assign_matrices([ms], 2, fixed_owners={"m0": 5})


def test_duplicate_names_are_rejected():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    with pytest.raises(ValueError, match="more than once"):
        assign_matrices([[MatrixSpec("w", (8, 8))], [MatrixSpec("w", (8, 8))]], 2)


def test_owned_placement_fn_carries_loads_across_buckets_and_puts_hosts_first():
    import torch
    import torch.nn as nn

    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn
    from tests.common import FakeMesh

    fn = make_bucketed_owned_full_param_placement_fn(carry_loads=True, ranks_per_host=2)
    owners = []
    for b in range(4):                                               # four identical one-matrix buckets
        named = [(f"b{b}.w", nn.Parameter(torch.zeros(64, 64)))]
        pl = fn(named, FakeMesh(4))[f"b{b}.w"]
        owners.append(pl.segments[0][0])
    assert sorted(owners) == [0, 1, 2, 3]                            # carried loads spread them over all ranks
    assert owners[:2] in ([0, 2], [2, 0])                            # the two hosts are used before a host's second rank
    fresh = make_bucketed_owned_full_param_placement_fn(carry_loads=False, ranks_per_host=2)
    same = {fresh([(f"b{b}.w", nn.Parameter(torch.zeros(64, 64)))], FakeMesh(4))[f"b{b}.w"].segments[0][0] for b in range(4)}
    assert len(same) == 1


def test_block_groups_can_be_confined_to_eligible_ranks():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    heads = MatrixSpec("wq", (8 * 64, 256), num_blocks=8, eligible_ranks=(2, 3))
    out = assign_matrices([[heads]], 4, ranks_per_host=4)
    assert out["wq"] == (0, 0, 4, 4)
    with pytest.raises(ValueError, match="eligible_ranks"):
        assign_matrices([[MatrixSpec("wq", (512, 256), num_blocks=8, eligible_ranks=(7,))]], 4)


def test_custom_assignment_is_used_and_checked():
    import torch
    import torch.nn as nn

    from flex_shard_b200.dist_muon import MatrixSpec, materialize_dist_muon_buckets, validate_assignment
    from flex_shard_b200.placements import BucketedOwned
    from tests.common import FakeMesh

    named = [("emb.weight", nn.Parameter(torch.zeros(32, 8))), ("l0.w", nn.Parameter(torch.zeros(16, 8))),
             ("l0.v", nn.Parameter(torch.zeros(8, 16))), ("l0.norm", nn.Parameter(torch.zeros(8)))]
    seen = {}

    def everything_on_the_last_rank(groups, *, num_ranks):
        seen["groups"] = [[m.fqn for m in g] for g in groups]
        return {m.fqn: num_ranks - 1 for g in groups for m in g}

    specs = materialize_dist_muon_buckets(named, FakeMesh(4), initial=["emb"], blocks=[["l0"]], final=[],
                                          assignment_fn=everything_on_the_last_rank)
    assert seen["groups"] == [["l0.w", "l0.v"]]                       # matrices of the block buckets only
    block_spec = specs[1]
    pls = block_spec.placement_fn([n for n in named if n[0].startswith("l0")], FakeMesh(4))
    owned = {f: pl.member for f, pl in pls.items() if isinstance(pl.member, BucketedOwned)}
    assert {f: pl.segments[0][0] for f, pl in owned.items()} == {"l0.w": 3, "l0.v": 3}
    # answers that do not fit the recipe are refused before any bucket exists
    groups = [[MatrixSpec("a", (8, 8)), MatrixSpec("h", (64, 8), num_blocks=4)]]
    validate_assignment(groups, 2, {"a": 1, "h": (1, 3)})
    for bad, msg in (({"a": 1}, "missing"), ({"a": 1, "h": (2, 2), "x": 0}, "unexpected"), ({"a": 2, "h": (2, 2)}, "rank in"),
                     ({"a": 0, "h": (1, 2)}, "sum to 4"), ({"a": 0, "h": (4,)}, "2 non-negative")):
        with pytest.raises(ValueError, match=msg):
            validate_assignment(groups, 2, bad)
    with pytest.raises(ValueError, match="missing"):
        materialize_dist_muon_buckets(named, FakeMesh(4), initial=["emb"], blocks=[["l0"]], final=[],
                                      assignment_fn=lambda groups, *, num_ranks: {})


def test_recipe_types_of_the_reference_are_accepted():
    """``assign_matrices`` over ``AssignmentGroup``s (element counts as loads, carried from group to group) answers
    with a ``MatrixAssignment``; goldens restated from ``tests/test_matrix_assignment.py:73-165`` of the reference.
    A custom balancer may answer ``materialize_dist_muon_buckets`` in that form too."""
    import torch
    import torch.nn as nn

    from flex_shard_b200.dist_muon import (AssignmentGroup, MatrixAssignment, MatrixBlockGroupSpec, WholeMatrixSpec,
                                           assign_matrices, materialize_dist_muon_buckets)
    from flex_shard_b200.placements import BlockShard
    from tests.common import FakeMesh

    a = assign_matrices((AssignmentGroup((WholeMatrixSpec("attention", 100),)),
                         AssignmentGroup((WholeMatrixSpec("ff0", 60), WholeMatrixSpec("ff1", 60)))), num_ranks=2)
    assert a.rank_by_matrix["attention"] == 0 and {a.rank_by_matrix["ff0"], a.rank_by_matrix["ff1"]} == {0, 1}
    q, w = AssignmentGroup((WholeMatrixSpec("q", 100),)), AssignmentGroup((WholeMatrixSpec("w", 60),))
    assert assign_matrices((q, w), num_ranks=2).rank_by_matrix == {"q": 0, "w": 1}
    assert assign_matrices((w, q), num_ranks=2).rank_by_matrix == {"w": 0, "q": 1}
    with pytest.raises(ValueError, match="Duplicate assignment name"):
        assign_matrices((q, q), num_ranks=2)
    b = assign_matrices((AssignmentGroup((WholeMatrixSpec("matrix", 100),),
                                         (MatrixBlockGroupSpec("heads", 2, 60, (0, 1)),)),), num_ranks=2)
    assert b.rank_by_matrix == {"matrix": 0} and b.blocks_per_rank_by_group == {"heads": (0, 2)}
    # counts follow the order of eligible_ranks, and blocks stay inside them
    c = assign_matrices((AssignmentGroup((), (MatrixBlockGroupSpec("heads", 5, 10, (3, 1)),)),), num_ranks=4)
    assert c.blocks_per_rank_by_group == {"heads": (3, 2)}
    # with hosts, the two heaviest matrices land on different hosts
    d = assign_matrices((AssignmentGroup(tuple(WholeMatrixSpec(f"m{i}", 100 - i) for i in range(4))),), num_ranks=4,
                        hosts=(0, 0, 1, 1))
    assert {d.rank_by_matrix["m0"] // 2, d.rank_by_matrix["m1"] // 2} == {0, 1}
    for bad in ((AssignmentGroup((WholeMatrixSpec("z", 0),)),),
                (AssignmentGroup((), (MatrixBlockGroupSpec("h", 2, 8, (0, 0)),)),),
                (AssignmentGroup((), (MatrixBlockGroupSpec("h", 2, 8, (5,)),)),)):
        with pytest.raises(ValueError):
            assign_matrices(bad, num_ranks=2)
    with pytest.raises(ValueError, match="hosts"):
        assign_matrices((q,), num_ranks=2, hosts=(0,))

    named = [("l0.w", nn.Parameter(torch.zeros(16, 8))), ("l0.heads", nn.Parameter(torch.zeros(32, 8)))]

    def custom(groups, *, num_ranks):
        return MatrixAssignment({"l0.w": 1}, {"l0.heads": (1, 3)})

    specs = materialize_dist_muon_buckets(named, FakeMesh(2), initial=[], blocks=[["l0"]], final=[],
                                          num_blocks_of=lambda n, p: 4 if n.endswith("heads") else 1,
                                          assignment_fn=custom)
    pls = specs[0].placement_fn(named, FakeMesh(2))
    assert pls["l0.w"].member.segments[0][0] == 1
    assert isinstance(pls["l0.heads"].member, BlockShard) and tuple(pls["l0.heads"].member.blocks_per_rank) == (1, 3)


class _Mesh:
    """Stand-in for a DeviceMesh in planner tests: ranks as a tensor, axis names, this rank's coordinates."""

    def __init__(self, ranks, names=None, coords=None):
        import torch

        self.mesh = torch.tensor(ranks)
        self.mesh_dim_names = names
        self._coords = coords or {}
        self.world_size, self.rank, self.ndim, self.device = self.mesh.numel(), 0, self.mesh.dim(), "cpu"

    def size(self):
        return self.mesh.numel()

    def get_local_rank(self, axis=None):
        return self._coords.get(axis, 0)

    def __getitem__(self, axis):
        i = self.mesh_dim_names.index(axis)
        other = 1 - i
        line = self.mesh.select(other, self._coords[self.mesh_dim_names[other]])
        return _Mesh(line.tolist(), (axis,), {axis: self._coords[axis]})


def test_recipe_form_of_the_bucket_materializer():
    """``bucket_plans``: owned + packed parameters in a mixed bucket, partitioned expert weights in a flat block
    bucket on the partition's own ranks, ``Shard(0)`` around them, every bucket summing its gradients.  Restated from
    ``tests/test_matrix_assignment.py:41-71,166-260`` of the reference."""
    import torch
    import torch.distributed as dist
    import torch.nn as nn

    from flex_shard_b200 import GlobalLayout, set_global_layout
    from flex_shard_b200.dist_muon import (BlockShardPlan, MatrixAssignment, PackedParameterPlan, ParameterBucketPlan,
                                           materialize_dist_muon_buckets)
    from flex_shard_b200.placements import BlockShard, BucketedBlockShard, BucketedOwned, Shard

    owned, blocks = nn.Parameter(torch.empty(2, 2)), nn.Parameter(torch.empty(4, 2, 3))
    plan = ParameterBucketPlan(mixed_fqns=("owned",), owned_parameters=(("owned", owned),),
                               partitioned_parameters=(("blocks", blocks),), partition_group_name_prefix="blocks#")
    common = dict(bucket_plans=(plan,), assignment_name_by_fqn={"owned": "matrix"}, initial_sharded_fqns=(),
                  final_sharded_fqn_groups=(), assignment_mesh=_Mesh([0, 1]), partition_mesh=None,
                  partition_rank_axis_name="rank", partition_axis_name="partition")
    seen = {}

    def custom(groups, *, num_ranks):
        seen["n"], seen["groups"] = num_ranks, groups
        return MatrixAssignment({"matrix": 1}, {"blocks#0": (1, 3)})

    specs = materialize_dist_muon_buckets(**common, assignment_fn=custom)
    assert seen["n"] == 2 and len(seen["groups"]) == 1
    assert seen["groups"][0].block_groups[0].block_numel == 6 and seen["groups"][0].block_groups[0].num_blocks == 4
    assert [s.gradient_reduce_op for s in specs] == [dist.ReduceOp.SUM] * 2
    pl = specs[0].placement_fn([("owned", owned)], common["assignment_mesh"])["owned"]
    assert isinstance(pl.member, BucketedOwned) and pl.member.segments == ((1, 0, 2),)
    bp = specs[1].placement_fn([("blocks", blocks)], common["assignment_mesh"])["blocks"]
    assert isinstance(bp, BucketedBlockShard) and tuple(bp.blocks_per_rank) == (1, 3)
    for bad, msg in ((MatrixAssignment({}, {"blocks#0": (1, 3)}), "Matrix assignment names"),
                     (MatrixAssignment({"matrix": 1}, {}), "Block group names"),
                     (MatrixAssignment({"matrix": 2}, {"blocks#0": (1, 3)}), "rank in"),
                     (MatrixAssignment({"matrix": 1}, {"blocks#0": (1, 2)}), "sum to 4"),
                     (MatrixAssignment({"matrix": 1}, {"blocks#0": (4,)}), "2 non-negative")):
        with pytest.raises(ValueError, match=msg):
            materialize_dist_muon_buckets(**common, assignment_fn=lambda g, *, num_ranks, bad=bad: bad)
    with pytest.raises(TypeError, match="MatrixAssignment"):
        materialize_dist_muon_buckets(**common, assignment_fn=lambda g, *, num_ranks: {"matrix": 1})

    # the built-in balancer, a packed parameter (4 heads of 2 rows) and the buckets around the blocks
    heads = nn.Parameter(torch.empty(8, 3))
    plan2 = ParameterBucketPlan(mixed_fqns=("owned", "heads", "norm"), owned_parameters=(("owned", owned),),
                                packed_parameters=(PackedParameterPlan("heads", heads, BlockShardPlan(4)),))
    specs = materialize_dist_muon_buckets(bucket_plans=(plan2,), assignment_name_by_fqn={"owned": "o", "heads": "h"},
                                          initial_sharded_fqns=("emb",), final_sharded_fqn_groups=(("norm_f",), ()),
                                          assignment_mesh=_Mesh([0, 1]))
    assert [s.patterns for s in specs] == [("emb",), ("owned", "heads", "norm"), ("norm_f",)]
    assert [s.reshard_after_forward for s in specs] == [True, True, False]
    pls = specs[1].placement_fn([("owned", owned), ("heads", heads), ("norm", nn.Parameter(torch.empty(3)))], None)
    assert isinstance(pls["heads"].member, BlockShard) and sum(pls["heads"].member.blocks_per_rank) == 4
    assert isinstance(pls["norm"].member, Shard) or pls["norm"].member.__class__.__name__ == "ShardSlice"
    with pytest.raises(ValueError, match="divisible"):
        materialize_dist_muon_buckets(
            bucket_plans=(ParameterBucketPlan(packed_parameters=(PackedParameterPlan("heads", heads, BlockShardPlan(3)),)),),
            assignment_name_by_fqn={"heads": "h"}, assignment_mesh=_Mesh([0, 1]))

    # experts cut by an outer axis: 4 ranks as efsdp x ep = 2 x 2, this rank at (efsdp 1, ep 1)
    flat = _Mesh([0, 1, 2, 3])
    grid = _Mesh([[0, 1], [2, 3]], ("efsdp", "ep"), {"efsdp": 1, "ep": 1})
    experts = nn.Parameter(torch.empty(4, 2, 3))           # this partition's 4 of 8 experts
    eplan = ParameterBucketPlan(partitioned_parameters=(("experts", experts),), partition_group_name_prefix="e#")
    args = dict(bucket_plans=(eplan,), assignment_name_by_fqn={}, assignment_mesh=flat, partition_mesh=grid,
                partition_rank_axis_name="efsdp", partition_axis_name="ep")
    with pytest.raises(ValueError, match="set_global_layout"):
        materialize_dist_muon_buckets(**args)
    set_global_layout(experts, GlobalLayout((8, 2, 3), ((4, 0, 0),), ((0, 0, 0),), ((4, 2, 3),)))

    def spy(groups, *, num_ranks):
        seen["eligible"] = [b.eligible_ranks for b in groups[0].block_groups]
        return MatrixAssignment({}, {"e#0": (4, 0), "e#1": (1, 3)})

    (spec,) = materialize_dist_muon_buckets(**args, assignment_fn=spy)
    assert seen["eligible"] == [(0, 2), (1, 3)]              # ranks sharing ep 0, ranks sharing ep 1
    assert spec.mesh.mesh.tolist() == [1, 3]                 # stored on this partition's ranks
    assert tuple(spec.placement_fn([("experts", experts)], spec.mesh)["experts"].blocks_per_rank) == (1, 3)
    with pytest.raises(ValueError, match="exactly the axes"):
        materialize_dist_muon_buckets(**{**args, "partition_axis_name": "pp"})


_MOE_LAYER = (7168 * 16384, 1536 * 7168, 2048 * 7168, 2048 * 7168, 7168 * 2048, 256 * 7168)


def test_two_level_owner_goldens_of_the_reference(monkeypatch):
    """Hosts first, then ranks, through the reference's call forms; goldens restated from
    ``tests/test_matrix_assignment.py:266-360`` of the reference (one MoE layer of DeepSeek-V3 671B: attention ``wo``
    and ``wq_a``, the shared experts' three matrices, the router)."""
    import torch
    import torch.nn as nn

    from flex_shard_b200.dist_muon import AssignmentGroup, WholeMatrixSpec, assign_matrices
    from flex_shard_b200.placements import make_bucketed_owned_full_param_segments
    from flex_shard_b200.utils.validation import assign_to_hosts_then_ranks, mesh_rank_hosts

    assert mesh_rank_hosts(range(8), 4) == (0, 0, 0, 0, 1, 1, 1, 1)
    assert mesh_rank_hosts((64, 65, 72, 73), 8) == (0, 0, 1, 1)      # global ranks of a sub-mesh, hosts in mesh order
    assert mesh_rank_hosts(range(4), 1) == (0, 1, 2, 3)
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")
    assert mesh_rank_hosts(range(4)) == (0, 0, 1, 1)
    monkeypatch.delenv("LOCAL_WORLD_SIZE")

    # four MoE layers on 64 ranks of 8 hosts: each wo exceeds a host's share, so the hosts that hold one alternate
    # with the others in rank order, and a second bucket on top of the carried loads flips them
    hosts = mesh_rank_hosts(range(64), 8)
    group = AssignmentGroup(tuple(WholeMatrixSpec(f"layer{l}.m{i}", n) for l in range(4) for i, n in enumerate(_MOE_LAYER)))
    a = assign_matrices((group,), num_ranks=64, hosts=hosts)
    assert sorted(hosts[a.rank_by_matrix[f"layer{l}.m0"]] for l in range(4)) == [0, 2, 4, 6]
    per_host = [0] * 8
    for m in group.matrices:
        per_host[hosts[a.rank_by_matrix[m.name]]] += m.numel
    assert per_host[0::2] == [_MOE_LAYER[0]] * 4 and per_host[1::2] == [sum(_MOE_LAYER) - _MOE_LAYER[0]] * 4
    carried = [sum(m.numel for m in group.matrices if a.rank_by_matrix[m.name] == r) for r in range(64)]
    second = assign_to_hosts_then_ranks([m.numel for m in group.matrices], hosts, carried_loads=carried, one_per_rank=True)
    assert sorted(hosts[second[6 * l]] for l in range(4)) == [1, 3, 5, 7]

    eight = AssignmentGroup(tuple(WholeMatrixSpec(f"m{i}", n) for i, n in enumerate((100,) * 4 + (10,) * 4)))
    one_host = assign_matrices((eight,), num_ranks=8, hosts=(0,) * 8)
    assert sorted(one_host.rank_by_matrix[f"m{i}"] for i in range(4)) == [0, 2, 4, 6]

    six = AssignmentGroup(tuple(WholeMatrixSpec(f"m{i}", n) for i, n in enumerate((100, 100, 10, 10, 10, 10))))
    two_level = assign_matrices((six,), num_ranks=8, hosts=mesh_rank_hosts(range(8), 4))
    rank_order = assign_matrices((six,), num_ranks=8)
    assert {two_level.rank_by_matrix[m] for m in ("m0", "m1")} == {0, 4}
    assert {rank_order.rank_by_matrix[m] for m in ("m0", "m1")} == {0, 1}

    named = [(f"p{i}", nn.Parameter(torch.empty(n))) for i, n in enumerate((100, 100, 10, 10))]
    hosts_first = make_bucketed_owned_full_param_segments(named, 8, hosts=mesh_rank_hosts(range(8), 4))
    plain = make_bucketed_owned_full_param_segments(named, 8)
    assert {hosts_first[p][0].owner_rank for p in ("p0", "p1")} == {0, 4}
    assert {plain[p][0].owner_rank for p in ("p0", "p1")} == {0, 1}
    with pytest.raises(ValueError, match="one per rank"):
        assign_to_hosts_then_ranks([1, 1, 1], (0, 0), one_per_rank=True)
    with pytest.raises(ValueError, match="numbered"):
        assign_to_hosts_then_ranks([1], (0, 2), carried_loads=[0, 0])


def test_sixteen_identical_blocks_on_64_ranks(monkeypatch):
    """16 identical buckets of a DeepSeek-V3 MoE block's owned matrices on 64 ranks of 8 hosts: placed one at a time
    every bucket gets the same 6 owners; carrying the loads spreads them, each rank owning at most one ``wo`` and
    about a fair share in all.  Restated from ``tests/test_matrix_assignment.py:361-404`` of the reference."""
    import torch
    import torch.nn as nn

    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn
    from tests.common import FakeMesh

    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    shapes = ((7168, 16384), (1536, 7168), (576, 7168), (256, 7168), (2, 2048, 7168), (7168, 2048))

    def owned_numel(fn):
        loads = [0] * 64
        for block in range(16):
            named = [(f"layers.{block}.m{i}", nn.Parameter(torch.empty(s, device="meta"))) for i, s in enumerate(shapes)]
            sizes = {f: p.numel() for f, p in named}
            for f, pl in fn(named, FakeMesh(64)).items():
                for r, _, _ in pl.segments:
                    loads[r] += sizes[f]
        return loads

    per_bucket = owned_numel(make_bucketed_owned_full_param_placement_fn())
    carried = owned_numel(make_bucketed_owned_full_param_placement_fn(carry_loads=True))
    assert sum(load > 0 for load in per_bucket) == 6 and max(per_bucket) == 16 * 7168 * 16384
    assert sum(load > 0 for load in carried) >= 60
    assert max(carried) <= 7168 * 16384 + sum(carried) // 64


def test_rank_group_and_block_partition_helpers_take_both_forms():
    """Parity: ``dist_muon/placement.py:69-161`` of the reference (mesh form) next to this library's integer form."""
    import torch
    import torch.nn as nn

    from flex_shard_b200 import GlobalLayout, set_global_layout
    from flex_shard_b200.dist_muon.placement import (get_dim0_block_partitions, get_mesh_rank_groups,
                                                     get_strided_rank_groups)

    assert get_mesh_rank_groups(8, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert get_strided_rank_groups(8, 4) == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert get_dim0_block_partitions(10, 4) == (3, 3, 2, 2)
    # a pipeline stage's ranks 8..15 as efsdp x ep = 2 x 4: positions in the flat mesh, one group per ep index
    flat, grid = _Mesh(list(range(8, 16))), _Mesh([[8, 9, 10, 11], [12, 13, 14, 15]], ("efsdp", "ep"))
    groups = get_mesh_rank_groups(flat, grid, rank_axis_name="efsdp", partition_axis_name="ep")
    assert groups == ((0, 4), (1, 5), (2, 6), (3, 7))
    swapped = _Mesh([[8, 12], [9, 13], [10, 14], [11, 15]], ("ep", "efsdp"))
    assert get_mesh_rank_groups(flat, swapped, rank_axis_name="efsdp", partition_axis_name="ep") == groups
    with pytest.raises(ValueError, match="same ranks"):
        get_mesh_rank_groups(_Mesh(list(range(8))), grid, rank_axis_name="efsdp", partition_axis_name="ep")

    w1, w2 = nn.Parameter(torch.empty(4, 2, 3)), nn.Parameter(torch.empty(4, 3, 2))
    assert get_dim0_block_partitions([("w1", w1), ("w2", w2)], num_partitions=1, partition_index=0) == ((4, 12),)
    with pytest.raises(ValueError, match="set_global_layout"):
        get_dim0_block_partitions([("w1", w1)], num_partitions=2, partition_index=1)
    for w, shape in ((w1, (2, 3)), (w2, (3, 2))):
        set_global_layout(w, GlobalLayout((8, *shape), ((4, 0, 0),), ((0, 0, 0),), ((4, *shape),)))
    assert get_dim0_block_partitions([("w1", w1), ("w2", w2)], num_partitions=2, partition_index=1) == ((4, 12),) * 2
    with pytest.raises(ValueError, match="set_global_layout"):       # declared for partition 1, asked for partition 0
        get_dim0_block_partitions([("w1", w1)], num_partitions=2, partition_index=0)
    with pytest.raises(ValueError, match="3 dims"):
        get_dim0_block_partitions([("m", nn.Parameter(torch.empty(4, 2)))], num_partitions=1, partition_index=0)
    with pytest.raises(ValueError, match="same, positive number"):
        get_dim0_block_partitions([("w1", w1), ("x", nn.Parameter(torch.empty(3, 2, 2)))], num_partitions=1,
                                  partition_index=0)
