"""The recipe form of ``materialize_dist_muon_buckets`` on real meshes: 4 gloo ranks as a flat mesh and as an
``efsdp x ep = 2 x 2`` grid.  Owned matrices, per-head blocks and ``Shard(0)`` vectors share a mixed bucket on the flat
mesh; each expert-parallel partition's experts sit in a flat block bucket on the two ranks that share the partition.
Gradients (summed, as the recipe asks) equal the hand-reduced gradients of an unsharded replica."""
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self, ep_index):
        super().__init__()
        self.w = nn.Linear(8, 8, bias=False)
        self.heads = nn.Linear(8, 8, bias=False)            # 4 heads of 2 rows
        self.norm = nn.LayerNorm(8)
        g = torch.Generator().manual_seed(100 + ep_index)   # every partition holds its own two experts
        self.experts = nn.Parameter(0.1 * torch.randn(2, 8, 8, generator=g))

    def forward(self, x):
        h = self.norm(self.heads(torch.relu(self.w(x))))
        return h + sum(h @ self.experts[e] for e in range(2))


def _work(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    from flex_shard_b200 import GlobalLayout, flex_shard, set_global_layout
    from flex_shard_b200.dist_muon import (BlockShardPlan, PackedParameterPlan, ParameterBucketPlan,
                                           build_local_dist_muon, materialize_dist_muon_buckets)
    from flex_shard_b200.placements import BucketedBlockShard

    flat = init_device_mesh("cpu", (4,))
    grid = init_device_mesh("cpu", (2, 2), mesh_dim_names=("efsdp", "ep"))
    ep = grid.get_local_rank("ep")
    torch.manual_seed(0)
    model, ref = Net(ep), Net(ep)
    ref.load_state_dict(model.state_dict())
    set_global_layout(model.experts, GlobalLayout((4, 8, 8), ((2 * ep, 0, 0),), ((0, 0, 0),), ((2, 8, 8),)))
    named = dict(model.named_parameters())
    plan = ParameterBucketPlan(
        mixed_fqns=("w.weight", "heads.weight", "norm.weight", "norm.bias"),
        owned_parameters=(("w.weight", named["w.weight"]),),
        packed_parameters=(PackedParameterPlan("heads.weight", named["heads.weight"], BlockShardPlan(4)),),
        partitioned_parameters=(("experts", named["experts"]),), partition_group_name_prefix="experts#")
    specs = materialize_dist_muon_buckets(
        bucket_plans=(plan,), assignment_name_by_fqn={"w.weight": "w", "heads.weight": "heads"},
        assignment_mesh=flat, partition_mesh=grid, partition_rank_axis_name="efsdp", partition_axis_name="ep")
    flex_shard(model, specs)
    mixed, experts = model.sharded_bucket_storages
    out = {"meshes": (mixed.comm.world_size, experts.comm.world_size),
           "expert_placement": isinstance(experts.placement, BucketedBlockShard),
           "expert_ranks": sorted(dist.get_process_group_ranks(experts.comm.group))}
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(rank))
    model(x).square().mean().backward()
    ref(x).square().mean().backward()
    for n, p in ref.named_parameters():
        dist.all_reduce(p.grad, group=grid.get_group("efsdp") if n == "experts" else None)
    from flex_shard_b200.checkpoint import get_flex_shard_global_layouts

    err = 0.0
    for n, lay in get_flex_shard_global_layouts(model).items():
        mine, want = dict(model.named_parameters())[n].grad, dict(ref.named_parameters())[n].grad
        if n == "experts":      # the layout is in the coordinates of all 4 experts: this partition's start at 2 * ep
            want = torch.cat([torch.zeros_like(want)] * ep + [want] + [torch.zeros_like(want)] * (1 - ep))
        for goff, loff, size in zip(lay.global_offsets, lay.local_offsets, lay.local_sizes):
            a, b = mine, want
            for d, (g0, l0, sz) in enumerate(zip(goff, loff, size)):
                a, b = a.narrow(d, l0, sz), b.narrow(d, g0, sz)
            if a.numel():
                err = max(err, float((a - b).abs().max()))
    out["grad_err"] = err
    # every matrix sits whole where it is stored: the Muon step needs no collective
    opt = build_local_dist_muon(model, lr=0.02)
    opt.step()
    out["collectives"] = opt.collectives_issued
    return out


def test_recipe_buckets_on_a_flat_mesh_and_an_expert_grid():
    for r, out in enumerate(run_ranks(_work, 4)):
        assert out["meshes"] == (4, 2) and out["expert_placement"]
        assert out["expert_ranks"] == ([0, 2] if r % 2 == 0 else [1, 3])
        assert out["grad_err"] < 1e-5, out
        assert out["collectives"] == 0
