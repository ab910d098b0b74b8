"""``init_from_full``: every rank draws the full tensor (the generator advances as in an unsharded run) and keeps its
own region, for every kind of placement, for tied parameters reached through their second name and for parameters with
a declared outer layout; plus the preconditions of ``relayout_bucket``.  2 gloo ranks.
Parity: the behaviours pinned by the reference's ``tests/test_flex_shard_param_init.py:117-260`` and
``tests/test_relayout_bucket.py:30-80``."""
import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(6, 8)
        self.b = nn.Linear(8, 4, bias=False)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


def _placement(kind):
    from flex_shard_b200.placements import (BlockShard, make_bucketed_block_shard_placement_fn,
                                            make_bucketed_owned_full_param_placement_fn, shard_placement_fn)

    return {"shard": shard_placement_fn(0), "shard1": shard_placement_fn(1),
            "block": lambda named, mesh: {f: BlockShard((1, 1), 0) for f, _ in named},
            "owned": make_bucketed_owned_full_param_placement_fn(),
            "flat": make_bucketed_block_shard_placement_fn()}[kind]


def _init_like_unsharded(rank, world, kind):
    from flex_shard_b200 import BucketSpec, flex_shard, init_from_full

    def fill(mod):
        torch.manual_seed(1234)
        for p in mod.parameters():
            init_from_full(p, lambda t: torch.nn.init.trunc_normal_(t, std=0.02))
        return torch.rand(1).item()            # where the generator stands afterwards

    ref = Net()
    after_ref = fill(ref)
    m = Net()
    pats = ["*"] if kind != "shard1" else ["a.weight", "b.weight"]
    specs = [BucketSpec(pats, placement_fn=_placement(kind))]
    if kind == "shard1":
        specs.append(BucketSpec(["a.bias"]))
    flex_shard(m, specs)
    after = fill(m)
    m.unshard()
    same = all(torch.equal(p.detach(), q.detach()) for p, q in zip(m.parameters(), ref.parameters()))
    m.reshard()
    return {"same": same, "rng": after == after_ref}


@pytest.mark.parametrize("kind", ["shard", "shard1", "block", "owned", "flat"])
def test_sharded_init_equals_the_unsharded_draw(kind):
    for r in run_ranks(_init_like_unsharded, 2, kind):
        assert r["same"] and r["rng"], (kind, r)


def _tied_and_outer(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard, init_from_full
    from flex_shard_b200.placement_contract import GlobalLayout, set_global_layout

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(12, 4)
            self.out = nn.Linear(4, 12, bias=False)
            self.out.weight = self.emb.weight

    out = {}
    t = Tied()
    flex_shard(t, [BucketSpec(["*"])])
    torch.manual_seed(7)
    init_from_full(t.out.weight, lambda x: x.normal_())          # through the later name
    torch.manual_seed(7)
    want = torch.empty(12, 4).normal_()
    t.unshard()
    out["tied"] = bool(torch.equal(t.emb.weight.detach(), want) and t.out.weight is t.emb.weight)
    t.reshard()
    # a parameter that is rows [4r, 4r+4) of an outer (expert-parallel style) sharding of an [8, 3] tensor
    m = nn.Module()
    m.weight = nn.Parameter(torch.zeros(4, 3))
    set_global_layout(m.weight, GlobalLayout((8, 3), ((4 * rank, 0),), ((0, 0),), ((4, 3),)))
    m.forward = lambda x: x
    flex_shard(m, [BucketSpec(["*"])])
    torch.manual_seed(9)
    init_from_full(m.weight, lambda x: x.uniform_())
    torch.manual_seed(9)
    full = torch.empty(8, 3).uniform_()
    mine = full[4 * rank:4 * rank + 4]
    n = 2                                                       # Shard(0) over 2 ranks of the 4 local rows
    out["outer"] = bool(torch.equal(m.weight.detach(), mine[rank * n:(rank + 1) * n]))
    return out


def test_tied_parameter_and_outer_layout_init():
    for r in run_ranks(_tied_and_outer, 2):
        assert r["tied"] and r["outer"], r


def _relayout_rules(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard, relayout_bucket
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn

    torch.manual_seed(0)
    m, other = Net(), Net()
    full = {k: v.clone() for k, v in m.state_dict().items()}
    flex_shard(m, [BucketSpec(["a.*"]), BucketSpec(["b.*"])])
    flex_shard(other, [BucketSpec(["*"])])
    out = {}
    try:
        relayout_bucket(m, other.sharded_bucket_storages[0], make_bucketed_owned_full_param_placement_fn())
        out["foreign"] = ""
    except ValueError as e:
        out["foreign"] = str(e)
    m(torch.randn(2, 6))                                         # the first bucket has been gathered once now
    try:
        relayout_bucket(m, m.sharded_bucket_storages[0], make_bucketed_owned_full_param_placement_fn())
        out["late"] = ""
    except RuntimeError as e:
        out["late"] = str(e)
    fresh = Net()
    fresh.load_state_dict(full)
    flex_shard(fresh, [BucketSpec(["a.*"]), BucketSpec(["b.*"])])
    new = relayout_bucket(fresh, fresh.sharded_bucket_storages[0], make_bucketed_owned_full_param_placement_fn())
    out["replaced"] = fresh.sharded_bucket_storages[0] is new
    fresh.unshard()
    out["bitwise"] = all(torch.equal(p.detach(), full[n]) for n, p in fresh.named_parameters())
    fresh.reshard()
    x = torch.randn(2, 6, generator=torch.Generator().manual_seed(3))
    ref = Net()
    ref.load_state_dict(full)
    out["forward"] = bool(torch.equal(fresh(x), ref(x)))
    return out


def test_relayout_bucket_preconditions_and_result():
    for r in run_ranks(_relayout_rules, 2):
        assert "not one of the module's bucket storages" in r["foreign"], r
        assert "before the bucket's first unshard" in r["late"]
        assert r["replaced"] and r["bitwise"] and r["forward"], r


def _gather_paths(rank, world):
    """``relayout_bucket`` from an uneven Shard(0) layout (byte all-gather path) and from an owner layout (integer-sum
    path): both give back the full tensors bit for bit."""
    from flex_shard_b200 import BucketSpec, flex_shard, relayout_bucket
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn, shard_placement_fn

    class Odd(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Parameter(torch.randn(5, 3))
            self.v = nn.Parameter(torch.randn(7))

        def forward(self, x):
            return x @ self.w.t() + self.v[:5]

    torch.manual_seed(0)
    m = Odd()
    full = {k: v.clone() for k, v in m.state_dict().items()}
    flex_shard(m, [BucketSpec(["*"])])
    st = relayout_bucket(m, m.sharded_bucket_storages[0], make_bucketed_owned_full_param_placement_fn())   # uneven rows
    st = relayout_bucket(m, st, shard_placement_fn(0))                                                     # from owners
    m.unshard()
    ok = all(torch.equal(p.detach(), full[n]) for n, p in m.named_parameters())
    m.reshard()
    return ok


def test_relayout_gathers_bitwise_from_uneven_and_owner_layouts():
    assert all(run_ranks(_gather_paths, 2))
