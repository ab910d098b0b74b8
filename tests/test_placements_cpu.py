"""Sliced placements (BlockShard, BucketedOwned, mixed buckets) on 2 gloo ranks: training parity
with an unsharded model, storage goldens, relayout and checkpoint resharding."""
import os
import tempfile

import pytest
import torch
import torch.nn as nn

from tests.common import FakeMesh, run_ranks


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(16, 16)
        self.b = nn.Linear(16, 8)
        self.norm = nn.LayerNorm(8)

    def forward(self, x):
        return self.norm(self.b(torch.relu(self.a(x))))


def _placement_fn(kind):
    from flex_shard_b200.placements import (BlockShard, BucketedOwned, MixedBucketPlacement, Shard,
                                            make_bucketed_owned_full_param_placement_fn)

    if kind == "block":
        return lambda named, mesh: {f: BlockShard((1, 1) if p.shape[0] % 2 == 0 else (1, 0), 0) for f, p in named}
    if kind == "owned":
        return make_bucketed_owned_full_param_placement_fn()
    if kind == "flat":
        from flex_shard_b200.placements import make_bucketed_block_shard_placement_fn

        return make_bucketed_block_shard_placement_fn()
    if kind == "flat_uneven":
        from flex_shard_b200.placements import make_bucketed_block_shard_placement_fn

        return make_bucketed_block_shard_placement_fn((1, 3))
    if kind == "owned_segments":    # the bucket-level form: one BucketedOwned built from {fqn: segment specs}
        from flex_shard_b200.placements import make_bucketed_owned_full_param_segments

        def fn(named, mesh):
            whole = BucketedOwned(make_bucketed_owned_full_param_segments(named, 2))
            return {f: (whole,) for f, _ in named}
        return fn
    if kind == "mixed_factory":     # the reference's way: one MixedBucketPlacement per bucket hands out the members
        from flex_shard_b200.placements import make_bucketed_owned_full_param_segments

        def fn(named, mesh):
            owned = [(f, p) for f, p in named if f == "a.weight"]
            mixed = MixedBucketPlacement(make_bucketed_owned_full_param_segments(owned, 2))
            out = {}
            for f, p in named:
                if f == "a.weight":
                    out[f] = (mixed.bucketed_owned,)
                elif p.dim() == 2:
                    out[f] = (mixed.block_shard(blocks_per_rank=(1, 1), dim=0),)
                else:
                    out[f] = (mixed.shard0,)
            return out
        return fn
    if kind == "mixed_owned":      # every member whole on one owner: gradients accumulate in one mirror buffer
        return lambda named, mesh: {f: MixedBucketPlacement(BucketedOwned(((i % 2, 0, p.shape[0]),)))
                                    for i, (f, p) in enumerate(named)}
    if kind == "mixed":
        def fn(named, mesh):
            out = {}
            for i, (f, p) in enumerate(named):
                if p.dim() == 2 and i % 2 == 0:
                    out[f] = MixedBucketPlacement(BucketedOwned(((i % 2, 0, p.shape[0]),)))
                elif p.dim() == 2:
                    out[f] = MixedBucketPlacement(BlockShard((1, 1), 1))
                else:
                    out[f] = MixedBucketPlacement(Shard(0))
            return out
        return fn
    raise ValueError(kind)


def _train(rank, world, kind, steps):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    model = MLP()
    ref = MLP()
    ref.load_state_dict(model.state_dict())
    flex_shard(model, [BucketSpec(["*"], placement_fn=_placement_fn(kind))])
    st = model.sharded_bucket_storages[0]
    assert st.placement.reduces_grads_in_param_layout(st.infos) == (
        kind in ("owned", "owned_segments", "mixed_owned", "flat", "flat_uneven"))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for s in range(steps):
        xs = [torch.randn(4, 16, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)]
        model(xs[rank]).square().mean().backward()
        opt.step()
        opt.zero_grad()
        sum(ref(x).square().mean() for x in xs).div(world).backward()
        ropt.step()
        ropt.zero_grad()
    # compare full parameters
    model.unshard()
    err = 0.0
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        err = max(err, float((p.detach() - q.detach()).abs().max()))
    model.reshard()
    sizes = [sp.numel() for sp in model.sharded_bucket_storages[0].sharded_params]
    return err, sizes, model.sharded_bucket_storages[0].total_bytes


@pytest.mark.parametrize("kind", ["block", "owned", "owned_segments", "mixed", "mixed_factory", "mixed_owned", "flat",
                                  "flat_uneven"])
def test_sliced_placements_train_like_unsharded(kind):
    res = run_ranks(_train, 2, kind, 3)
    for err, sizes, nbytes in res:
        assert err < 1e-5, (kind, err)
    if kind == "owned":
        # owners hold whole parameters and no padding; the other rank holds nothing of them
        total = sum(p.numel() for p in MLP().parameters())
        assert sum(res[0][1]) + sum(res[1][1]) == total
        assert all(a == 0 or b == 0 for a, b in zip(res[0][1], res[1][1]))


def test_owner_segment_specs():
    """The bucket-level description of ownership: whole parameters by element count (hosts first, carried loads),
    experts of stacked weights in contiguous runs, and the narrowing to one parameter's dim-0 rows.
    Parity: ``custom_placements/owned.py:39-48, 425-583`` of the reference."""
    from flex_shard_b200.placements import (BucketedOwned, BucketedOwnedSegmentSpec,
                                            make_bucketed_owned_expert_block_segments,
                                            make_bucketed_owned_full_param_segments)

    named = [("big", torch.zeros(8, 8)), ("mid", torch.zeros(4, 8)), ("small", torch.zeros(8))]
    segs = make_bucketed_owned_full_param_segments(named, 2)
    assert {f: (s[0].owner_rank, s[0].param_offset, s[0].numel, s[0].storage_order) for f, s in segs.items()} == {
        "big": (0, 0, 64, 0), "mid": (1, 0, 32, 1), "small": (1, 0, 8, 2)}
    loads = [100.0, 0.0]
    carried = make_bucketed_owned_full_param_segments(named[:1], 2, carried_loads=loads)
    assert carried["big"][0].owner_rank == 1 and loads == [100.0, 0.0]       # the caller adds what was placed
    for kwargs in (dict(hosts=(0,)), dict(carried_loads=(0, 0, 0))):
        with pytest.raises(ValueError):
            make_bucketed_owned_full_param_segments(named, 2, **kwargs)
    whole = BucketedOwned(segs)
    assert whole.for_param("mid", (4, 8)).segments == ((1, 0, 4),)
    with pytest.raises(ValueError, match="no segments"):
        whole.for_param("other", (4, 8))
    with pytest.raises(ValueError, match="for_param"):
        whole.pieces((4, 8), 0, 2)
    ragged = BucketedOwned({"w": [BucketedOwnedSegmentSpec("w#0", "w", 0, 12, 0)]})
    with pytest.raises(ValueError, match="whole dim-0 rows"):
        ragged.for_param("w", (4, 8))

    experts = [("moe.w1", torch.zeros(5, 4, 2)), ("moe.w2", torch.zeros(5, 2, 4))]
    es = make_bucketed_owned_expert_block_segments(experts, 2)
    assert [s.owner_rank for s in es["moe.w1"]] == [0, 0, 0, 1, 1] == [s.owner_rank for s in es["moe.w2"]]
    assert [(s.param_offset, s.numel) for s in es["moe.w1"]][:2] == [(0, 8), (8, 8)]
    # one expert's weights sit together in the owner's storage, in suffix order (.w1, .w3, .w2)
    assert es["moe.w1"][1].storage_order < es["moe.w2"][1].storage_order < es["moe.w1"][2].storage_order
    per_param = BucketedOwned(es, view_kind="expert_block").for_param("moe.w2", (5, 2, 4))
    assert per_param.view_kind == "expert_block" and per_param.pieces((5, 2, 4), 1, 2)[0].start == 3
    with pytest.raises(ValueError, match="at least 3 dims"):
        make_bucketed_owned_expert_block_segments([("moe.w1", torch.zeros(4, 2))], 2)
    with pytest.raises(ValueError, match="suffix"):
        make_bucketed_owned_expert_block_segments(experts, 2, suffix_order=())


def test_owner_rows_hold_no_padding_golden():
    """Linear(16,16)+Linear(16,8) on 2 ranks: weights and biases are whole on their owners."""
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn
    from flex_shard_b200.placements.sliced import plan_rows
    from flex_shard_b200.bucket_storage import BucketSpec, create_param_infos

    m = nn.Sequential(nn.Linear(16, 16), nn.Linear(16, 8))
    named = list(m.named_parameters())
    fn = make_bucketed_owned_full_param_placement_fn()
    pls = fn(named, FakeMesh(2))
    infos, total0 = create_param_infos(BucketSpec(["*"]), named, pls, 0, 2, {})
    _, total1 = create_param_infos(BucketSpec(["*"]), named, pls, 1, 2, {})
    assert total0 // 4 + total1 // 4 >= 408  # 256 + 16 + 128 + 8 elements in all
    plan = plan_rows(infos, 2, lambda i: 1)
    assert plan.owner_only and sum(plan.row_by_rank) >= 408


def _relayout_and_checkpoint(rank, world, tmp):
    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard, relayout_bucket, set_state_dict_global_layouts
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn

    torch.manual_seed(0)
    model = MLP()
    full = {k: v.clone() for k, v in model.state_dict().items()}
    flex_shard(model, [BucketSpec(["a", "b"]), BucketSpec(["norm"])])
    st = model.sharded_bucket_storages[0]
    relayout_bucket(model, st, make_bucketed_owned_full_param_placement_fn())
    sd = model.state_dict()
    set_state_dict_global_layouts(model, sd)
    checkpoint.save({"model": sd}, tmp)
    # reload into a Shard(0) model and compare against the original full tensors
    other = MLP()
    for p in other.parameters():
        p.data.zero_()
    flex_shard(other, [BucketSpec(["*"])])
    sd2 = other.state_dict()
    set_state_dict_global_layouts(other, sd2)
    checkpoint.load({"model": sd2}, tmp)
    other.load_state_dict(sd2)
    other.unshard()
    err = max(float((p.detach() - full[n]).abs().max()) for n, p in other.named_parameters())
    other.reshard()
    x = torch.randn(3, 16, generator=torch.Generator().manual_seed(5))
    ref = MLP()
    ref.load_state_dict(full)
    out_err = float((model(x) - ref(x)).abs().max())
    return err, out_err


def test_relayout_then_checkpoint_reshards_bitwise():
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks(_relayout_and_checkpoint, 2, os.path.join(d, "ckpt"))
    for err, out_err in res:
        assert err == 0.0
        assert out_err < 1e-6


def test_flat_bucket_plan_formulas():
    """align = lcm(row sizes); offsets aligned; padded_total multiple of align * sum(blocks)."""
    from flex_shard_b200.placements import FlatBucketPlan

    plan = FlatBucketPlan([(16, 8), (8, 12), (5,)], (1, 1))
    assert plan.align == 24
    assert plan.param_off == [0, 144, 240]
    assert plan.padded_total % (24 * 2) == 0 and plan.padded_total >= 245
    lo, hi = plan.rank_range(1)
    assert hi - lo == plan.padded_total // 2
    # every rank holds whole rows of every parameter
    for i in range(3):
        rows = sum(plan.local_rows(i, r)[1] - plan.local_rows(i, r)[0] for r in range(2))
        assert rows == plan.shapes[i][0]


class _TwoDtypes(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(8, 6)
        self.b = nn.Linear(6, 4).to(torch.bfloat16)

    def forward(self, x):
        return self.b(self.a(x).to(torch.bfloat16))


def _mixed_dtype_bucket(rank, world):
    import torch.distributed as dist

    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import BlockShard, BucketedOwned, MixedBucketPlacement, Shard

    torch.manual_seed(0)
    model, ref = _TwoDtypes(), _TwoDtypes()
    ref.load_state_dict(model.state_dict())

    def fn(named, mesh):
        out = {}
        for f, p in named:
            if f == "a.weight":
                out[f] = MixedBucketPlacement(BucketedOwned(((1, 0, p.shape[0]),)))
            elif f == "b.weight":
                out[f] = MixedBucketPlacement(BlockShard((1, 1), 1))
            else:
                out[f] = MixedBucketPlacement(Shard(0))
        return out

    flex_shard(model, [BucketSpec(["*"], placement_fn=fn)])
    (st,) = model.sharded_bucket_storages
    local_dtypes = sorted({str(sp.dtype) for sp in st.sharded_params})
    gathered = []
    plain = dist.all_gather_into_tensor

    def spy(out, inp, *a, **k):
        gathered.append((out.dtype, out.numel()))
        return plain(out, inp, *a, **k)

    dist.all_gather_into_tensor = spy
    try:
        model.unshard()
    finally:
        dist.all_gather_into_tensor = plain
    same = all(p.dtype == q.dtype and torch.equal(p.detach(), q.detach())
               for (_, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()))
    model.reshard()
    xs = [torch.randn(4, 8, generator=torch.Generator().manual_seed(3 + r)) for r in range(world)]
    model(xs[rank]).float().sum().backward()
    sum(ref(x).float().sum() for x in xs).div(world).backward()
    grad_dtypes = {n: p.grad.dtype for n, p in model.named_parameters()}
    from flex_shard_b200.checkpoint import get_flex_shard_global_layouts

    layouts = get_flex_shard_global_layouts(model)
    err = 0.0
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        lay = layouts[n]
        for goff, loff, size in zip(lay.global_offsets, lay.local_offsets, lay.local_sizes):
            mine, want = p.grad, q.grad
            for d, (g0, l0, sz) in enumerate(zip(goff, loff, size)):
                mine, want = mine.narrow(d, l0, sz), want.narrow(d, g0, sz)
            if mine.numel():
                err = max(err, float((mine.float() - want.float()).abs().max()))
    return local_dtypes, gathered, st.total_bytes, same, grad_dtypes, err


def test_mixed_bucket_holds_two_dtypes_and_gathers_bytes_once():
    """fp32 and bf16 members of one mixed bucket travel as one byte all-gather and come back in their own
    dtypes with every rank's values (parity: ``flex_shard/tests/test_flex_shard_buckets.py``
    ``test_mixed_payload_dtypes_use_one_byte_all_gather`` and ``..._reconstruct_rank_distinct_values``)."""
    res = run_ranks(_mixed_dtype_bucket, 2)
    for local_dtypes, gathered, nbytes, same, grad_dtypes, err in res:
        assert local_dtypes == ["torch.bfloat16", "torch.float32"]
        assert len(gathered) == 1 and gathered[0][0] == torch.uint8
        assert same
        assert grad_dtypes["a.weight"] == torch.float32 and grad_dtypes["b.weight"] == torch.bfloat16
        assert err < 2e-2, err
