"""Fp8BucketedBlockShard on 2 gloo ranks: planner goldens, FP8 payload smaller than bf16, gathered
weight bitwise equal to quantise-after-gather, training equal to the unsharded twin."""
import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


def test_partition_and_row_range_goldens():
    from flex_shard_b200.placements import partition_min_max, plan_row_ranges

    assert partition_min_max([4, 4, 4, 4], 2) == [0, 2, 4]
    assert partition_min_max([1, 1, 8], 2) == [0, 2, 3]
    assert partition_min_max([5], 3) == [0, 1, 1, 1]
    # block 4, 2 ranks, w1 16x8 + w2 8x8: rank 0 gets 12 rows of w1, rank 1 the rest
    r = plan_row_ranges([(16, 8), (8, 8)], 2, 4, lambda rows, cols: rows * cols)
    assert r[0] == [(0, 12), (12, 16)] and r[1] == [(0, 0), (0, 8)]
    # 9 x 32 with block 2 on 2 ranks: 4/5 rows (whole blocks, the last one partial)
    r = plan_row_ranges([(9, 32)], 2, 2, lambda rows, cols: rows * cols)
    assert [b - a for a, b in r[0]] in ([4, 5], [6, 3])


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        from flex_shard_b200.quant import FlexShardFloat8BlockwiseLinear

        self.a = FlexShardFloat8BlockwiseLinear(256, 384)
        self.b = FlexShardFloat8BlockwiseLinear(384, 128)

    def forward(self, x):
        return self.b(torch.relu(self.a(x).float()).to(x.dtype))


def _init(m):
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_((0.05 * torch.randn(p.shape, generator=g)).to(p.dtype))


_factory_calls = []


def _consumer_weight(fp8_data, recip_scale, block_size, *, orig_dtype, requires_grad):
    """A ``weight_factory``: the consumer builds its own tensor from the gathered operands (views, not copies)."""
    from flex_shard_b200.quant import BlockwiseFp8Weight

    _factory_calls.append((tuple(fp8_data.shape), tuple(recip_scale.shape), block_size, orig_dtype, requires_grad))
    rows = fp8_data.numel() // fp8_data.shape[-1]
    return BlockwiseFp8Weight(fp8_data.view(rows, fp8_data.shape[-1]), recip_scale, fp8_data.shape, orig_dtype)


def _run(rank, world, steps, factory=False):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import make_fp8_bucketed_block_placement_fn
    from flex_shard_b200.ops.fp8 import quantize_blockwise

    model, twin = Net(), Net()
    _init(model)
    _init(twin)
    fn = make_fp8_bucketed_block_placement_fn(weight_factory=_consumer_weight if factory else None)
    flex_shard(model, [BucketSpec(["*"], placement_fn=fn)])
    st = model.sharded_bucket_storages[0]
    sizes = [sp.numel() * 2 for sp in st.sharded_params]
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    topt = torch.optim.SGD(twin.parameters(), lr=0.05)
    out = {"equal_logits": [], "send_bytes": None}
    for s in range(steps):
        xs = [torch.randn(8, 256, generator=torch.Generator().manual_seed(10 * s + r)).bfloat16() for r in range(world)]
        if out["send_bytes"] is None:
            rt = st.runtime
            out["send_bytes"] = st.placement._payload_layout(st.infos, world)[1]
            model.unshard()
            # gathered payload vs quantise-after-gather of the twin's full weights
            for up, (n, tw) in zip(rt.unsharded_params, twin.named_parameters()):
                q, sc = quantize_blockwise(tw.detach())
                out.setdefault("bitwise", []).append(
                    bool(torch.equal(up.qdata.view(torch.uint8), q.view(torch.uint8)) and torch.equal(up.scale, sc)))
            model.reshard()
        y = model(xs[rank])
        y.float().square().mean().backward()
        opt.step()
        opt.zero_grad()
        ty = [twin(x) for x in xs]
        out["equal_logits"].append(bool(torch.equal(ty[rank], y)))
        sum(t.float().square().mean() for t in ty).div(world).backward()
        topt.step()
        topt.zero_grad()
    out["bf16_bytes"] = sum(p.numel() for p in twin.parameters()) * 2 // world
    out["master_dtype"] = str(st.sharded_params[0].dtype)
    out["factory_calls"] = sorted(set(_factory_calls))
    return out


@pytest.mark.parametrize("factory", [False, True])
def test_fp8_bucket_trains_like_gather_then_quantize(factory):
    """Also with a consumer's ``weight_factory`` (parity: ``custom_placements/fp8_bucketed_block_shard.py:43-65`` of
    the reference): it receives the data in the parameter's shape, one scale per 128x128 block, the block size, the
    compute dtype and whether the parameter trains."""
    res = run_ranks(_run, 2, 3, factory)
    for r in res:
        assert r["factory_calls"] == ([((128, 384), (1, 3), 128, torch.bfloat16, True),
                                       ((384, 256), (3, 2), 128, torch.bfloat16, True)] if factory else [])
        assert all(r["bitwise"]), r
        assert r["equal_logits"][0] is True            # identical weights -> identical logits
        assert r["send_bytes"] < r["bf16_bytes"]       # FP8 + scales is smaller than a bf16 shard
        assert r["master_dtype"] == "torch.bfloat16"
        assert all(r["equal_logits"]), r               # stays bitwise through SGD steps


class ExpertNet(nn.Module):
    """A stacked expert weight [4, 128, 256] next to a plain 2-D weight in the same FP8 bucket."""

    def __init__(self):
        super().__init__()
        from flex_shard_b200.quant import FlexShardFloat8BlockwiseLinear, FlexShardFloat8BlockwiseStackedLinear

        self.inp = FlexShardFloat8BlockwiseLinear(256, 256)
        self.experts = FlexShardFloat8BlockwiseStackedLinear(4, 256, 128)

    def forward(self, x):                       # x [4, T, 256]
        h = self.inp(x.reshape(-1, 256)).view(x.shape)
        return self.experts(h)


def _run_stacked(rank, world, steps):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.ops.fp8 import quantize_blockwise
    from flex_shard_b200.placements import make_fp8_bucketed_block_shard_placement_fn

    model, twin = ExpertNet(), ExpertNet()
    _init(model)
    _init(twin)
    flex_shard(model, [BucketSpec(["*"], placement_fn=make_fp8_bucketed_block_shard_placement_fn())])
    st = model.sharded_bucket_storages[0]
    out = {"ranges": [i.placement.row_ranges for i in st.infos], "bitwise": [], "matrix": [], "equal": []}
    model.unshard()
    for up, (n, tw) in zip(st.runtime.unsharded_params, twin.named_parameters()):
        q, sc = quantize_blockwise(tw.detach().reshape(-1, tw.shape[-1]))
        out["bitwise"].append(bool(torch.equal(up.qdata.view(torch.uint8), q.view(torch.uint8)) and torch.equal(up.scale, sc)))
        if tw.dim() == 3:
            for e in range(tw.shape[0]):       # every matrix equals quantising that matrix alone
                qe, se = quantize_blockwise(tw.detach()[e])
                m = up.matrix(e)
                out["matrix"].append(bool(torch.equal(m.qdata.view(torch.uint8), qe.view(torch.uint8))
                                          and torch.equal(m.scale, se) and tuple(m.shape) == tuple(tw.shape[1:])))
    model.reshard()
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    topt = torch.optim.SGD(twin.parameters(), lr=0.05)
    for s in range(steps):
        xs = [torch.randn(4, 8, 256, generator=torch.Generator().manual_seed(10 * s + r)).bfloat16() for r in range(world)]
        y = model(xs[rank])
        y.float().square().mean().backward()
        opt.step()
        opt.zero_grad()
        ty = [twin(x) for x in xs]
        out["equal"].append(bool(torch.equal(ty[rank], y)))
        sum(t.float().square().mean() for t in ty).div(world).backward()
        topt.step()
        topt.zero_grad()
    return out


def test_stacked_expert_weights_gather_quantised_matrix_by_matrix():
    res = run_ranks(_run_stacked, 2, 3)
    for r in res:
        assert all(r["bitwise"]) and len(r["matrix"]) == 4 and all(r["matrix"]), r
        assert all(r["equal"]), r
    # the stacked weight is handed out in whole matrices (entries of its leading dimension)
    stacked = [rg for rg in res[0]["ranges"] if max(b for _, b in rg) == 4]
    assert stacked and all(0 <= a <= b <= 4 for rg in stacked for a, b in rg)


def test_stacked_weight_whose_matrices_split_a_block_is_refused():
    import pytest
    from flex_shard_b200.placements import make_fp8_bucketed_block_shard_placement_fn
    from tests.common import FakeMesh

    fn = make_fp8_bucketed_block_shard_placement_fn()
    with pytest.raises(ValueError, match="multiple of 128"):
        fn([("w", nn.Parameter(torch.zeros(4, 96, 256)))], FakeMesh(2))
