"""Mxfp8BucketedBlockShard on 2 gloo ranks: payload smaller than bf16, gathered weight bitwise equal
to quantise-after-gather, training equal to the unsharded twin; the MXFP8 linear against a
high-precision reference; the weight wrapper's invariants."""
import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        from flex_shard_b200.quant import FlexShardMxfp8BlockwiseLinear

        self.a = FlexShardMxfp8BlockwiseLinear(256, 384)
        self.b = FlexShardMxfp8BlockwiseLinear(384, 128)

    def forward(self, x):
        return self.b(torch.relu(self.a(x).float()).to(x.dtype))


def _init(m):
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_((0.05 * torch.randn(p.shape, generator=g)).to(p.dtype))


_factory_calls = []


def _consumer_weight(fp8_data, fwd_scale, dgrad_scale, *, orig_dtype, requires_grad):
    """A ``weight_factory``: the consumer's own tensor from the gathered data and the two blocked scale tensors."""
    from flex_shard_b200.quant import BlockwiseMxfp8Weight

    _factory_calls.append((tuple(fp8_data.shape), fwd_scale.dtype, dgrad_scale.dtype, orig_dtype, requires_grad))
    rows = fp8_data.numel() // fp8_data.shape[-1]
    return BlockwiseMxfp8Weight(fp8_data.view(rows, fp8_data.shape[-1]), fwd_scale, fp8_data.shape, orig_dtype,
                                dgrad_scale=dgrad_scale)


def _run(rank, world, steps, factory=False):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.ops.mxfp8 import mx_expand_scales, mx_quantize_weight
    from flex_shard_b200.placements import make_mxfp8_bucketed_block_placement_fn

    model, twin = Net(), Net()
    _init(model)
    _init(twin)
    fn = make_mxfp8_bucketed_block_placement_fn(weight_factory=_consumer_weight if factory else None)
    flex_shard(model, [BucketSpec(["*"], placement_fn=fn)])
    st = model.sharded_bucket_storages[0]
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    topt = torch.optim.SGD(twin.parameters(), lr=0.05)
    out = {"equal_logits": [], "send_bytes": None, "ranges": [i.placement.row_ranges for i in st.infos]}
    for s in range(steps):
        xs = [torch.randn(8, 256, generator=torch.Generator().manual_seed(10 * s + r)).bfloat16() for r in range(world)]
        if out["send_bytes"] is None:
            rt = st.runtime
            out["send_bytes"] = st.placement._payload_layout(st.infos, world)[1]
            model.unshard()
            for up, (n, tw) in zip(rt.unsharded_params, twin.named_parameters()):
                q, e = mx_quantize_weight(tw.detach())
                rows, cols = tw.shape
                out.setdefault("bitwise", []).append(bool(
                    torch.equal(up.qdata.view(torch.uint8), q.view(torch.uint8))
                    and torch.equal(up.fwd_scale, mx_expand_scales(e, rows, cols, False))
                    and torch.equal(up.dgrad_scale, mx_expand_scales(e, rows, cols, True))))
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
    out["factory_calls"] = len(_factory_calls)
    return out


@pytest.mark.parametrize("factory", [False, True])
def test_mxfp8_bucket_trains_like_gather_then_quantize(factory):
    """Also with a consumer's ``weight_factory`` (parity: ``custom_placements/mxfp8_bucketed_block_shard.py:68-90``
    of the reference)."""
    res = run_ranks(_run, 2, 3, factory)
    for r in res:
        assert (r["factory_calls"] > 0) == factory
        assert all(r["bitwise"]), r
        assert all(r["equal_logits"]), r
        assert r["send_bytes"] < r["bf16_bytes"]
        assert r["master_dtype"] == "torch.bfloat16"
        for ranges in r["ranges"]:           # whole 128-row units per rank
            assert all(a % 128 == 0 for a, _ in ranges)


def test_mxfp8_linear_tracks_a_high_precision_linear_and_emits_wgrad_in_grad_dtype():
    from flex_shard_b200.quant import FlexShardMxfp8BlockwiseLinear, convert_to_flex_shard_mxfp8_blockwise_linear

    torch.manual_seed(0)
    lin = nn.Linear(256, 128, bias=False).to(torch.bfloat16)
    seq = convert_to_flex_shard_mxfp8_blockwise_linear(nn.Sequential(lin))
    mx = seq[0]
    assert isinstance(mx, FlexShardMxfp8BlockwiseLinear) and mx.weight is lin.weight
    mx.weight.grad_dtype = torch.float32
    x = torch.randn(48, 256).bfloat16().requires_grad_()
    y = mx(x)
    y.float().square().mean().backward()
    ref_w = lin.weight.detach().float().requires_grad_()
    xr = x.detach().float().requires_grad_()
    yr = xr @ ref_w.t()
    yr.square().mean().backward()
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y, yr) < 0.06 and rel(x.grad, xr.grad) < 0.08
    assert mx.weight.grad.dtype == torch.float32 and rel(mx.weight.grad, ref_w.grad) < 0.08


def test_mxfp8_weight_wrapper_keeps_all_three_tensors_through_detach():
    from flex_shard_b200.ops.mxfp8 import mx_quantize_weight
    from flex_shard_b200.quant import BlockwiseMxfp8Weight, blockwise_mxfp8_dequant_weight

    w = torch.randn(160, 96).bfloat16()
    q, e = mx_quantize_weight(w)
    mw = BlockwiseMxfp8Weight.from_tile_exponents(q, e, w.shape)
    d = mw.detach()
    assert type(d) is BlockwiseMxfp8Weight and d.dgrad_scale is mw.dgrad_scale and d.fwd_scale is mw.fwd_scale
    assert mw.fwd_scale.numel() == 256 * 4 and mw.dgrad_scale.numel() == 128 * 8   # blocked: rows to 128, groups to 4
    deq = mw.dequantize()
    assert deq.shape == w.shape and ((deq - w.float()).norm() / w.float().norm()).item() < 0.04
    assert torch.equal(deq, blockwise_mxfp8_dequant_weight(mw.fp8_data, mw.fwd_scale))
    names, meta = mw.__tensor_flatten__()
    assert names == ["qdata", "scale", "dgrad_scale"]
