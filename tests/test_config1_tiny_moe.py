"""Acceptance config 1: tiny MoE transformer on CPU/gloo, world size 2, fp32, Shard(0) buckets one
per layer, AdamW, 10 steps; the mean of the rank losses must match the non-sharded run."""
import torch

from tests.common import run_ranks


def _buckets(model, mesh=None):
    from flex_shard_b200 import BucketSpec

    specs = [BucketSpec(["tok_embeddings"], mesh=mesh)]
    for i in range(len(model.layers)):
        specs.append(BucketSpec([f"layers.{i}.*"], mesh=mesh))
    specs.append(BucketSpec(["norm", "output"], mesh=mesh, reshard_after_forward=False))
    return specs


def _data(step, rank, B=4, S=128, V=1024):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return torch.randint(0, V, (B, S), generator=g)


def _sharded(rank, world, steps):
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.models.tiny_moe import TinyMoEConfig, TinyMoETransformer, next_token_loss

    torch.manual_seed(0)
    model = TinyMoETransformer(TinyMoEConfig())
    model.init_weights(0)
    flex_shard(model, _buckets(model))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    losses = []
    for step in range(steps):
        tok = _data(step, rank)
        loss = next_token_loss(model(tok), tok)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()))
    ctx = model._fsb_ctx()
    return {"losses": losses, "stats": dict(ctx.stats), "idle": ctx.idle()}


def _reference(steps, world):
    from flex_shard_b200.models.tiny_moe import TinyMoEConfig, TinyMoETransformer, next_token_loss

    torch.manual_seed(0)
    model = TinyMoETransformer(TinyMoEConfig())
    model.init_weights(0)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    losses = []
    for step in range(steps):
        tot = 0.0
        for r in range(world):
            tok = _data(step, r)
            loss = next_token_loss(model(tok), tok) / world
            loss.backward()
            tot += float(loss.detach())
        opt.step()
        opt.zero_grad()
        losses.append(tot)
    return losses


def test_tiny_moe_gloo_ws2_matches_unsharded():
    steps, world = 10, 2
    res = run_ranks(_sharded, world, steps)
    ref = _reference(steps, world)
    mean = [sum(r["losses"][i] for r in res) / world for i in range(steps)]
    for a, b in zip(mean, ref):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (mean, ref)
    for r in res:
        assert r["idle"]
        # 6 buckets, gathered for forward and again for backward except the resident last one
        assert r["stats"]["reduces"] == 6 * steps
