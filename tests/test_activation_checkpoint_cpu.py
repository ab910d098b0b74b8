"""Activation checkpointing x placements x gradient accumulation on gloo ranks: a checkpointed model
(non-reentrant, reentrant, selective) trains to the same sharded gradients as the un-checkpointed model
under the same placement, and a step that does not accumulate gathers every bucket exactly twice
(forward and backward), wherever the checkpoint boundary sits relative to the bucket's hooks.
Behaviours restated from ``src/flex_shard/tests/test_flex_shard_training.py:2027-2337`` of the reference."""
import pytest
import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from tests.common import run_ranks

DIM = 16


class Inner(nn.Module):
    def __init__(self):
        super().__init__()
        self.up = nn.Linear(DIM, 2 * DIM)
        self.down = nn.Linear(2 * DIM, DIM, bias=False)

    def forward(self, x):
        return x + self.down(torch.relu(self.up(x)))


class Ckpt(nn.Module):
    def __init__(self, mode):
        super().__init__()
        self.inner = Inner()
        self.mode = mode

    def forward(self, x):
        if self.mode == "none":
            return self.inner(x)
        if self.mode == "reentrant":
            return checkpoint(self.inner, x, use_reentrant=True)
        if self.mode == "selective":
            from torch.utils.checkpoint import CheckpointPolicy, create_selective_checkpoint_contexts

            def policy(ctx, op, *a, **k):
                return (CheckpointPolicy.MUST_SAVE if op in (torch.ops.aten.mm.default, torch.ops.aten.addmm.default)
                        else CheckpointPolicy.PREFER_RECOMPUTE)

            return checkpoint(self.inner, x, use_reentrant=False,
                              context_fn=lambda: create_selective_checkpoint_contexts(policy))
        return checkpoint(self.inner, x, use_reentrant=False)


class Net(nn.Module):
    def __init__(self, mode):
        super().__init__()
        self.layers = nn.ModuleList(Ckpt(mode) for _ in range(3))
        self.head = nn.Linear(DIM, 5)

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return self.head(x)


def _placement_fn(kind):
    from flex_shard_b200.placements import (make_block_shard_placement_fn, make_bucketed_block_shard_placement_fn,
                                            make_bucketed_owned_full_param_placement_fn, shard_placement_fn)

    return {"shard": shard_placement_fn(0), "block_shard": make_block_shard_placement_fn(),
            "bucketed_block_shard": make_bucketed_block_shard_placement_fn(),
            "owned": make_bucketed_owned_full_param_placement_fn()}[kind]


def _train(rank, world, kind, mode, hooks_inside, accumulate):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = Net(mode)
    fn = _placement_fn(kind)
    names = [f"layers.{i}.inner" if hooks_inside else f"layers.{i}" for i in range(3)]
    flex_shard(m, [*(BucketSpec([n], placement_fn=fn) for n in names), BucketSpec(["head"], placement_fn=fn)])
    ctx = m._fsb_ctx()
    counts = []
    for step in range(2):
        before = ctx.stats["unshards"]
        micro = 2 if accumulate else 1
        for mb in range(micro):
            if accumulate:
                m.set_requires_gradient_sync(mb == micro - 1)
            x = torch.randn(6, DIM, generator=torch.Generator().manual_seed(100 * step + 10 * mb + rank))
            x.requires_grad_(mode == "reentrant")    # reentrant checkpointing needs an input that requires grad
            m(x).square().mean().backward()
        counts.append(ctx.stats["unshards"] - before)
    grads = {n: p.grad.detach().clone() for n, p in m.named_parameters()}
    return grads, counts, ctx.idle()


def _all_modes(rank, world, kind):
    bad = []
    base = _train(rank, world, kind, "none", False, False)
    base_acc = _train(rank, world, kind, "none", False, True)
    for mode in ("non_reentrant", "reentrant", "selective"):
        for inside in (False, True):
            for acc, ref in ((False, base), (True, base_acc)):
                g, counts, idle = _train(rank, world, kind, mode, inside, acc)
                tag = (kind, mode, "hooks inside" if inside else "hooks outside", "accumulate" if acc else "sync")
                if not idle:
                    bad.append((tag, "runtime not idle after the step"))
                bad += [(tag, n) for n in ref[0] if not torch.equal(g[n], ref[0][n])]
                if not acc and counts[1] != 2 * 4:      # 4 buckets, gathered for forward and for backward
                    bad.append((tag, f"{counts[1]} gathers in a step"))
    return bad


@pytest.mark.parametrize("kind", ["shard", "block_shard", "bucketed_block_shard", "owned"])
def test_checkpointed_model_equals_plain_model(kind):
    for bad in run_ranks(_all_modes, 2, kind, timeout=900):
        assert not bad, bad[:10]
