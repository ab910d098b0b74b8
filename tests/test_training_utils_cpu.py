"""Training-loop helpers: the warm-up / plateau / decay schedule, the sharded gradient-norm clip against
``torch.nn.utils.clip_grad_norm_`` on the unsharded twin (2 gloo ranks), the JSON step metrics.
Parity: the helpers of the reference's example (``examples/deepseek_v3/train.py:230-291``)."""
import io
import json

import torch
import torch.nn as nn

from tests.common import run_ranks


def test_lr_schedule_warms_up_holds_and_decays():
    from flex_shard_b200.utils.training import lr_lambda

    f = lambda s: lr_lambda(s, warmup_steps=3, total_steps=20, decay_ratio=0.25, min_lr_factor=0.1)
    assert [round(f(s), 4) for s in range(3)] == [0.25, 0.5, 0.75]          # linear warm-up, never zero
    assert all(f(s) == 1.0 for s in range(3, 15))                           # plateau
    tail = [f(s) for s in range(15, 20)]
    assert all(a > b for a, b in zip(tail, tail[1:])) and abs(tail[-1] - 0.1) < 1e-9   # linear decay to the floor
    assert lr_lambda(0, 0, 10) == 1.0 and lr_lambda(9, 0, 10) == 1.0        # no warm-up, no decay


def _clip(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn
    from flex_shard_b200.utils.training import clip_grad_norm_

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    ref = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    ref.load_state_dict(m.state_dict())
    # two kinds of placement, so that the local shards differ in shape and ownership
    flex_shard(m, [BucketSpec(["0.*"]), BucketSpec(["2.*"], placement_fn=make_bucketed_owned_full_param_placement_fn())])
    xs = [torch.randn(4, 8, generator=torch.Generator().manual_seed(r)) * 10 for r in range(world)]
    m(xs[rank]).square().mean().backward()
    sum(ref(x).square().mean() for x in xs).div(world).backward()
    want = torch.nn.utils.clip_grad_norm_(ref.parameters(), max_norm=0.5)
    got = clip_grad_norm_(m, max_norm=0.5)
    opt, ropt = torch.optim.SGD(m.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    opt.step()
    ropt.step()
    m.unshard()
    err = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(m.parameters(), ref.parameters()))
    m.reshard()
    small = clip_grad_norm_(m, max_norm=1e9)                                 # far above the norm: nothing is scaled
    return {"norm": float(got), "want": float(want), "err": err, "after": float(small)}


def test_sharded_grad_norm_clip_matches_the_unsharded_clip():
    res = run_ranks(_clip, 2)
    for r in res:
        assert abs(r["norm"] - r["want"]) < 1e-4 * r["want"] and r["want"] > 0.5, r
        assert r["err"] < 1e-6, r
        assert abs(r["after"] - 0.5) < 1e-3                                   # the clipped gradients have the target norm
    assert res[0]["norm"] == res[1]["norm"]                                   # every rank sees the same global norm


def test_json_metrics_write_one_line_per_step_on_rank_zero():
    from flex_shard_b200.utils.training import JsonMetrics

    buf = io.StringIO()
    m = JsonMetrics(stream=buf, rank=0)
    m.start_step()
    rec = m.end_step(7, tokens=1000, loss=torch.tensor(2.5), lr=3e-4)
    line = json.loads(buf.getvalue().strip())
    assert line == rec and line["step"] == 7 and line["loss"] == 2.5 and line["lr"] == 3e-4
    assert line["ms"] >= 0 and line["tokens_per_s_per_gpu"] > 0
    quiet = io.StringIO()
    other = JsonMetrics(stream=quiet, rank=1)
    other.start_step()
    other.end_step(0, tokens=10)
    assert quiet.getvalue() == ""                                             # only rank 0 prints
