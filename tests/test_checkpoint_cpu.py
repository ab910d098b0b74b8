"""Checkpoints across world sizes: model + AdamW state saved from 2 gloo ranks (Shard(0) with uneven
rows) reload bitwise into a single unsharded-size process; optimizer-hook error cases."""
import os
import tempfile

import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(6, 7)        # 7 rows over 2 ranks: uneven
        self.b = nn.Linear(7, 3)

    def forward(self, x):
        return self.b(torch.tanh(self.a(x)))


def _train_and_save(rank, world, path):
    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard, set_state_dict_global_layouts
    from flex_shard_b200.checkpoint import register_optimizer_checkpoint_hook

    torch.manual_seed(0)
    m = Net()
    flex_shard(m, [BucketSpec(["*"])])
    opt = torch.optim.AdamW(m.parameters(), lr=0.05)
    register_optimizer_checkpoint_hook(opt, m)
    register_optimizer_checkpoint_hook(opt, m)          # registering again replaces the earlier hook
    second = str(len(opt._optimizer_state_dict_post_hooks))
    for s in range(3):
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(100 + s))   # same data on both ranks
        m(x).square().mean().backward()
        opt.step()
        opt.zero_grad()
    sd = m.state_dict()
    set_state_dict_global_layouts(m, sd)
    checkpoint.save({"model": sd, "optim": opt.state_dict()}, path)
    return second


def test_save_on_two_ranks_load_on_one():
    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard, set_state_dict_global_layouts
    from flex_shard_b200.checkpoint import register_optimizer_checkpoint_hook

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ckpt")
        res = run_ranks(_train_and_save, 2, path)
        assert all(r == "1" for r in res)      # registered twice, one hook
        # the same three steps without sharding
        torch.manual_seed(0)
        ref = Net()
        ropt = torch.optim.AdamW(ref.parameters(), lr=0.05)
        for s in range(3):
            x = torch.randn(4, 6, generator=torch.Generator().manual_seed(100 + s))
            ref(x).square().mean().backward()
            ropt.step()
            ropt.zero_grad()
        # reload into a 1-rank flex_shard model (no process group at all)
        torch.manual_seed(1)
        m = Net()
        flex_shard(m, [BucketSpec(["*"])])
        opt = torch.optim.AdamW(m.parameters(), lr=0.05)
        register_optimizer_checkpoint_hook(opt, m)
        x = torch.randn(4, 6)
        m(x).square().mean().backward()   # materialise the optimizer state so there is something to load into
        opt.step()
        opt.zero_grad()
        sd = m.state_dict()
        set_state_dict_global_layouts(m, sd)
        osd = opt.state_dict()
        checkpoint.load({"model": sd, "optim": osd}, path)
        m.load_state_dict(sd)
        opt.load_state_dict(osd)
        m.unshard()
        for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
            torch.testing.assert_close(p.detach(), q.detach(), rtol=0, atol=1e-6), n
        m.reshard()
        for p, q in zip(m.parameters(), ref.parameters()):
            for key in ("exp_avg", "exp_avg_sq"):
                torch.testing.assert_close(opt.state[p][key].reshape(-1), ropt.state[q][key].reshape(-1)[: opt.state[p][key].numel()],
                                           rtol=0, atol=1e-6)
        # and the next step agrees
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(7))
        m(x).square().mean().backward()
        opt.step()
        ref(x).square().mean().backward()
        ropt.step()
        m.unshard()
        for p, q in zip(m.parameters(), ref.parameters()):
            torch.testing.assert_close(p.detach(), q.detach(), rtol=0, atol=1e-5)
        m.reshard()


def test_optimizer_hook_rejects_foreign_optimizers():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.checkpoint import register_optimizer_checkpoint_hook

    m = Net()
    flex_shard(m, [BucketSpec(["*"])])
    with pytest.raises(NotImplementedError, match="supports Adam and AdamW, got SGD"):
        register_optimizer_checkpoint_hook(torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9), m)
    other = Net()
    with pytest.raises(ValueError, match="not a sharded parameter of the module"):
        register_optimizer_checkpoint_hook(torch.optim.AdamW(other.parameters(), lr=0.1), m)
    # one foreign parameter among the module's own is refused too
    with pytest.raises(ValueError, match="not a sharded parameter of the module"):
        register_optimizer_checkpoint_hook(torch.optim.AdamW([*m.parameters(), *other.parameters()], lr=0.1), m)


def test_optimizer_state_of_another_shape_cannot_take_the_layout():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.checkpoint import register_optimizer_checkpoint_hook
    from flex_shard_b200.placement_contract import get_global_layout

    m = Net()
    flex_shard(m, [BucketSpec(["*"])])
    opt = torch.optim.Adam(m.parameters(), amsgrad=True)
    register_optimizer_checkpoint_hook(opt, m)
    for p in m.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    state = opt.state_dict()["state"]
    for pid in state:
        for key in ("exp_avg", "exp_avg_sq", "max_exp_avg_sq"):
            assert get_global_layout(state[pid][key]) is not None
        assert get_global_layout(state[pid]["step"]) is None
    first = next(iter(m.parameters()))
    opt.state[first]["exp_avg"] = torch.zeros(1)
    with pytest.raises(NotImplementedError, match=r"'exp_avg' of FlexShard parameter '.*' has shape \(1,\)"):
        opt.state_dict()


def _bf16_net(seed):
    torch.manual_seed(seed)
    return Net().to(torch.bfloat16)


def _fused_step(m, opt, seed):
    x = torch.randn(4, 6, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    m(x).float().square().mean().backward()
    opt.step()
    opt.zero_grad()


@pytest.mark.parametrize("warm_target", [False, True])
def test_fused_adamw_reload_keeps_fp32_moments(warm_target):
    """bf16 parameters: after ``load_state_dict`` both moments are still fp32 (the base optimizer would
    cast them to bf16), flat bucket buffers hold the loaded values, and the next step equals the
    uninterrupted run's; ``warm_target`` loads into an optimizer that already built flat buffers."""
    import copy

    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.optim.adamw import FusedAdamW

    a = _bf16_net(0)
    flex_shard(a, [BucketSpec(["*"])])
    oa = FusedAdamW(a.parameters(), lr=0.05)
    for s in range(2):
        _fused_step(a, oa, 10 + s)
    saved_model = copy.deepcopy(a.state_dict())
    saved_opt = copy.deepcopy(oa.state_dict())
    _fused_step(a, oa, 99)

    b = _bf16_net(5)
    flex_shard(b, [BucketSpec(["*"])])
    ob = FusedAdamW(b.parameters(), lr=0.05)
    if warm_target:
        _fused_step(b, ob, 3)
    b.load_state_dict(saved_model)
    ob.load_state_dict(saved_opt)
    for p in b.parameters():
        st = ob.state[p]
        assert st["exp_avg"].dtype == torch.float32 and st["exp_avg_sq"].dtype == torch.float32
        assert st["exp_avg"].shape == p.shape and int(st["step"]) == 2
    for p, q in zip(a.parameters(), b.parameters()):   # loaded moments equal the saved fp32 values
        pid = [id(x) for x in a.parameters()].index(id(p))
        assert torch.equal(ob.state[q]["exp_avg"], saved_opt["state"][pid]["exp_avg"].reshape(q.shape))
    _fused_step(b, ob, 99)
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.equal(p.detach(), q.detach())
        assert torch.equal(oa.state[p]["exp_avg_sq"], ob.state[q]["exp_avg_sq"])
    if ob._flat:   # flat buffers are the storage behind the per-parameter views
        flat = next(iter(ob._flat.values()))
        q = next(iter(b.parameters()))
        assert ob.state[q]["exp_avg"].untyped_storage().data_ptr() == flat["m"].untyped_storage().data_ptr()


def test_adamw_kernel_wrapper_rejects_narrow_moments():
    from flex_shard_b200.ops.elementwise import adamw_step_

    p = torch.zeros(8, dtype=torch.bfloat16)
    g = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="fp32"):
        adamw_step_(p, g, torch.zeros(8, dtype=torch.bfloat16), torch.zeros(8), lr=1e-3, beta1=0.9, beta2=0.99,
                    eps=1e-8, weight_decay=0.0, step=1)
    with pytest.raises(ValueError, match="at least"):
        adamw_step_(p, g, torch.zeros(4), torch.zeros(8), lr=1e-3, beta1=0.9, beta2=0.99, eps=1e-8,
                    weight_decay=0.0, step=1)


def _per_rank(rank, world, path):
    from flex_shard_b200 import checkpoint

    state = {"pos": checkpoint.PerRank({"file": rank, "seen": [rank] * 3}), "step": 7}
    checkpoint.save(state, path)
    back = {"pos": checkpoint.PerRank(None), "step": 0}
    checkpoint.load(back, path)
    return back["pos"].value, back["step"]


def test_per_rank_objects_come_back_to_their_rank(tmp_path):
    """Plain objects are taken from rank 0; values wrapped in ``PerRank`` are saved and restored rank by rank, and
    refuse to load at another world size."""
    from flex_shard_b200 import checkpoint

    path = str(tmp_path / "ckpt")
    res = run_ranks(_per_rank, 2, path)
    assert res[0] == ({"file": 0, "seen": [0, 0, 0]}, 7) and res[1] == ({"file": 1, "seen": [1, 1, 1]}, 7)
    with pytest.raises(RuntimeError, match="per-rank state saved by 2 ranks"):
        checkpoint.load({"pos": checkpoint.PerRank(None)}, path)       # one process, no group: world size 1


def _wrapped_and_tied(rank, world, path):
    from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper

    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard
    from flex_shard_b200.placement_contract import get_global_layout

    expected = torch.arange(20, dtype=torch.float32).view(5, 4)
    rows = [(0, 5)] if world == 1 else [(0, 3), (3, 5)]
    lo, hi = rows[rank]
    out = {}

    # (a) a sharded module under an activation-checkpoint wrapper, seen from a plain parent
    linear = nn.Linear(4, 5, bias=False)
    with torch.no_grad():
        linear.weight.copy_(expected)
    parent = nn.Module()
    parent.layer = checkpoint_wrapper(linear)
    flex_shard(parent.layer, [BucketSpec(["*"])])

    def tagged(m):
        sd = m.state_dict()
        checkpoint.set_state_dict_global_layouts(m, sd)
        return sd

    sd = tagged(parent)
    out["keys"] = list(sd)
    lay = get_global_layout(sd["layer.weight"])
    out["layout"] = (lay.global_shape, lay.global_offsets, lay.local_sizes)
    checkpoint.save(sd, os.path.join(path, "wrapped"))
    next(parent.parameters()).detach().fill_(-1)
    sd = tagged(parent)
    checkpoint.load(sd, os.path.join(path, "wrapped"))
    parent.load_state_dict(sd)
    out["wrapped_ok"] = torch.equal(next(parent.parameters()).detach(), expected[lo:hi])

    # (b) a tied weight: both names carry the layout, each is saved and loaded as the shard it is, and
    # the weight stays shared
    tied = nn.Module()
    tied.embed = nn.Embedding(5, 4)
    tied.head = nn.Linear(4, 5, bias=False)
    tied.head.weight = tied.embed.weight
    with torch.no_grad():
        tied.embed.weight.copy_(expected)
    flex_shard(tied, [BucketSpec(["*"])])
    sd = tagged(tied)
    out["tied_layouts"] = [get_global_layout(sd[k]) is not None
                           and get_global_layout(sd[k]) == get_global_layout(sd["embed.weight"])
                           for k in ("embed.weight", "head.weight")]
    checkpoint.save(sd, os.path.join(path, "tied"))
    tied.embed.weight.detach().fill_(-1)
    sd = tagged(tied)
    checkpoint.load(sd, os.path.join(path, "tied"))
    tied.load_state_dict(sd)
    out["still_shared"] = tied.head.weight is tied.embed.weight
    out["tied_ok"] = torch.equal(tied.embed.weight.detach(), expected[lo:hi])
    return out


@pytest.mark.parametrize("world", [1, 2])
def test_round_trip_of_a_checkpoint_wrapped_submodule_and_of_tied_weights(world, tmp_path):
    """Parity: ``flex_shard/tests/test_flex_shard_checkpoint.py:192-245`` of the reference."""
    for r, out in enumerate(run_ranks(_wrapped_and_tied, world, str(tmp_path))):
        assert out["keys"] == ["layer.weight"]
        lo, hi = ((0, 5),)[r] if world == 1 else ((0, 3), (3, 5))[r]
        assert out["layout"] == ((5, 4), ((lo, 0),), ((hi - lo, 4),))
        assert out["wrapped_ok"] and out["tied_ok"] and out["still_shared"]
        assert out["tied_layouts"] == [True, True]


def _load_failures(rank, world, path):
    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard

    def tagged(m):
        sd = m.state_dict()
        checkpoint.set_state_dict_global_layouts(m, sd)
        return sd

    saved = flex_shard(nn.Linear(4, 6), [BucketSpec(["*"])])
    checkpoint.save(tagged(saved), path)
    out = {}

    def attempt(name, sd):
        try:
            checkpoint.load(sd, path)
            out[name] = "loaded"
        except Exception as e:
            out[name] = f"{type(e).__name__}: {e}"

    # rows 0..3 of the taller weight are all in the files, rows 4..7 are not: without the shape check only rank 1 failed
    attempt("taller", tagged(flex_shard(nn.Linear(4, 8), [BucketSpec(["*"])])))
    attempt("renamed", tagged(flex_shard(nn.Sequential(nn.Linear(4, 6)), [BucketSpec(["*"])])))
    one_sided = tagged(saved)
    if rank == 1:
        one_sided["extra"] = torch.zeros(2)          # only this rank asks for a tensor the files do not have
    attempt("one_sided", one_sided)
    attempt("good", tagged(saved))
    return out


def test_load_failures_are_named_and_raise_on_every_rank(tmp_path):
    """A shape that differs from the saved one is a "size mismatch" (parity:
    ``tests/test_flex_shard_state_dict.py:68-75`` of the reference), a missing key is named, and a failure on one rank
    raises on the others too instead of leaving them in the closing barrier."""
    res = run_ranks(_load_failures, 2, str(tmp_path / "ckpt"))
    for rank, out in enumerate(res):
        assert "size mismatch for weight" in out["taller"] and "(6, 4)" in out["taller"], out
        assert out["renamed"].startswith("KeyError") and "0.weight not in checkpoint" in out["renamed"]
        assert out["good"] == "loaded"
    assert res[1]["one_sided"].startswith("KeyError") and "extra not in checkpoint" in res[1]["one_sided"]
    assert "failed on rank(s) [1]" in res[0]["one_sided"] and "extra not in checkpoint" in res[0]["one_sided"]
