"""The communication-free Muon builder and the checkpoint form of Muon's state on 2 gloo ranks: Shard(0)-stored matrices
are refused, owner-stored ones step without a collective, the momentum (tagged with the parameters' layouts) survives
a save / load into a fresh optimizer so that the next step is the same bits, and bad states are refused.
Parity: the behaviours pinned by the reference's ``tests/test_dist_muon.py:404-560`` and the adapter's momentum
translation (``dist_muon/comm_free_adapter.py:103-131``)."""
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(16, 32, bias=False)
        self.b = nn.Linear(32, 16, bias=False)
        self.norm = nn.LayerNorm(16)

    def forward(self, x):
        return self.norm(self.b(torch.relu(self.a(x))))


def _owner_model():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn

    torch.manual_seed(0)
    m = Net()
    flex_shard(m, [BucketSpec(["a.*", "b.*"], placement_fn=make_bucketed_owned_full_param_placement_fn()),
                   BucketSpec(["norm.*"])])
    return m


def _work(rank, world, tmp):
    import torch.distributed as dist

    from flex_shard_b200 import BucketSpec, checkpoint, flex_shard
    from flex_shard_b200.dist_muon import build_local_dist_muon, load_muon_checkpoint_state, muon_checkpoint_state
    from flex_shard_b200.placement_contract import get_global_layout

    out = {}
    # matrices stored as Shard(0) on two ranks need redistribution: the communication-free builder refuses them
    plain = Net()
    flex_shard(plain, [BucketSpec(["*"])])
    try:
        build_local_dist_muon(plain)
        out["shard0"] = ""
    except ValueError as e:
        out["shard0"] = str(e)

    def boom(*a, **k):
        raise AssertionError("the owner-stored Muon step must not call a collective")

    def data(step):
        return torch.randn(8, 16, generator=torch.Generator().manual_seed(100 * step + rank))

    m = _owner_model()
    opt = build_local_dist_muon(m, lr=0.02)
    state0 = muon_checkpoint_state(opt, m)
    out["unstepped_zero"] = all(float(t.abs().sum()) == 0.0 for t in state0["momentum"].values())
    out["keys"] = sorted(state0["momentum"])
    out["tagged"] = all(get_global_layout(t) is not None for t in state0["momentum"].values())
    saved = {n: getattr(dist, n) for n in ("all_reduce", "all_gather_into_tensor", "reduce_scatter_tensor", "all_to_all_single")}
    for s in range(2):
        m(data(s)).square().mean().backward()
        for n in saved:
            setattr(dist, n, boom)
        try:
            opt.step()
        finally:
            for n, f in saved.items():
                setattr(dist, n, f)
        opt.zero_grad()
    out["zero_grad_none"] = all(p.grad is None for g in opt.param_groups for p in g["params"])
    sd = m.state_dict()
    from flex_shard_b200 import set_state_dict_global_layouts

    set_state_dict_global_layouts(m, sd)
    checkpoint.save({"model": sd, "muon": muon_checkpoint_state(opt, m)}, tmp)
    # the uninterrupted run's next step
    m(data(2)).square().mean().backward()
    opt.step()
    want = {n: p.detach().clone() for n, p in m.named_parameters()}
    # a fresh model + optimizer restored from the checkpoint takes the same step
    m2 = _owner_model()
    opt2 = build_local_dist_muon(m2, lr=0.02)
    sd2 = m2.state_dict()
    set_state_dict_global_layouts(m2, sd2)
    st2 = {"model": sd2, "muon": muon_checkpoint_state(opt2, m2)}
    checkpoint.load(st2, tmp)
    m2.load_state_dict(st2["model"])
    load_muon_checkpoint_state(opt2, st2["muon"])
    m2(data(2)).square().mean().backward()
    opt2.step()
    out["resumed_bitwise"] = all(torch.equal(p.detach(), want[n]) for n, p in m2.named_parameters())
    # refused states
    bad = muon_checkpoint_state(opt2, m2)
    name = out["keys"][0]
    bad["momentum"][name] = torch.zeros(3)
    try:
        load_muon_checkpoint_state(opt2, bad)
        out["bad_shape"] = ""
    except ValueError as e:
        out["bad_shape"] = str(e)
    del bad["momentum"][name]
    try:
        load_muon_checkpoint_state(opt2, bad)
        out["missing"] = ""
    except KeyError as e:
        out["missing"] = str(e)
    # zero_grad(set_to_none=False) keeps zeroed gradients
    m2(data(3)).square().mean().backward()
    opt2.zero_grad(set_to_none=False)
    out["zero_grad_zeros"] = all(p.grad is None or float(p.grad.abs().sum()) == 0.0
                                 for g in opt2.param_groups for p in g["params"])
    return out


def test_owner_stored_muon_checkpoint_round_trip(tmp_path):
    res = run_ranks(_work, 2, str(tmp_path / "ckpt"))
    for r in res:
        assert "Shard(0) on several ranks" in r["shard0"]
        assert r["unstepped_zero"] and r["tagged"] and r["keys"] == ["a.weight", "b.weight"]
        assert r["zero_grad_none"] and r["zero_grad_zeros"]
        assert r["resumed_bitwise"], r
        assert "has shape (3,)" in r["bad_shape"] and "no Muon momentum" in r["missing"]
