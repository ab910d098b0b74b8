"""DistMuon on CPU: math against a restated reference, owned vs redistributed storage on 2 gloo
ranks, planner goldens."""

import torch
import torch.nn as nn

from tests.common import run_ranks


def _ref_muon_step(p, g, m, lr=0.02, wd=0.1, mu=0.95, steps=5, eps=1e-7, mode=None):
    a, b, c = 3.4445, -4.7750, 2.0315
    m.lerp_(g, 1 - mu)
    u = g.lerp(m, mu)
    x = u.bfloat16()
    if x.shape[0] > x.shape[1]:
        x = x.t()
        tr = True
    else:
        tr = False
    x = x / x.float().norm().clamp_min(eps).bfloat16()
    for _ in range(steps):
        A = (x.float() @ x.float().t()).bfloat16()
        B = (b * A.float() + c * (A.float() @ A.float())).bfloat16()
        x = (a * x.float() + B.float() @ x.float()).bfloat16()
    if tr:
        x = x.t()
    from flex_shard_b200.dist_muon import lr_ratio

    p.mul_(1 - lr * wd).add_(x.float(), alpha=-lr * lr_ratio(mode, *p.shape))


def test_muon_owned_matches_reference_math():
    from flex_shard_b200.dist_muon import DistMuon

    torch.manual_seed(0)
    for shape in [(32, 64), (96, 32)]:
        p = nn.Parameter(torch.randn(*shape))
        ref_p, ref_m = p.detach().clone(), torch.zeros(*shape)
        opt = DistMuon([p], param_names=["w"], lr=0.02, adjust_lr_fn="match_rms_adamw")
        for _ in range(3):
            g = torch.randn(*shape)
            p.grad = g.clone()
            opt.step()
            _ref_muon_step(ref_p, g, ref_m, mode="match_rms_adamw")
        torch.testing.assert_close(p.detach(), ref_p, rtol=0, atol=2e-2)


def test_owner_stored_matrices_step_bitwise_like_torch_muon_across_a_state_dict_round_trip():
    """On CPU the step of a matrix that sits whole on its rank equals ``torch.optim.Muon`` bit for bit (same
    operations), also after the optimizer's state went through ``state_dict`` into an optimizer built with other
    hyper-parameters, which the loaded groups replace.  Restated from
    ``tests/test_dist_muon_optimizer.py:48-249`` of the reference."""
    import warnings

    from flex_shard_b200.dist_muon import DistMuon

    warnings.simplefilter("ignore")
    torch.manual_seed(0)
    for mode in ("match_rms_adamw", "original"):
        shapes = [(32, 64), (96, 32), (48, 48)]
        ours = [nn.Parameter(torch.randn(*s)) for s in shapes]
        theirs = [nn.Parameter(p.detach().clone()) for p in ours]
        kw = dict(lr=0.02, weight_decay=0.1, momentum=0.95, nesterov=True, adjust_lr_fn=mode)
        a = DistMuon(ours, param_names=[f"w{i}" for i in range(3)], **kw)
        b = torch.optim.Muon(theirs, **kw)

        def step(opt_a):
            for p, q in zip(ours, theirs):
                g = torch.randn(*p.shape)
                p.grad, q.grad = g.clone(), g.clone()
            opt_a.step()
            b.step()

        step(a)
        step(a)
        fresh = DistMuon(ours, param_names=[f"w{i}" for i in range(3)], lr=1.0, ns_steps=3, adjust_lr_fn=mode)
        fresh.load_state_dict(a.state_dict())
        assert fresh.param_groups[0]["ns_steps"] == 5 and fresh.param_groups[0]["lr"] == 0.02
        step(fresh)
        for p, q in zip(ours, theirs):
            assert torch.equal(p.detach(), q.detach()), (mode, tuple(p.shape))


def test_missing_grad_rejects_before_any_update():
    from flex_shard_b200.dist_muon import DistMuon

    a, b = nn.Parameter(torch.randn(8, 8)), nn.Parameter(torch.randn(8, 8))
    a0 = a.detach().clone()
    opt = DistMuon([a, b], param_names=["a", "b"])
    a.grad = torch.randn(8, 8)
    try:
        opt.step()
        raise AssertionError("expected a RuntimeError")
    except RuntimeError as e:
        assert "no gradient" in str(e)
    assert torch.equal(a.detach(), a0)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1 = nn.Linear(32, 64, bias=False)
        self.w2 = nn.Linear(64, 32, bias=False)
        self.heads = nn.Linear(32, 4 * 16, bias=False)  # 4 heads of 16 rows

    def forward(self, x):
        return self.w2(torch.relu(self.w1(x))) + self.heads(x)[:, :32]


def _train(rank, world, storage, steps, head_blocks=16):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.dist_muon import DistMuon, build_local_dist_muon, get_flex_shard_muon_compute_layouts
    from flex_shard_b200.placements import BlockShard, BucketedOwned
    import torch.distributed as dist

    torch.manual_seed(0)
    model = Net()
    if storage == "owned":
        def fn(named, mesh):
            out = {}
            for i, (n, p) in enumerate(named):
                out[n] = BlockShard((2, 2), 0) if n.startswith("heads") else BucketedOwned(((i % 2, 0, p.shape[0]),))
            return out
        flex_shard(model, [BucketSpec(["*"], placement_fn=fn, gradient_reduce_op=dist.ReduceOp.AVG)])
        opt = build_local_dist_muon(model, lr=0.02, block_rows_by_fqn={"heads.weight": head_blocks})
    else:
        flex_shard(model, [BucketSpec(["*"])])
        lays = get_flex_shard_muon_compute_layouts(model)
        names = [n for n, _ in model.named_parameters()]
        opt = DistMuon(list(model.parameters()), param_names=names, compute_layouts=lays, lr=0.02)
    for s in range(steps):
        xs = [torch.randn(8, 32, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)]
        model(xs[rank]).square().mean().backward()
        opt.step()
        opt.zero_grad()
    model.unshard()
    full = {n: p.detach().clone() for n, p in model.named_parameters()}
    model.reshard()
    return full, opt.collectives_issued


def _reference(world, steps, head_blocks=(16,)):
    torch.manual_seed(0)
    model = Net()
    moms = {n: torch.zeros_like(p) for n, p in model.named_parameters()}
    for s in range(steps):
        xs = [torch.randn(8, 32, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)]
        sum(model(x).square().mean() for x in xs).div(world).backward()
        with torch.no_grad():
            for n, p in model.named_parameters():
                if n.startswith("heads"):
                    pos = 0
                    while pos < p.shape[0]:
                        for rows in head_blocks:
                            sl = slice(pos, pos + rows)
                            _ref_muon_step(p[sl], p.grad[sl], moms[n][sl], mode=None)
                            pos += rows
                else:
                    _ref_muon_step(p, p.grad, moms[n], mode=None)
        model.zero_grad()
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def test_muon_owned_storage_is_comm_free_and_matches():
    ref = _reference(2, 3)
    res = run_ranks(_train, 2, "owned", 3)
    for full, ncoll in res:
        assert ncoll == 0
        for n in ref:
            torch.testing.assert_close(full[n], ref[n], rtol=0, atol=3e-2)


def test_blocks_of_two_sizes_repeat_down_the_rows():
    """``block_rows_by_fqn = {name: (12, 4)}``: every head is two matrices (12 rows, then 4 rows), each orthogonalised
    on its own, whether the head blocks are spread over the ranks or not; rows that are not whole periods are refused.
    Parity: ``BlockShard(dim=0, block_sizes=(a, b))`` compute layouts of the reference's Kimi recipe
    (``examples/deepseek_v3/muon.py:29-48``)."""
    import pytest

    ref = _reference(2, 3, head_blocks=(12, 4))
    plain = _reference(2, 3)
    assert not torch.equal(ref["heads.weight"], plain["heads.weight"])
    for full, ncoll in run_ranks(_train, 2, "owned", 3, (12, 4)):
        assert ncoll == 0
        for n in ref:
            torch.testing.assert_close(full[n], ref[n], rtol=0, atol=3e-2)
    err = float((full["heads.weight"] - ref["heads.weight"]).abs().max())
    other = float((full["heads.weight"] - plain["heads.weight"]).abs().max())
    assert err < other          # closer to the two-matrix reference than to the one-matrix-per-head one
    with pytest.raises(AssertionError, match="whole blocks|whole repetitions"):
        run_ranks(_train, 2, "owned", 1, (12, 5))


def test_muon_row_shard_storage_redistributes_and_matches():
    ref = _reference(2, 3)
    res = run_ranks(_train, 2, "shard", 3)
    for full, ncoll in res:
        assert ncoll == 2 * 3
        for n in ref:
            if n.startswith("heads"):
                continue  # stored Shard(0): orthogonalised as one matrix here, per head in the reference run
            torch.testing.assert_close(full[n], ref[n], rtol=0, atol=3e-2)


def test_assign_matrices_goldens():
    from flex_shard_b200.dist_muon import MatrixSpec, assign_matrices

    q, w = MatrixSpec("q", (64, 64)), MatrixSpec("w", (256, 64))
    assert assign_matrices([[q, w]], 2) == {"w": 0, "q": 1}
    # carried loads spread identical buckets over the mesh
    groups = [[MatrixSpec(f"b{i}.w", (128, 128))] for i in range(16)]
    spread = set(assign_matrices(groups, 64, ranks_per_host=8, carry_loads=True).values())
    same = set(assign_matrices(groups, 64, ranks_per_host=8, carry_loads=False).values())
    assert len(spread) == 16 and len(same) == 1
    # block groups return blocks-per-rank
    heads = MatrixSpec("wq", (8 * 16, 64), num_blocks=8)
    assert sum(assign_matrices([[heads]], 4)["wq"]) == 8
