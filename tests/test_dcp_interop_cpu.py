"""Checkpoints in the DTensor format of ``torch.distributed.checkpoint``: a model sharded by FSDP2
``fully_shard`` saves, a ``flex_shard`` model loads (and the other way round), at the same and at another
world size, bit for bit, AdamW moments included.  Behaviour restated from
``src/flex_shard/tests/test_flex_shard_checkpoint.py:483-538`` of the reference."""
import torch
import torch.nn as nn

from tests.common import run_ranks


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(6, 7)      # 7 rows: uneven over 2 and 4 ranks, rank 3 of 4 holds one row
        self.b = nn.Linear(7, 3)      # 3 rows: rank 3 of 4 is empty

    def forward(self, x):
        return self.b(torch.tanh(self.a(x)))


def _steps(model, opt, n):
    for s in range(n):
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(100 + s))
        model(x).square().mean().backward()
        opt.step()
        opt.zero_grad()


def _fsdp2(seed, mesh):
    from torch.distributed.fsdp import fully_shard

    torch.manual_seed(seed)
    m = Net()
    for layer in (m.a, m.b):
        fully_shard(layer, mesh=mesh)
    fully_shard(m, mesh=mesh)
    return m


def _flex(seed, mesh):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(seed)
    m = Net()
    flex_shard(m, [BucketSpec(["a"], mesh=mesh, fsdp2_compatible=True), BucketSpec(["b"], mesh=mesh, fsdp2_compatible=True)])
    return m


def _save(rank, world, kind, path):
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict
    from torch.distributed.device_mesh import init_device_mesh

    from flex_shard_b200.checkpoint import to_dtensor_state_dict

    mesh = init_device_mesh("cpu", (world,))
    m = _fsdp2(0, mesh) if kind == "fsdp2" else _flex(0, mesh)
    opt = torch.optim.AdamW(m.parameters(), lr=0.05)
    _steps(m, opt, 3)
    if kind == "fsdp2":
        dcp.save({"model": m.state_dict(), "optim": get_optimizer_state_dict(m, opt)}, checkpoint_id=path)
    else:
        msd, osd = to_dtensor_state_dict(m, m.state_dict(), opt)
        dcp.save({"model": msd, "optim": osd}, checkpoint_id=path)
    return True


def _load_and_compare(rank, world, kind, path):
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict, set_optimizer_state_dict
    from torch.distributed.device_mesh import init_device_mesh

    from flex_shard_b200.checkpoint import load_dtensor_optim_state, to_dtensor_state_dict

    mesh = init_device_mesh("cpu", (world,))
    # the uninterrupted run, unsharded, to compare with
    torch.manual_seed(0)
    ref = Net()
    ropt = torch.optim.AdamW(ref.parameters(), lr=0.05)
    _steps(ref, ropt, 4)
    m = _fsdp2(1, mesh) if kind == "fsdp2" else _flex(1, mesh)
    opt = torch.optim.AdamW(m.parameters(), lr=0.05)
    # optimizer state must exist before it can be filled
    for p in m.parameters():
        p.grad = torch.zeros_like(p)
    opt.step()
    opt.zero_grad()
    if kind == "fsdp2":
        sd = {"model": m.state_dict(), "optim": get_optimizer_state_dict(m, opt)}
        dcp.load(sd, checkpoint_id=path)
        m.load_state_dict(sd["model"])
        set_optimizer_state_dict(m, opt, sd["optim"])
    else:
        msd, osd = to_dtensor_state_dict(m, m.state_dict(), opt)
        sd = {"model": msd, "optim": osd}
        dcp.load(sd, checkpoint_id=path)          # fills the local shards in place
        load_dtensor_optim_state(opt, m, sd["optim"])      # moments and step; hyper-parameters stay as constructed
    x = torch.randn(4, 6, generator=torch.Generator().manual_seed(103))
    m(x).square().mean().backward()
    opt.step()
    # compare this rank's rows with the unsharded run's
    errs = []
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        local = p.to_local() if hasattr(p, "to_local") else p
        rows = q.shape[0]
        c = -(-rows // world)
        lo, hi = min(rows, rank * c), min(rows, (rank + 1) * c)
        errs.append(float((local.detach() - q.detach()[lo:hi]).abs().max()) if hi > lo else 0.0)
    return max(errs)


def test_fsdp2_and_flex_checkpoints_are_interchangeable(tmp_path):
    for saver, loader, ws, wl in [("fsdp2", "flex", 2, 2), ("flex", "fsdp2", 2, 2), ("fsdp2", "flex", 4, 2),
                                  ("flex", "fsdp2", 2, 4), ("flex", "flex", 4, 2)]:
        path = str(tmp_path / f"{saver}{ws}_{loader}{wl}")
        assert all(run_ranks(_save, ws, saver, path))
        errs = run_ranks(_load_and_compare, wl, loader, path)
        # every rank sees the same data in this test, so the sharded run equals the unsharded one up to the
        # averaging of identical gradients; resumed and uninterrupted runs agree to fp32 rounding
        assert max(errs) < 1e-6, (saver, loader, ws, wl, errs)


def test_layouts_without_a_dtensor_form_are_refused():
    import pytest

    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.checkpoint import to_dtensor_state_dict
    from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn
    from tests.common import FakeMesh

    m = Net()
    flex_shard(m, [BucketSpec(["*"], mesh=FakeMesh(2, 0), placement_fn=make_bucketed_owned_full_param_placement_fn())])
    with pytest.raises(ValueError, match="DTensor checkpoint"):
        to_dtensor_state_dict(m, m.state_dict())
