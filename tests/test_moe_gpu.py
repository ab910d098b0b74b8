"""MoE dispatch / grouped tcgen05 GEMM / combine on the GPU against the CPU reference paths."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import moe

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,k,E,D,F", [(300, 2, 4, 256, 384), (2048, 6, 64, 512, 256), (64, 1, 8, 128, 128)])
def test_moe_layer_matches_cpu_reference(T, k, E, D, F):
    torch.manual_seed(0)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    x = torch.randn(T, D).bfloat16()
    w1 = (0.1 * torch.randn(E, F, D)).bfloat16()
    gw = torch.rand(T, k)
    res = {}
    for dev in ("cpu", "cuda"):
        xi = x.clone().to(dev).requires_grad_()
        wi = w1.clone().to(dev).requires_grad_()
        gi = gw.clone().to(dev).requires_grad_()
        plan = moe.plan_routes(idx.to(dev), E)
        y = moe.moe_combine(moe.grouped_linear(moe.moe_dispatch(xi, plan), wi, plan), gi, plan)
        y.float().square().sum().backward()
        res[dev] = [t.detach().float().cpu() for t in (y, xi.grad, wi.grad, gi.grad)]
    ops.check_status()
    names = ["y", "dx", "dw", "dgate"]
    for n, a, b in zip(names, res["cpu"], res["cuda"]):
        scale = max(a.abs().max().item(), 1e-3)
        assert (a - b).abs().max().item() < 4e-2 * scale, (n, (a - b).abs().max().item(), scale)
