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


@pytest.mark.parametrize("mode,normalize,E,k", [("sigmoid", True, 256, 8), ("softmax", True, 8, 2),
                                                ("softmax", False, 64, 6), ("sigmoid", True, 40, 3)])
def test_router_kernel_matches_reference(mode, normalize, E, k):
    torch.manual_seed(3)
    T = 1000
    logits = torch.randn(T, E) * 2
    bias = torch.randn(E) * 0.1 if mode == "sigmoid" else None
    res = {}
    for dev in ("cpu", "cuda"):
        lg = logits.clone().to(dev).requires_grad_()
        counts = torch.zeros(E, device=dev)
        idx, w = moe.route_topk(lg, k, bias=None if bias is None else bias.to(dev), mode=mode, scale=2.5,
                                normalize=normalize, counts=counts)
        (w * torch.arange(1, k + 1, device=dev)).sum().backward()
        res[dev] = (idx.cpu(), w.detach().cpu(), counts.cpu(), lg.grad.cpu())
    assert torch.equal(res["cpu"][0], res["cuda"][0])
    torch.testing.assert_close(res["cpu"][1], res["cuda"][1], rtol=1e-4, atol=1e-6)
    assert torch.equal(res["cpu"][2], res["cuda"][2])
    torch.testing.assert_close(res["cpu"][3], res["cuda"][3], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("T,k,E", [(300, 2, 4), (4096, 6, 64), (7, 1, 8), (50000, 1, 16), (1000, 8, 256), (33, 3, 5)])
def test_route_plan_kernel_equals_operator_plan(T, k, E):
    """Histogram, padded offsets, tile table and stable rows from the one-launch kernel equal the plan
    computed with sort / bincount / cumsum operators, exactly; skewed and empty experts included."""
    g = torch.Generator().manual_seed(T + E)
    idx = torch.randint(0, E, (T, k), generator=g)
    idx[idx == E - 1] = 0                      # the last expert stays empty, the first is overloaded
    for dtype in (torch.int64, torch.int32):
        before = ops.launch_count()
        got = moe.plan_routes(idx.to("cuda", dtype), E)
        assert ops.launch_count() - before == 1
        want = moe.plan_routes(idx, E)         # CPU tensors take the operator path
        torch.cuda.synchronize()
        assert torch.equal(got.pos.cpu(), want.pos)
        assert torch.equal(got.src.cpu(), want.src)
        assert torch.equal(got.offs.cpu(), want.offs)
        assert int(got.num_mtiles) == int(want.num_mtiles)
        n_tiles = int(want.num_mtiles)
        assert torch.equal(got.tile_expert.cpu()[:n_tiles], want.tile_expert[:n_tiles])
        assert got.max_rows == want.max_rows
    ops.check_status()
