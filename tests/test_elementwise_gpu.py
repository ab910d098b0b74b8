"""Bandwidth kernels against fp32 PyTorch references (the CPU path of the same wrappers)."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_rmsnorm_fwd_bwd():
    torch.manual_seed(0)
    x = torch.randn(3, 70, 512, device=DEV).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(512, device=DEV)).bfloat16().requires_grad_()
    y = ew.rmsnorm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xc = x.detach().cpu().requires_grad_()
    wc = w.detach().cpu().requires_grad_()
    yc = ew.rmsnorm(xc, wc, 1e-5)
    yc.backward(g.cpu())
    torch.testing.assert_close(y.cpu().float(), yc.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.cpu().float(), xc.grad.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad.cpu().float(), wc.grad.float(), rtol=3e-2, atol=1e-1)


def test_add_rmsnorm():
    torch.manual_seed(1)
    x = torch.randn(130, 256, device=DEV).bfloat16().requires_grad_()
    r = torch.randn(130, 256, device=DEV).bfloat16().requires_grad_()
    w = torch.ones(256, device=DEV).bfloat16().requires_grad_()
    y, s = ew.add_rmsnorm(x, r, w)
    (y.float().sum() + 2 * s.float().sum()).backward()
    xc, rc_, wc = (t.detach().cpu().requires_grad_() for t in (x, r, w))
    yc, sc = ew.add_rmsnorm(xc, rc_, wc)
    (yc.float().sum() + 2 * sc.float().sum()).backward()
    torch.testing.assert_close(y.cpu().float(), yc.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(s.cpu().float(), sc.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(x.grad.cpu().float(), xc.grad.float(), rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(r.grad.cpu().float(), rc_.grad.float(), rtol=2e-2, atol=3e-2)


def test_rope_roundtrip_and_reference():
    torch.manual_seed(2)
    B, S, H, hd = 2, 48, 4, 64
    table = ew.rope_table(S, hd, 5e5, DEV)
    x = torch.randn(B, S, H, hd, device=DEV).bfloat16()
    ref = ew._rope_ref(x.cpu(), table.cpu(), False)
    xr = x.clone().requires_grad_()
    y = ew.rope(xr * 1.0, table)
    torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
    g = torch.randn_like(y)
    y.backward(g)
    gref = ew._rope_ref(g.cpu(), table.cpu(), True)
    torch.testing.assert_close(xr.grad.cpu().float(), gref.float(), rtol=1e-2, atol=1e-2)


def test_swiglu():
    torch.manual_seed(3)
    gu = torch.randn(100, 2 * 320, device=DEV).bfloat16().requires_grad_()
    h = ew.swiglu(gu)
    g = torch.randn_like(h)
    h.backward(g)
    gc = gu.detach().cpu().requires_grad_()
    hc = ew.swiglu(gc)
    hc.backward(g.cpu())
    torch.testing.assert_close(h.cpu().float(), hc.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(gu.grad.cpu().float(), gc.grad.float(), rtol=2e-2, atol=2e-2)


def test_cross_entropy_matches_torch():
    torch.manual_seed(4)
    T, V = 64, 1024
    logits = (3 * torch.randn(T, V, device=DEV)).bfloat16()
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[5] = -100
    lf = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lf, tgt, reduction="sum") / T
    ref.backward()
    lg = logits.clone().requires_grad_()
    loss = ew.cross_entropy(lg * 1.0, tgt)
    loss.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(lg.grad.float(), lf.grad, rtol=2e-2, atol=2e-4)


@pytest.mark.parametrize("pdt,gdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                     (torch.float32, torch.bfloat16)])
def test_adamw_matches_torch(pdt, gdt):
    torch.manual_seed(5)
    n = 10007
    p0 = torch.randn(n, device=DEV)
    p = p0.to(pdt).clone()
    ref = torch.nn.Parameter(p.float().clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(gdt)
        ref.grad = g.float()
        opt.step()
        ew.adamw_step_(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        if pdt == torch.bfloat16:
            ref.data.copy_(ref.data.bfloat16().float())
    tol = 1e-5 if pdt == torch.float32 else 2e-2
    torch.testing.assert_close(p.float(), ref.data, rtol=tol, atol=tol)
    ops.check_status()


def test_cast_scale():
    a = torch.randn(5000, device=DEV)
    b = torch.zeros(5000, device=DEV, dtype=torch.bfloat16)
    ew.cast_scale_(b, a, 0.5)
    torch.testing.assert_close(b.float(), (a * 0.5).bfloat16().float())
    c = torch.ones(5000, device=DEV)
    ew.cast_scale_(c, b, 2.0, accumulate=True)
    torch.testing.assert_close(c, 1 + 2 * b.float())
