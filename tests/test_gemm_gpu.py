"""tcgen05 bf16 GEMM against an fp32 PyTorch reference, all operand layouts."""
import pytest
import torch

from flex_shard_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(a, b, a_t, b_t):
    af = (a.t() if a_t else a).float()
    bf = (b.t() if b_t else b).float()
    return af @ bf.t()


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 320, 192), (1000, 264, 136),
                                   (2048, 1024, 4096)])
def test_gemm_layouts(M, N, K, a_t, b_t):
    if (a_t and M % 8) or (b_t and N % 8):
        pytest.skip("transposed operands need a multiple of 8")
    torch.manual_seed(0)
    dev = torch.device("cuda")
    a = torch.randn((K, M) if a_t else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_t else (N, K), device=dev).bfloat16()
    out = ops.gemm(a, b, a_t=a_t, b_t=b_t, out_dtype=torch.float32)
    ops.check_status()
    ref = _ref(a, b, a_t, b_t)
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-3 * K ** 0.5)
    out16 = ops.gemm(a, b, a_t=a_t, b_t=b_t)
    ops.check_status()
    torch.testing.assert_close(out16.float(), ref, rtol=2e-2, atol=2e-2 * K ** 0.5)


def test_gemm_epilogue_variants():
    torch.manual_seed(1)
    dev = torch.device("cuda")
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device=dev).bfloat16()
    b = torch.randn(N, K, device=dev).bfloat16()
    c = torch.randn(M, N, device=dev).bfloat16()
    ref = 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float()
    out = ops.gemm(a, b, c=c, alpha=0.5, beta=2.0, out_dtype=torch.float32)
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=5e-2)
    acc = torch.ones(M, N, device=dev, dtype=torch.float32)
    ops.gemm(a, b, out=acc, accumulate=True)
    torch.testing.assert_close(acc, a.float() @ b.float().t() + 1.0, rtol=2e-3, atol=5e-2)
    acc.fill_(1.0)
    ops.gemm(a, b, out=acc, accumulate=True)
    ops.gemm(a, b, out=acc, accumulate=True)
    torch.testing.assert_close(acc, 2 * (a.float() @ b.float().t()) + 1.0, rtol=2e-3, atol=1e-1)
    ops.check_status()


def test_linear_autograd_matches_torch():
    torch.manual_seed(2)
    dev = torch.device("cuda")
    x = torch.randn(4, 96, 256, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device=dev) * 0.05).bfloat16().requires_grad_()
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=2e-1)
    ops.check_status()


@pytest.mark.parametrize("n,k", [(1024, 512), (2304, 1024), (4096, 640)])
def test_symmetric_product_computes_upper_tiles_and_mirrors(n, k):
    """``symmetric=True``: X X^T (and a symmetric matrix times itself with a symmetric addend) must equal the
    full product; the result is exactly symmetric."""
    torch.manual_seed(0)
    dev = torch.device("cuda")
    x = torch.randn(n, k, device=dev).bfloat16()
    full = ops.gemm(x, x)
    sym = ops.gemm(x, x, symmetric=True)
    ref = x.float() @ x.float().t()
    torch.testing.assert_close(sym.float(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()) / 16)
    assert torch.equal(sym, sym.t())
    assert torch.equal(torch.triu(sym), torch.triu(full))          # the computed half is the same arithmetic
    a = sym
    full2 = ops.gemm(a, a, c=a, alpha=0.5, beta=-1.5)
    sym2 = ops.gemm(a, a, c=a, alpha=0.5, beta=-1.5, symmetric=True)
    assert torch.equal(torch.triu(sym2), torch.triu(full2)) and torch.equal(sym2, sym2.t())
    xt = x.t().contiguous()                                          # [k, n]: A = X^T X through the transposed modes
    sym3 = ops.gemm(xt, xt, a_t=True, b_t=True, symmetric=True)
    torch.testing.assert_close(sym3.float(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()) / 16)
    ops.check_status()
