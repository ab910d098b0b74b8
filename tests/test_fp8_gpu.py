"""FP8 blockwise quantisers (bitwise vs the PyTorch restatement) and the block-scaled GEMM."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import fp8

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("shape", [(256, 384), (300, 200), (128, 128), (1, 130)])
def test_weight_quantiser_bitwise_matches_reference(shape):
    torch.manual_seed(0)
    w = (torch.randn(*shape, device=DEV) * 3).bfloat16()
    q, s = fp8.quantize_blockwise(w)
    qr, sr = fp8.quantize_blockwise_ref(w)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(s, sr)


def test_local_quantisation_equals_quantise_after_gather():
    """Quantising whole 128-row blocks separately gives the same bytes as quantising the full matrix."""
    torch.manual_seed(1)
    w = torch.randn(512, 256, device=DEV).bfloat16()
    q, s = fp8.quantize_blockwise(w)
    for lo, hi in [(0, 128), (128, 512)]:
        ql, sl = fp8.quantize_blockwise(w[lo:hi])
        assert torch.equal(ql.view(torch.uint8), q[lo:hi].view(torch.uint8))
        assert torch.equal(sl, s[lo // 128: hi // 128])


def test_act_quantiser_bitwise_matches_reference():
    torch.manual_seed(2)
    x = torch.randn(200, 512, device=DEV).bfloat16()
    q, s = fp8.quantize_act(x)
    qr, sr = fp8.quantize_act_ref(x)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(s, sr)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 640, 1024)])
def test_fp8_gemm_forward_and_transposed(M, N, K):
    torch.manual_seed(3)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    wq, ws = fp8.quantize_blockwise(w)
    xq, sx = fp8.quantize_act(x)
    y = fp8.gemm_fp8(xq, sx, wq, ws)
    ops.check_status()
    ref = (xq.float().view(M, K // 128, 128) * sx.t()[..., None]).view(M, K) @ fp8.dequantize_blockwise(wq, ws).t()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2 * K ** 0.5)
    # transposed use of the same weight (dgrad): dy [M, N] @ W [N, K]
    dy = torch.randn(M, N, device=DEV).bfloat16()
    dq, sd = fp8.quantize_act(dy)
    dx = fp8.gemm_fp8(dq, sd, wq, ws, b_t=True)
    ops.check_status()
    ref2 = (dq.float().view(M, N // 128, 128) * sd.t()[..., None]).view(M, N) @ fp8.dequantize_blockwise(wq, ws)
    torch.testing.assert_close(dx.float(), ref2, rtol=2e-2, atol=2e-2 * N ** 0.5)


def test_fp8_linear_close_to_bf16_linear():
    torch.manual_seed(4)
    x = torch.randn(4, 64, 512, device=DEV).bfloat16().requires_grad_()
    w = (0.05 * torch.randn(768, 512, device=DEV)).bfloat16().requires_grad_()
    wq, ws = fp8.quantize_blockwise(w.detach())
    y = fp8.fp8_linear(x, w, wq, ws)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.15 * yr.abs().max()
    assert (x.grad.float() - xr.grad).abs().max() < 0.15 * xr.grad.abs().max()
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=3e-2, atol=3e-1)
    ops.check_status()


def test_stacked_fp8_linear_runs_every_matrix_through_its_own_tiles():
    """A stacked weight [E, out, in] quantised as its matrices one under the other: every x[e] goes through matrix e;
    forward, input gradient and stacked weight gradient against per-matrix fp32 linears."""
    from flex_shard_b200.quant import FlexShardFloat8BlockwiseStackedLinear

    torch.manual_seed(5)
    E, T, cin, cout = 3, 128, 512, 256
    lin = FlexShardFloat8BlockwiseStackedLinear(E, cin, cout, device=DEV)
    with torch.no_grad():
        lin.weight.copy_(0.05 * torch.randn(E, cout, cin, device=DEV))
    x = torch.randn(E, T, cin, device=DEV).bfloat16().requires_grad_()
    y = lin(x)
    g = torch.randn_like(y)
    y.backward(g)
    ops.check_status()
    xr = x.detach().float().requires_grad_()
    wr = lin.weight.detach().float().requires_grad_()
    yr = torch.einsum("etk,enk->etn", xr, wr)
    yr.backward(g.float())
    assert y.shape == (E, T, cout)
    assert (y.float() - yr).abs().max() < 0.15 * yr.abs().max()
    assert (x.grad.float() - xr.grad).abs().max() < 0.15 * xr.grad.abs().max()
    torch.testing.assert_close(lin.weight.grad.float(), wr.grad, rtol=3e-2, atol=3e-1)
