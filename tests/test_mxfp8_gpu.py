"""MXFP8 quantisers and the block-scaled tcgen05 GEMM against the PyTorch restatement of the format."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import mxfp8 as mx

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(256, 256), (200, 384), (96, 160), (1024, 512)])
def test_weight_quantiser_matches_reference_bitwise(rows, cols):
    torch.manual_seed(0)
    w = (torch.randn(rows, cols) * torch.rand(rows, 1) * 3).bfloat16()
    w[5:37, 64:96] = 0     # an all-zero tile
    q_ref, e_ref = mx.mx_quantize_weight(w)
    q, e = mx.mx_quantize_weight(w.cuda())
    assert torch.equal(e.cpu(), e_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    for tr in (False, True):
        assert torch.equal(mx.mx_expand_scales(e, rows, cols, tr).cpu(), mx.mx_expand_scales(e_ref, rows, cols, tr))
    ops.check_status()


@pytest.mark.parametrize("T,K", [(128, 128), (300, 512), (77, 256)])
def test_activation_quantiser_matches_reference_bitwise(T, K):
    torch.manual_seed(1)
    x = (torch.randn(T, K) * 5).bfloat16()
    x[3, 32:64] = 0
    q_ref, s_ref = mx.mx_quantize_act(x)
    q, s = mx.mx_quantize_act(x.cuda())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(mx.from_blocked(s.cpu(), T, K // 32), mx.from_blocked(s_ref, T, K // 32))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (300, 200, 256), (1024, 1024, 2048)])
def test_block_scaled_gemm_matches_dequantised_product(M, N, K):
    torch.manual_seed(2)
    dev = torch.device("cuda")
    x = (torch.randn(M, K, device=dev) * (1 + 4 * torch.rand(M, 1, device=dev))).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
    xq, sx = mx.mx_quantize_act(x)
    wq, e = mx.mx_quantize_weight(w)
    fwd = mx.mx_expand_scales(e, N, K, False)
    y = mx.gemm_mxfp8(xq, sx, wq, fwd, out_dtype=torch.float32)
    ops.check_status()
    ref = mx.mx_dequantize(xq, sx) @ mx.mx_dequantize(wq, fwd).t()
    torch.testing.assert_close(y, ref, rtol=1e-3, atol=1e-3 * K ** 0.5)
    if N % 128 == 0 and K % 16 == 0:
        # input-gradient orientation: contraction over the weight's rows, the weight read transposed
        dy = torch.randn(M, N, device=dev).bfloat16()
        dq, sd = mx.mx_quantize_act(dy)
        dgs = mx.mx_expand_scales(e, N, K, True)
        dx = mx.gemm_mxfp8(dq, sd, wq, dgs, b_t=True, out_dtype=torch.float32)
        ops.check_status()
        wt = wq.float().t() * torch.exp2(mx.from_blocked(dgs, K, N // 32).float() - 127).repeat_interleave(32, 1)
        ref2 = mx.mx_dequantize(dq, sd) @ wt.t()
        torch.testing.assert_close(dx, ref2, rtol=1e-3, atol=1e-3 * N ** 0.5)


def test_mxfp8_linear_gpu_matches_cpu_restatement():
    from flex_shard_b200.quant import FlexShardMxfp8BlockwiseLinear

    torch.manual_seed(4)
    res = {}
    w0 = (torch.randn(384, 256) * 0.05).bfloat16()
    x0 = torch.randn(4, 50, 256).bfloat16()
    g0 = torch.randn(4, 50, 384).bfloat16()
    for dev in ("cpu", "cuda"):
        lin = FlexShardMxfp8BlockwiseLinear(256, 384, device=dev)
        with torch.no_grad():
            lin.weight.copy_(w0)
        x = x0.clone().to(dev).requires_grad_()
        y = lin(x)
        y.backward(g0.to(dev))
        res[dev] = [t.detach().float().cpu() for t in (y, x.grad, lin.weight.grad)]
    ops.check_status()
    for a, b in zip(res["cpu"], res["cuda"]):
        torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2 * max(1.0, a.abs().max().item()))


@pytest.mark.parametrize("T,K", [(128, 128), (512, 384)])
def test_row_group_quantiser_matches_reference_bitwise(T, K):
    torch.manual_seed(5)
    x = (torch.randn(T, K) * 3).bfloat16()
    x[32:64, 7] = 0
    q_ref, s_ref = mx.mx_quantize_rows(x)
    q, s = mx.mx_quantize_rows(x.cuda())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu(), s_ref)


@pytest.mark.parametrize("T,N,K", [(128, 128, 128), (512, 256, 384), (2048, 1024, 512)])
def test_weight_gradient_product_reads_both_operands_transposed(T, N, K):
    torch.manual_seed(6)
    dev = torch.device("cuda")
    dy = torch.randn(T, N, device=dev).bfloat16()
    x = (torch.randn(T, K, device=dev) * 2).bfloat16()
    dq, sd = mx.mx_quantize_rows(dy)
    xq, sx = mx.mx_quantize_rows(x)
    dw = mx.gemm_mxfp8(dq, sd, xq, sx, a_t=True, b_t=True, out_dtype=torch.float32)
    ops.check_status()
    ref = mx.gemm_mxfp8(dq.cpu(), sd.cpu(), xq.cpu(), sx.cpu(), a_t=True, b_t=True, out_dtype=torch.float32)
    torch.testing.assert_close(dw.cpu(), ref, rtol=1e-3, atol=1e-3 * T ** 0.5)
