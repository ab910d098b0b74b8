"""Numerics at the shapes the benchmark runs (sequence 8192, FFN width 14336, vocabulary 128256) against plain
PyTorch fp32 references: the three products of the gate/up projection, flash attention forward/backward on
8192-token sequences with grouped KV heads, and the fused cross-entropy over the full vocabulary."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import attention as att
from flex_shard_b200.ops import elementwise as ew

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_ffn_products_at_llama_width():
    """x [8192, 4096] . W13 [28672, 4096]^T and its two gradients (MN-major operands read in place)."""
    torch.manual_seed(0)
    M, N, K = 8192, 2 * 14336, 4096
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
    dy = (torch.randn(M, N, device=DEV) * 0.1).bfloat16()
    y = ops.gemm(x, w)                                           # forward
    dx = ops.gemm(dy, w, b_t=True)                               # dgrad: dy . W
    dw = ops.gemm(dy, x, a_t=True, b_t=True, out_dtype=torch.float32)   # wgrad: dy^T . x
    ops.check_status()
    # compare 512-row / 512-column slabs in fp32 (a full fp32 reference would need 3 GEMMs of 2 TFLOP each)
    rows = slice(3000, 3512)
    torch.testing.assert_close(y[rows].float(), x[rows].float() @ w.float().t(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dx[rows].float(), dy[rows].float() @ w.float(), rtol=2e-2, atol=5e-2)
    cols = slice(20000, 20512)
    ref_dw = dy[:, cols].float().t() @ x.float()
    torch.testing.assert_close(dw[cols], ref_dw, rtol=2e-3, atol=2e-3 * M ** 0.5)


def test_attention_at_sequence_8192():
    torch.manual_seed(1)
    B, S, Hq, Hkv = 1, 8192, 4, 1
    C = (Hq + 2 * Hkv) * 128
    qkv = (0.5 * torch.randn(B, S, C, device=DEV)).bfloat16()
    x = qkv.clone().requires_grad_()
    o = att.qkv_attention(x * 1.0, None, Hq, Hkv)
    g = torch.randn_like(o)
    o.backward(g)
    ops.check_status()
    ref_in = qkv.clone().float().requires_grad_()
    q = ref_in[..., : Hq * 128].reshape(B, S, Hq, 128)
    k = ref_in[..., Hq * 128:(Hq + Hkv) * 128].reshape(B, S, Hkv, 128)
    v = ref_in[..., (Hq + Hkv) * 128:].reshape(B, S, Hkv, 128)
    oref = att.attention_ref(q, k, v).reshape(B, S, Hq * 128)      # fp32, materialises the [4, 8192, 8192] scores
    oref.backward(g.float())
    torch.testing.assert_close(o.float(), oref, rtol=2e-2, atol=2e-2)
    gr = ref_in.grad
    scale = gr.abs().max().item()
    assert (x.grad.float() - gr).abs().max().item() < 3e-2 * max(scale, 1.0)


def test_cross_entropy_over_the_full_vocabulary():
    torch.manual_seed(2)
    T, V = 2048, 128256
    logits = (2 * torch.randn(T, V, device=DEV)).bfloat16()
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[7] = -100
    lf = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lf, tgt, reduction="sum") / T
    ref.backward()
    lg = logits.clone().requires_grad_()
    loss = ew.cross_entropy(lg * 1.0, tgt)
    loss.backward()
    ops.check_status()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(lg.grad.float(), lf.grad, rtol=2e-2, atol=2e-6)
