"""Newton-Schulz on the tcgen05 GEMM and the Muon elementwise kernels against the CPU path."""
import pytest
import torch

from flex_shard_b200 import ops
from flex_shard_b200.ops import newton_schulz as ns

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(256, 1024), (1024, 256), (512, 512)])
def test_newton_schulz_matches_cpu_reference(shape):
    torch.manual_seed(0)
    g = torch.randn(*shape)
    ref = ns.newton_schulz_kernel_reference(g).float()
    out = ns.newton_schulz(g.cuda()).float().cpu()
    ops.check_status()
    # bf16 rounding differs between the two GEMM implementations and is amplified along the
    # small singular directions of a square matrix, so compare in a relative Frobenius sense
    assert (out - ref).norm() / ref.norm() < 3e-2
    sv = torch.linalg.svdvals(out)
    assert sv.max() < 1.3
    if shape[0] != shape[1]:
        assert 0.5 < sv.min()


def test_muon_direction_and_apply_match_cpu():
    torch.manual_seed(1)
    g = torch.randn(384, 640)
    m_cpu = 0.1 * torch.randn(384, 640)
    m_gpu = m_cpu.clone().cuda()
    x_cpu = ns.muon_direction_(m_cpu, g, 0.95, True, 5)
    x_gpu = ns.muon_direction_(m_gpu, g.cuda(), 0.95, True, 5)
    torch.testing.assert_close(m_gpu.cpu(), m_cpu, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(x_gpu.float().cpu(), x_cpu.float(), rtol=0, atol=4e-2)
    for dt in (torch.float32, torch.bfloat16):
        p = torch.randn(384, 640).to(dt)
        pg = p.clone().cuda()
        ns.muon_apply_(p, x_cpu, 0.02, 0.1, 1.5)
        ns.muon_apply_(pg, x_cpu.cuda(), 0.02, 0.1, 1.5)
        torch.testing.assert_close(pg.float().cpu(), p.float(), rtol=1e-2, atol=1e-2)
    ops.check_status()


def test_prepare_sum_is_reproducible_and_vector_paths_match_scalar():
    """The sum of squares is formed from per-block partials in index order: identical bits on every run.
    An odd length and a misaligned view go through the scalar loop and must agree with the vector path."""
    torch.manual_seed(3)
    dev = torch.device("cuda")
    for n, off in ((4096 * 3000, 0), (1234567, 0), (4096 * 64, 1)):
        g = torch.randn(n + off, device=dev)[off:].view(1, -1)
        m0 = 0.1 * torch.randn(n + off, device=dev)[off:].view(1, -1)
        outs = []
        for _ in range(3):
            m = torch.empty(n + off, device=dev)[off:].view(1, -1)
            m.copy_(m0)
            u = ns.muon_momentum_direction_(m, g, 0.95, True)
            outs.append((m.clone(), u.clone()))
        m_ref = torch.lerp(m0, g, 0.05)
        u_ref = torch.lerp(g, m_ref, 0.95).bfloat16()
        for m, u in outs:
            torch.testing.assert_close(m, m_ref, rtol=1e-6, atol=1e-7)
            assert (u.float() - u_ref.float()).abs().max() <= 2 ** -7 * u_ref.float().abs().max()
            assert torch.equal(u, outs[0][1]) and torch.equal(m, outs[0][0])
    g = torch.randn(2048, 3000, device=dev)
    xs = []
    for _ in range(3):
        m = torch.zeros_like(g)
        xs.append(ns.muon_direction_(m, g, 0.95, True, 0))      # zero iterations: the normalised matrix itself
    assert torch.equal(xs[0], xs[1]) and torch.equal(xs[0], xs[2])
    ref = torch.lerp(g, 0.05 * g, 0.95).bfloat16().float()
    torch.testing.assert_close(xs[0].float(), ref / ref.norm(), rtol=2e-2, atol=1e-6)
    ops.check_status()


@pytest.mark.parametrize("shape", [(6, 256, 512), (4, 512, 256), (3, 384, 384)])
def test_batched_newton_schulz_matches_one_matrix_at_a_time(shape):
    """A stack of equal matrices runs each product of an iteration as one grouped launch; every matrix must
    come out as if it had been orthogonalised alone."""
    torch.manual_seed(4)
    g = torch.randn(*shape, device="cuda")
    assert ns.batched_ns_supported(g)
    before = ops.launch_count()
    out = ns.newton_schulz(g)
    assert ops.launch_count() - before == 15                       # 3 launches per iteration for the whole stack
    for i in range(shape[0]):
        one = ns.newton_schulz(g[i])
        assert (out[i].float() - one.float()).norm() / one.float().norm() < 1e-2
        ref = ns.newton_schulz_kernel_reference(g[i]).float()
        assert (out[i].float().cpu() - ref).norm() / ref.norm() < 3e-2
    ops.check_status()


def test_dist_muon_steps_a_stack_of_equal_matrices_in_one_go():
    """A 3-D parameter (experts) takes the batched path: same update, up to the arithmetic of the iteration, as the
    same matrices held as separate 2-D parameters; far fewer launches."""
    import torch.nn as nn

    from flex_shard_b200.dist_muon import DistMuon

    torch.manual_seed(6)
    E, r, c = 6, 256, 384
    w = torch.randn(E, r, c, device="cuda")
    stacked = nn.Parameter(w.clone())
    singles = [nn.Parameter(w[i].clone()) for i in range(E)]
    opt_a = DistMuon([stacked], param_names=["experts"], lr=0.02)
    opt_b = DistMuon(singles, param_names=[f"e{i}" for i in range(E)], lr=0.02)
    launches = []
    for step in range(2):
        g = torch.randn(E, r, c, device="cuda")
        stacked.grad = g.clone()
        for i, p in enumerate(singles):
            p.grad = g[i].clone()
        for opt in (opt_a, opt_b):
            before = ops.launch_count()
            opt.step()
            launches.append(ops.launch_count() - before)
    for i, p in enumerate(singles):
        torch.testing.assert_close(stacked.detach()[i], p.detach(), rtol=0, atol=2e-3)
    assert launches[0] * 3 < launches[1]            # 1 + 15 + 1 launches (plus normalisation) against 6 x 18
    ops.check_status()
