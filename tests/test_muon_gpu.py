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
    ref = ns.newton_schulz(g).float()
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
