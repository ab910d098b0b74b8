"""The smallest example end to end on 4 gloo ranks: dense buckets on the data-parallel mesh, expert buckets on an
"efsdp" sub-mesh of two ranks, with ``--check`` asserting one gather per pass and one reduction per bucket per step
and an idle runtime between steps (the role of the reference example's ``--trace`` check,
``examples/train_adamw.py:52-81``)."""
import os
import subprocess
import sys

from tests.common import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, steps=3):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "examples", "train_adamw.py"),
           "--steps", str(steps), "--check"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    losses = [float(l.split()[-1]) for l in p.stdout.splitlines() if l.startswith("step ")]
    assert "check ok" in p.stdout
    return losses


def test_tiny_example_with_expert_sub_mesh_passes_its_collective_check():
    losses = _run(4)
    assert len(losses) == 3 and all(l == l and 0 < l < 20 for l in losses)   # finite, plausible next-token losses


def test_tiny_example_on_two_ranks_uses_one_mesh():
    assert len(_run(2, steps=2)) == 2
