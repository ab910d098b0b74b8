"""The package builds into a wheel that carries the Python package and the CUDA sources and nothing else
of the repository (restating the reference's wheel sanity check, ``.github/scripts/check_dist.py``)."""
import importlib.util
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_wheel_contents(tmp_path):
    src = tmp_path / "src"
    # build from a copy so that no build folder appears in the working tree
    subprocess.run(["git", "-C", ROOT, "checkout-index", "-a", f"--prefix={src}/"], check=True)
    for extra in ("pyproject.toml",):       # also cover a not-yet-committed packaging file
        if not (src / extra).exists():
            (src / extra).write_bytes(open(os.path.join(ROOT, extra), "rb").read())
    out = tmp_path / "dist"
    p = subprocess.run([sys.executable, "-m", "pip", "wheel", str(src), "--no-deps", "--no-build-isolation", "-w",
                        str(out), "-q"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    spec = importlib.util.spec_from_file_location("check_dist", os.path.join(ROOT, ".github", "scripts", "check_dist.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    wheels = list(out.glob("*.whl"))
    assert len(wheels) == 1
    names = mod.names_of(wheels[0])
    for req in mod.REQUIRED:
        assert req in names, req
    assert not [n for n in names if any(n.startswith(f) for f in mod.FORBIDDEN)]
