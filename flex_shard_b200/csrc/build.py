"""Builds the native library of flex_shard_b200 for sm_100a.

Every ``*.cu`` file beside this script is compiled with nvcc into an object
file and the objects are linked into ``flex_shard_b200/lib/libfsb200.so``.
The kernels expose a plain C ABI (pointers, sizes, a ``cudaStream_t``), so the
build needs neither the PyTorch headers nor pybind11 and takes seconds.

Run ``python -m flex_shard_b200.csrc.build`` (add ``-v`` for ptxas resource
usage, ``-f`` to force a rebuild).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_DIR = CSRC.parent / "lib"
OBJ_DIR = CSRC / "build"
LIB_PATH = LIB_DIR / "libfsb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    srcs = sources()
    jobs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, p in ex.map(run, jobs):
                if verbose or p.returncode != 0:
                    sys.stderr.write(f"--- {src.name}\n{p.stdout}{p.stderr}\n")
                if p.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ_DIR / (s.stem + ".o") for s in srcs]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="-f" in sys.argv, verbose="-v" in sys.argv)
    print(path)
