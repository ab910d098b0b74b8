"""Sanity check of built distributions: the wheel and the sdist carry the package, the CUDA sources and no
tests, scratch folders or reference code.

    python .github/scripts/check_dist.py dist
"""
import sys
import tarfile
import zipfile
from pathlib import Path

REQUIRED = ["flex_shard_b200/__init__.py", "flex_shard_b200/flex_shard.py", "flex_shard_b200/csrc/gemm_bf16.cu",
            "flex_shard_b200/csrc/common.cuh", "flex_shard_b200/placements/shard.py"]
FORBIDDEN = ["baseline/", "_work/", "gpurun_out/", "tests/"]


def names_of(path: Path) -> list[str]:
    if path.suffix == ".whl":
        with zipfile.ZipFile(path) as z:
            return z.namelist()
    with tarfile.open(path) as t:
        return ["/".join(n.split("/")[1:]) for n in t.getnames()]


def main(dist_dir: str) -> int:
    files = sorted(Path(dist_dir).glob("*"))
    wheels = [f for f in files if f.suffix == ".whl"]
    sdists = [f for f in files if f.name.endswith(".tar.gz")]
    if len(wheels) != 1 or len(sdists) != 1:
        print(f"expected one wheel and one sdist in {dist_dir}, found {[f.name for f in files]}")
        return 1
    bad = 0
    for f in wheels + sdists:
        names = names_of(f)
        for req in REQUIRED:
            if req not in names:
                print(f"{f.name}: missing {req}")
                bad += 1
        if f.suffix == ".whl":
            for n in names:
                if any(n.startswith(p) for p in FORBIDDEN):
                    print(f"{f.name}: must not ship {n}")
                    bad += 1
    print("ok" if not bad else f"{bad} problem(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "dist"))
