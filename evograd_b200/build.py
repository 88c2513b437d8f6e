"""Builds ``libevg_b200.so`` in-tree from ``csrc/*.cu`` with nvcc for sm_100a.

The shared library is the product's only compute path; nothing here falls back
to another backend. nvcc cross-compiles without a GPU, so the build also runs on
hosts that only have the CUDA toolkit.

    python -m evograd_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
INCLUDE = REPO_DIR / "include"
OBJ_DIR = REPO_DIR / "build" / "obj"
LIB_PATH = PKG_DIR / "libevg_b200.so"

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    f"-I{INCLUDE}",
    f"-I{CSRC}",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the evg_b200 kernels cannot be built")
    return found


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    (obj.with_suffix(".log")).write_text(log)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{log[-4000:]}")
    if verbose:
        print(f"[evg build] {src.name} ok")
    return log


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source and link the shared library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = _headers()
    jobs = []
    for src in _sources():
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    objs = [OBJ_DIR / (s.stem + ".o") for s in _sources()]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}{proc.stderr}")
        if verbose:
            print(f"[evg build] linked {LIB_PATH}")
    return LIB_PATH


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    path = build(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
