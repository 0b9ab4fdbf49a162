"""Build recipe for the CUDA library: nvcc, sm_100a only, one object per family, in-tree output.

``python -m better_benchmark_b200.build`` (or ``build_library()``) compiles every ``csrc/*.cu``
file to an object in ``csrc/_build/`` in parallel and links ``csrc/libb200_oracles.so``.
Objects are rebuilt only when their source (or a shared header) is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
BUILD_DIR = CSRC / "_build"
LIB_PATH = CSRC / "libb200_oracles.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # a*b+c stays two rounded operations, as in the decomposed aten graphs; no fast-math anywhere
    "-fmad=false",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH")


def _stale(obj: Path, src: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(dep.stat().st_mtime > t for dep in [src, *headers, Path(__file__)])


def build_library(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh"))
    jobs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        if force or _stale(obj, src, headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, res in pool.map(compile_one, jobs):
            if verbose and res.stderr:
                print(res.stderr, file=sys.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")

    objs = [BUILD_DIR / (s.stem + ".o") for s in sources]
    if force or jobs or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
