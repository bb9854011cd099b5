"""Build libq3b200.so from the .cu files next to this script with nvcc for sm_100a.

Usage: python build.py [--force] [--verbose]
The shared library is written beside the sources (in-tree) so that it ships with a snapshot of
the repository; object files go to csrc/build/. Only files whose sources (or shared headers)
changed are recompiled.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libq3b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
          "-Xcompiler", "-Wno-unused-function"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the q3b200 library cannot be built")
    return exe


def headers() -> list[Path]:
    return sorted(HERE.glob("*.cuh")) + [HERE.parent.parent / "include" / "q3b200.h"]


def stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(HERE.glob("*.cu"))
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    hdrs = headers()
    jobs = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        if force or stale(obj, [src, *hdrs]):
            cmd = [nvcc(), *ARCH, *COMMON, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for src, res in pool.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(f"--- {src.name}\n{res.stdout}{res.stderr}\n")
            failed |= res.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    objs = [objdir / (s.stem + ".o") for s in sources]
    if force or jobs or stale(LIB, objs):
        # One CUDA runtime per process: link libcudart dynamically so that, inside a PyTorch process, this
        # library shares torch's runtime instance (same per-thread current device and context).
        cmd = [nvcc(), *ARCH, "-shared", "-cudart", "shared", "-Xlinker", "-rpath=/usr/local/cuda/lib64",
               "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
