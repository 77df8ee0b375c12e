"""Compile the sm_100a CUDA sources into nvfp4_training/_lib/libnvfp4_b200.so (C ABI, no torch headers).

    python build.py [--force] [--verbose]

A source file may name extra compiler flags on its first line (`// nvcc-flags: --fmad=false`).
nvcc cross-compiles without a GPU; the shared object is loaded with ctypes by nvfp4_training._native.
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
CSRC = HERE / "csrc"
OUT_DIR = HERE / "nvfp4_training" / "_lib"
TARGET = OUT_DIR / "libnvfp4_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = HERE / "build"
    obj_dir.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    nvcc = _nvcc()
    jobs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            first = src.read_text().splitlines()[0]
            extra = first.split("nvcc-flags:", 1)[1].split() if "nvcc-flags:" in first else []
            cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        if verbose:
            sys.stderr.write(res.stderr)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    objs = [obj_dir / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(TARGET, objs):
        cmd = [nvcc, *ARCH, "--shared", "-o", str(TARGET), *map(str, objs)]
        run(cmd)
    return TARGET


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
