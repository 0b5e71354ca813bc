"""Builds libaxiom_b200.so in-tree with nvcc for sm_100a.

Usage: python axiom-kernel_b200/build.py [--force] [--verbose]

Every translation unit under csrc/ is compiled with
  -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17
and WITHOUT --use_fast_math, except the units listed in FAST_MATH_UNITS, which
mirror the reference's generic backend that is built with it
(reference Makefile:17 vs :71-73).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
INCLUDE = HERE.parent / "include"
LIB = HERE / "libaxiom_b200.so"
FAST_MATH_UNITS = {"generic_f32_fast.cu"}


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: libaxiom_b200.so cannot be built")
    return found


def _flags(unit: str, verbose: bool) -> list[str]:
    flags = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", f"-I{INCLUDE}", f"-I{CSRC}",
    ]
    if unit in FAST_MATH_UNITS:
        flags.append("--use_fast_math")
    if verbose:
        flags += ["-Xptxas", "-v"]
    return flags


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = nvcc_path()
    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hpp")) + sorted(INCLUDE.glob("*.h"))
    units = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in units:
        obj = OBJ / (src.stem + ".o")
        if force or verbose or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *_flags(src.name, verbose), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for src, res in pool.map(compile_one, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(f"== {src.name}\n{res.stdout}{res.stderr}")
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ / (s.stem + ".o") for s in units]
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libaxiom_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
