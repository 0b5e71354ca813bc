"""Builds oracle/_ref/libaxiom_ref.so: the reference's OWN kernels for the hot path, compiled for
sm_100a from the sources where they lie under the reference tree (never copied), behind small
launchers (oracle/ref/*.cu).  Test infrastructure only.

    python oracle/build_ref.py [/path/to/reference]     (default: $AXIOM_REFERENCE_DIR, else ../reference)

Each reference unit is built with the flags the reference's Makefile uses for it: the qwen38 and
precise units WITHOUT fast-math, the generic backend WITH --use_fast_math.  The reference's own
build system is not run.  Symbols the included files reference but that live in other reference
units (checkpoint readers, layer objects) are resolved by generated stubs that return
"not implemented": the launchers never reach them.
"""
from __future__ import annotations

import concurrent.futures
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NVCC = "/usr/local/cuda/bin/nvcc"

UNITS = [  # (source relative to oracle/ or to the reference root, fast_math, from_reference_tree)
    ("ref/ref_nvfp4_mlp.cu", False, False),
    ("ref/ref_fp8.cu", False, False),
    ("ref/ref_mtp.cu", False, False),
    ("ref/ref_model.cu", False, False),
    ("ref/ref_attention.cu", False, False),
    ("ref/ref_generic_fast.cu", True, False),
    ("ref/ref_bench.cu", False, False),
    ("ref/ref_dspark.cu", False, False),
    ("src/axiom_qwen38_nvfp4.cu", False, True),
    ("src/axiom_cuda_precise.cu", False, True),
]


def build(ref_root: Path) -> Path:
    OUT.mkdir(exist_ok=True)
    base = [NVCC, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
            f"-I{ref_root / 'include'}", f"-I{ref_root / 'third_party/flashinfer/include'}", f"-I{ref_root}",
            f"-I{ref_root / 'src'}", "-DAXIOM_BUILD_TARGET=\"sm_100a\"", "-w"]

    def compile_one(unit):
        rel, fast, in_ref = unit
        src = (ref_root if in_ref else HERE) / rel
        obj = OUT / (Path(rel).stem + ".o")
        cmd = base + (["--use_fast_math"] if fast else []) + ["-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{rel}:\n{res.stdout}{res.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, UNITS))

    defined, undefined = set(), set()
    for obj in objs:
        for line in subprocess.run(["nm", str(obj)], capture_output=True, text=True, check=True).stdout.splitlines():
            parts = line.split()
            if len(parts) == 2 and parts[0] == "U":
                undefined.add(parts[1])
            elif len(parts) == 3 and parts[1] in "TDBWV":
                defined.add(parts[2])
    missing = sorted(s for s in undefined - defined if s.startswith("axiom_"))
    stubs = OUT / "stubs.c"
    stubs.write_text("/* generated: symbols of other reference units, never reached by the launchers */\n" +
                     "".join(f"int {name}(void) {{ return 5; }}\n" for name in missing))
    stub_obj = OUT / "stubs.o"
    subprocess.run(["/usr/bin/gcc", "-fPIC", "-c", str(stubs), "-o", str(stub_obj)], check=True)
    lib = OUT / "libaxiom_ref.so"
    cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs), str(stub_obj),
           "-lcublasLt", "-lcublas"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(res.stdout + res.stderr)
    return lib


if __name__ == "__main__":
    import os

    # the reference tree: argument, else AXIOM_REFERENCE_DIR, else a checkout named "reference" beside this repository
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(os.environ.get("AXIOM_REFERENCE_DIR") or HERE.parent.parent / "reference")
    print(build(root))
