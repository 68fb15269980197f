"""Builds ``libtcfp_b200.so`` (sm_100a only) next to this file with nvcc.

Usage: ``python -m tcfp_b200.build [--force] [--verbose]``.  The library is a
plain C-ABI shared object (see ``include/tcfp_b200.h``); no torch headers are
involved, so the build takes a few seconds per translation unit and works on a
machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libtcfp_b200.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# quantize.cu decides rounding byte-for-byte: never let ptxas contract a*b+c
UNITS = [
    ("quantize.cu", ["--fmad=false"]),
    ("retarget.cu", ["--fmad=false"]),
    ("gemm_sm100.cu", []),
    ("gemm2_sm100.cu", []),
    ("noalloc.cu", []),
    ("api.cu", []),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or CUDA_HOME")


def _sources() -> list[Path]:
    return [p for p in CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".h")] + [
        HERE.parent / "include" / "tcfp_b200.h"
    ]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    for name, extra in UNITS:
        obj = objdir / (name + ".o")
        cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    # link under a temporary name and rename: a reader never sees a half-written library
    tmp = LIB.with_name(LIB.name + ".tmp")
    cmd = [nvcc, *ARCH, "-shared", "-o", str(tmp), *objs, "-cudart", "static"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    tmp.replace(LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
