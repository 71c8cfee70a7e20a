"""Builds libnf4b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m hackaton_b200.build            # build if sources are newer than the library
    python -m hackaton_b200.build --force

nvcc cross-compiles without a GPU, so this also serves as the "does it build" check.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libnf4b200.so"
SOURCES = ["capi.cu", "cross_entropy.cu", "dequant.cu", "gemm.cu", "gemv.cu", "lora.cu", "rmsnorm.cu", "rope.cu", "selftest.cu", "static_scratch.cu", "swiglu.cu"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "--use_fast_math=false",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def _stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(PKG.parent / "include" / "nf4b200.h")
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    flags += os.environ.get("NF4B200_NVCC_FLAGS", "").split()   # e.g. -DNF4B200_TRACE for tuning
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs = []
    build_dir = PKG / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = build_dir / (src + ".o")
        cmd = [_nvcc(), *flags, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
        objs.append(str(obj))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    tmp = LIB.with_suffix(".so.tmp")
    link = [_nvcc(), "-shared", "-o", str(tmp), *objs, "-lcudart"]
    subprocess.run(link, check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
