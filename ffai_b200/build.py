"""Build ``libffai_cuda.so`` in-tree with nvcc for sm_100a.

``python -m ffai_b200.build`` compiles ``csrc/ffai_cuda.cu`` (which includes the
kernel headers) into ``ffai_b200/lib/libffai_cuda.so``.  nvcc cross-compiles
without a GPU.  The CUDA runtime is linked statically, so the shared object
depends only on the driver at run time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
SRC = PKG / "csrc"
OUT = PKG / "lib" / "libffai_cuda.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-shared",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise FileNotFoundError("nvcc not found")


def sources():
    return sorted(SRC.glob("*.cu"))


def stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(SRC.glob("*.cu")) + list(SRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    if not force and not stale():
        return OUT
    OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc_path(), *NVCC_FLAGS, *extra_flags, "-ccbin", shutil.which("g++") or "g++",
           "-I", str(INCLUDE), "-o", str(OUT), *map(str, sources())]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libffai_cuda.so")
    return OUT


if __name__ == "__main__":
    flags = ["-Xptxas", "-v"] if "--ptxas-v" in sys.argv else []
    print(build(force=True, verbose=True, extra_flags=flags))
