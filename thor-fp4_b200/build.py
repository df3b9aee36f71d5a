"""Build libthorfp4_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

usage: python thor-fp4_b200/build.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "build"
LIB = OUT_DIR / "libthorfp4_b200.so"
SOURCES = ["quant.cu", "misc.cu", "gemm.cu", "peer.cu", "api.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def nvcc() -> str:
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES if (CSRC / s).exists()] + list(CSRC.glob("*.cuh")) + \
        [ROOT.parent / "include" / "thorfp4_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    objs = []
    procs = []
    for s in SOURCES:
        src = CSRC / s
        if not src.exists():
            continue
        obj = OUT_DIR / (s[:-3] + ".o")
        cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((s, subprocess.Popen(cmd)))
        objs.append(str(obj))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    subprocess.run([nvcc(), "-shared", "-o", str(LIB), *objs, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
