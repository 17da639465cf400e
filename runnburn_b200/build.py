"""Builds librnb_b200.so (the CUDA operator library) in-tree with nvcc for sm_100a.

    python -m runnburn_b200.build [--force] [--verbose]
    python -m runnburn_b200.build --static      # librnb_b200.a for a Rust / C link line
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "librnb_b200.so"
STATIC_LIB = PKG / "librnb_b200.a"
SOURCES = ["api.cu", "noalloc.cu", "gguf.cu", "expert_cache.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function",
    "--expt-relaxed-constexpr", "-cudart", "shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG.parent / "include" / "rnb_b200.h", Path(__file__)]
    return any(p.stat().st_mtime > t for p in deps if p.is_file())


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    extra = os.environ.get("RNB_B200_NVCC_FLAGS", "").split()   # development hook, e.g. -DGM_PROFILE
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-shared", "-o", str(LIB), *srcs, "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building librnb_b200.so")
    return LIB


def build_static_library(verbose: bool = False) -> Path:
    """`nvcc -lib`: the same sources as one static archive, the form the reference's build.rs links
    (crates/rnb-backend/cuda/build.rs:62-84 shells out to nvcc and hands rustc a static library).
    Link it with the CUDA runtime, libdl and the C++ runtime:
    `-L<dir> -lrnb_b200 -L/usr/local/cuda/lib64 -lcudart -ldl -lstdc++`."""
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    extra = os.environ.get("RNB_B200_NVCC_FLAGS", "").split()
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-lib", "-o", str(STATIC_LIB), *srcs]
    if verbose:
        print(" ".join(cmd))
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building librnb_b200.a")
    return STATIC_LIB


if __name__ == "__main__":
    if "--static" in sys.argv:
        print(build_static_library(verbose="--verbose" in sys.argv))
    else:
        build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
        print(LIB)
