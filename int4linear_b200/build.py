"""Compile the CUDA sources of this package into libint4linear_b200.so (in-tree).

    python -m int4linear_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU, so this runs anywhere the CUDA
toolkit is installed.  The shared library links the CUDA runtime statically
and resolves the one driver entry point it needs at run time, so it loads on a
machine without a driver too (its compute entry points then report
INT4L_ERR_NO_DEVICE).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libint4linear_b200.so")
SOURCES = ["api.cu", "gemm_tcgen05.cu", "gemm_tcgen05_s8.cu", "gemm_skinny.cu", "gemm_legacy.cu", "packer.cu", "probe.cu", "gemm_fewrows.cu", "no_alloc.cu"]


def _deps() -> list[str]:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "int4linear_b200.h"))
    return deps


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force: bool = False, verbose: bool = False, out: str | None = None,
          extra_flags: list[str] | None = None) -> str:
    """Build the library.  `out` / `extra_flags` produce a variant next to the regular one
    without replacing it."""
    if out is None and not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libint4linear_b200.so")
    cmd = [nvcc, "-std=c++17", "-O3", "-shared", "-Xcompiler", "-fPIC",
           "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-cudart", "static", "-o", out or LIB] + list(extra_flags or [])
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.run(cmd, check=True)
    return out or LIB


def build_compat_check() -> str:
    """Compile tests/compat_check.cu against the drop-in header and the library."""
    root = os.path.dirname(PKG)
    src = os.path.join(root, "tests", "compat_check.cu")
    out = os.path.join(root, "tests", "compat_check.bin")
    hdr = os.path.join(PKG, "compat", "kernels", "linear_v21.h")
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(build())):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", os.path.join(PKG, "compat"), src, "-L", PKG, "-lint4linear_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../int4linear_b200", "-o", out]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
