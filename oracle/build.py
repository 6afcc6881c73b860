"""Build the CPU oracle (and, when the reference tree is present, the shim
around the reference's own sources).

TEST INFRASTRUCTURE ONLY -- see linear_ref.c.

    python oracle/build.py            # liboracle.so (+ _ref/ when possible)

Outputs:
    oracle/liboracle.so               gcc -O3 -fopenmp build of linear_ref.c
    oracle/_ref/libint4linear_ref.so  nvcc build of ref_wrapper.cu +
                                      <reference>/utils/packer.cpp +
                                      <reference>/kernels/linear_v21.cu
The second one is only (re)built where the reference checkout exists; the
prebuilt file is what travels to a GPU machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# The reference checkout: named by INT4LINEAR_REFERENCE_ROOT, else a directory called
# `reference` beside this repository.  Where neither exists only the prebuilt files are used.
REFERENCE_ROOT = os.environ.get("INT4LINEAR_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "linear_ref.c")
    out = os.path.join(HERE, "liboracle.so")
    if not force and _newer(out, [src]):
        return out
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-shared", "-fPIC",
           "-std=c11", "-o", out, src]
    subprocess.run(cmd, check=True)
    return out


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "utils", "packer.cpp"))


def build_ref(force: bool = False) -> str | None:
    """Compile the reference's own packer, CPU GEMM and v21 launcher into
    oracle/_ref/.  Returns the path, or None when neither the reference tree
    nor a prebuilt library is there."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libint4linear_ref.so")
    if not reference_available():
        return out if os.path.exists(out) else None
    srcs = [os.path.join(HERE, "ref_wrapper.cu"),
            os.path.join(REFERENCE_ROOT, "utils", "packer.cpp"),
            os.path.join(REFERENCE_ROOT, "kernels", "linear_v21.cu")]
    if not force and _newer(out, srcs):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(out_dir, exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-shared", "-Xcompiler", "-fPIC",
           "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", REFERENCE_ROOT, "-o", out] + srcs
    subprocess.run(cmd, check=True)
    return out


def build_dropin(force: bool = False) -> list[str]:
    """Drop-in check: the reference's OWN harness sources, unchanged and compiled where they
    lie, against this repository's replacement header and library.
        oracle/_ref/test_correctness_dropin   test/test_correctness.cu + utils/packer.cpp,
                                              linear_v21_launch resolved from the library
        oracle/_ref/benchmark_dropin          test/benchmark.cu + utils/packer.cpp, kernel
                                              template taken from the compat header
        oracle/_ref/test_correctness_dropin_libonly   test/test_correctness.cu alone: the
                                              packer comes from the library as well
    Only possible where the reference checkout exists; returns the files built."""
    if not reference_available():
        return []
    repo = os.path.dirname(HERE)
    pkg = os.path.join(repo, "int4linear_b200")
    lib = os.path.join(pkg, "libint4linear_b200.so")
    if not os.path.exists(lib):
        return []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    built = []
    common = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-I", os.path.join(pkg, "compat"), "-I", REFERENCE_ROOT]
    link = ["-L", pkg, "-lint4linear_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../int4linear_b200"]
    packer = os.path.join(REFERENCE_ROOT, "utils", "packer.cpp")
    for name, src in [("test_correctness_dropin", "test/test_correctness.cu"),
                      ("benchmark_dropin", "test/benchmark.cu")]:
        out = os.path.join(out_dir, name)
        srcs = [os.path.join(REFERENCE_ROOT, src), packer]
        deps = srcs + [lib, os.path.join(pkg, "compat", "kernels", "linear_v21.h")]
        if force or not _newer(out, deps):
            subprocess.run(common + srcs + link + ["-o", out], check=True)
        built.append(out)
    # The same correctness program linked against the library alone: pack / unpack come from the
    # library too (compat/utils/packer.h), no source file of the reference besides the program.
    out = os.path.join(out_dir, "test_correctness_dropin_libonly")
    srcs = [os.path.join(REFERENCE_ROOT, "test/test_correctness.cu")]
    deps = srcs + [lib, os.path.join(pkg, "compat", "kernels", "linear_v21.h"), os.path.join(pkg, "compat", "utils", "packer.h")]
    if force or not _newer(out, deps):
        subprocess.run(common + srcs + link + ["-o", out], check=True)
    built.append(out)
    return built


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_dropin(force))
