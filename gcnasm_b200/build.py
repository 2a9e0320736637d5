"""Builds the native parts in-tree: ``libb200gemm.so`` (CUDA, sm_100a only) and the C++ host drivers.

nvcc cross-compiles without a GPU, so this runs on any machine that has the CUDA toolkit.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
DRIVERS = os.path.join(PKG, "drivers")
LIB = os.path.join(PKG, "libb200gemm.so")
BIN = os.path.join(PKG, "bin")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fopenmp,-fno-fast-math",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libb200gemm.so")


def _host_cxx() -> str:
    # a g++ with OpenMP; an environment-provided cross compiler may lack libgomp
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("g++ not found")


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))] + [os.path.join(ROOT, "include", "b200gemm.h")]
    if force or _newer(LIB, srcs):
        cmd = [_nvcc(), *NVCC_FLAGS, "-ccbin", _host_cxx(), "-shared", "-o", LIB, os.path.join(CSRC, "b200gemm.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.check_call(cmd)
    return LIB


def build_drivers(force: bool = False) -> list:
    """The C++ host drivers mirroring the reference's main() programs (three GEMM drivers and the bandwidth probe)."""
    os.makedirs(BIN, exist_ok=True)
    out = []
    if not os.path.isdir(DRIVERS):
        return out
    for name in sorted(os.listdir(DRIVERS)):
        if not name.endswith(".cc"):
            continue
        src = os.path.join(DRIVERS, name)
        exe = os.path.join(BIN, name[:-3])
        deps = [src, LIB] + [os.path.join(DRIVERS, h) for h in os.listdir(DRIVERS) if h.endswith(".h")]
        if force or _newer(exe, deps):
            subprocess.check_call([
                _nvcc(), "-O3", "-std=c++17", "-Wno-deprecated-gpu-targets", "-ccbin", _host_cxx(), "-Xcompiler", "-fopenmp,-fno-fast-math",
                "-I", os.path.join(ROOT, "include"), "-o", exe, src,
                "-L", PKG, "-lb200gemm", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..",
            ])
        out.append(exe)
    return out


def build_all(force: bool = False, verbose: bool = False):
    lib = build_library(force, verbose)
    exes = build_drivers(force)
    return lib, exes


if __name__ == "__main__":
    lib, exes = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(lib)
    for e in exes:
        print(e)
