"""Builds libxabe_moe_sm100.so (the C-ABI kernel library) in-tree with nvcc for sm_100a, and
libxabe_gguf.so (the GGUF container reader, host code) with g++."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libxabe_moe_sm100.so")
SOURCES = ["xabe_moe_api.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh")) + [
    os.path.join("..", "..", "include", "xabe_moe.h")]


GGUF_LIB = os.path.join(PKG, "libxabe_gguf.so")
GGUF_DEPS = [os.path.join(CSRC, "xabe_gguf.cpp"), os.path.join(PKG, "..", "include", "xabe_gguf.h")]


def build_gguf(force: bool = False) -> str:
    """The GGUF reader: plain C++17, no CUDA."""
    if not force and os.path.exists(GGUF_LIB) and all(
            os.path.getmtime(d) <= os.path.getmtime(GGUF_LIB) for d in GGUF_DEPS):
        return GGUF_LIB
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-o", GGUF_LIB, GGUF_DEPS[0]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
    return GGUF_LIB


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def _host_compiler() -> list[str]:
    # the distribution g++ is the one nvcc 12.9 is validated against on this image
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *_host_compiler(), "-std=c++17", "-O3", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v" if verbose else "-warn-spills",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose="-v" in sys.argv)
    print(LIB)
    print(build_gguf(force=True))
