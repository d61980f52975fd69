"""Builds libfdeep_b200.so (C-ABI shared library: loader, plan compiler, executor, sm_100a kernels).

    python frugally-deep_b200/build.py [--force]

CUDA sources are compiled for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`); nvcc
cross-compiles without a GPU.  Objects are cached under csrc/_obj and rebuilt when a source or any
header is newer.  The library is written next to this file so that it is found in-tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libfdeep_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = ["kernels.cu", "gemm_tc.cu", "gemm_rows.cu", "gemm_static.cu", "dwconv_tma.cu"]
CPP_SOURCES = ["model.cpp", "plan.cpp", "engine.cpp", "session.cpp", "capi.cpp"]

NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-I", os.path.join(CUDA_HOME, "include")]


def _headers_mtime() -> float:
    m = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for dp, _, fns in os.walk(root):
            if "_obj" in dp:
                continue
            for fn in fns:
                if fn.endswith((".hpp", ".cuh", ".h")):
                    m = max(m, os.path.getmtime(os.path.join(dp, fn)))
    return m


def _compile(src: str, force: bool, hdr_m: float) -> str:
    obj = os.path.join(OBJ, src + ".o")
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_m):
        return obj
    if src.endswith(".cu"):
        cmd = [NVCC] + NVCC_FLAGS + ["-c", path, "-o", obj]
    else:
        cmd = ["g++"] + CXX_FLAGS + ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return obj


def build(force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_m = _headers_mtime()
    srcs = CU_SOURCES + CPP_SOURCES
    with ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, hdr_m), srcs))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
