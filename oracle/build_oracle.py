"""Builds the CPU oracle (oracle/fdeep_oracle.cpp) into oracle/_build/libfdeep_oracle.so.

Test infrastructure only.  Built for x86-64-v3 (AVX2+FMA) rather than -march=native so that a library
built on one machine also runs on another.  The oracle parses model files with nlohmann/json, the JSON library the
reference itself uses; the copy bundled with the cudnn-frontend Python package is used.

The reference's own headers cannot be compiled here: they include Eigen 3.4.0 and FunctionalPlus
0.2.24, neither of which is available, so there is no oracle/_ref build.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libfdeep_oracle.so")
LIB_F64 = os.path.join(OUT_DIR, "libfdeep_oracle_f64.so")


def _json_include() -> str:
    cands = [os.path.join(sysconfig.get_paths()["purelib"], "include", "cudnn_frontend", "thirdparty")]
    for p in sys.path:
        cands.append(os.path.join(p, "include", "cudnn_frontend", "thirdparty"))
    for c in cands:
        if os.path.exists(os.path.join(c, "nlohmann", "json.hpp")):
            return c
    raise RuntimeError("nlohmann/json.hpp not found (expected in the cudnn_frontend package)")


def build(force: bool = False, double: bool = False) -> str:
    """double=True: the double-precision arbiter build (-DFDEEP_ORACLE_DOUBLE) next to the fp32 one."""
    src = os.path.join(HERE, "fdeep_oracle.cpp")
    lib = LIB_F64 if double else LIB
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= os.path.getmtime(src):
        return lib
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-DNDEBUG", "-fPIC", "-shared", "-pthread",
           "-I", _json_include(), src, "-o", lib]
    if double:
        cmd.insert(1, "-DFDEEP_ORACLE_DOUBLE")
    subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    print(build(force="--force" in sys.argv, double=True))
