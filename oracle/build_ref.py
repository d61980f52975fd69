"""Builds the REFERENCE (Dobiasd/frugally-deep, header-only) into oracle/_ref/ when that is possible, and pins the CPU
restatement against it.

    python oracle/build_ref.py            # build if the dependencies are found, then compare on every golden fixture

The reference needs Eigen 3.4.0, FunctionalPlus 0.2.24 and nlohmann/json.  They are looked for, in this order, under
$FDEEP_REF_DEPS (a directory with include trees: Eigen/, fplus/, nlohmann/ somewhere below it), under baseline/_ref/,
and on the system include paths.  The reference's own sources are compiled where they lie ($FDEEP_REFERENCE, default
the include/ directory of a checkout named reference/ beside this repository); nothing of them is copied.  When a dependency or the reference is missing, build() returns
None and says why: there is then no oracle/_ref, the oracle stays "parity unpinned", and the CPU arm of the benchmark
is the restatement.  Test infrastructure only.
"""
from __future__ import annotations

import glob
import os
import struct
import subprocess
import sys
import sysconfig
import tempfile
from typing import List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT_DIR = os.path.join(HERE, "_ref")
EXE = os.path.join(OUT_DIR, "ref_driver")
REFERENCE_INCLUDE = os.environ.get("FDEEP_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference", "include"))


def _find_header(rel: str, roots: Sequence[str]) -> Optional[str]:
    """Directory to pass with -I so that `#include <rel>` resolves, searching a few levels below every root."""
    for root in roots:
        if not root or not os.path.isdir(root):
            continue
        for depth in range(0, 6):
            for cand in glob.glob(os.path.join(root, *(["*"] * depth), rel)):
                return cand[: -len(rel)].rstrip("/") or "/"
    return None


def find_dependencies():
    roots = [os.environ.get("FDEEP_REF_DEPS", ""), os.path.join(ROOT, "baseline", "_ref"), "/usr/include", "/usr/local/include",
             "/usr/include/eigen3", os.path.join(sysconfig.get_paths()["purelib"], "include", "cudnn_frontend", "thirdparty")]
    for p in sys.path:
        roots.append(os.path.join(p, "include", "cudnn_frontend", "thirdparty"))
    found = {"Eigen/Core": _find_header("Eigen/Core", roots), "fplus/fplus.hpp": _find_header("fplus/fplus.hpp", roots),
             "nlohmann/json.hpp": _find_header("nlohmann/json.hpp", roots)}
    return found


def build(verbose: bool = True) -> Optional[str]:
    """Compiles oracle/ref_driver.cpp against the reference's headers.  Returns the executable, or None (with the
    reason printed) when the reference or one of its dependencies is not available."""
    if not os.path.exists(os.path.join(REFERENCE_INCLUDE, "fdeep", "fdeep.hpp")):
        if verbose:
            print(f"oracle/_ref: not built: no reference tree at {REFERENCE_INCLUDE}")
        return EXE if os.path.exists(EXE) else None
    deps = find_dependencies()
    missing = [k for k, v in deps.items() if v is None]
    if missing:
        if verbose:
            print("oracle/_ref: not built: missing " + ", ".join(missing) + " (set FDEEP_REF_DEPS or put them under baseline/_ref/)")
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    src = os.path.join(HERE, "ref_driver.cpp")
    if os.path.exists(EXE) and os.path.getmtime(EXE) >= os.path.getmtime(src):
        return EXE
    cmd = ["g++", "-std=c++14", "-O3", "-march=x86-64-v3", "-DNDEBUG", "-pthread", "-I", REFERENCE_INCLUDE]
    for inc in sorted(set(deps.values())):
        cmd += ["-I", inc]
    cmd += [src, "-o", EXE]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if verbose:
            print("oracle/_ref: the reference did not compile:\n" + r.stderr[-2000:])
        return None
    return EXE


def write_samples(path: str, samples: Sequence[Sequence[np.ndarray]]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<qq", len(samples), len(samples[0]) if samples else 0))
        for s in samples:
            for a in s:
                a = np.ascontiguousarray(a, np.float32)
                f.write(struct.pack("<q", a.ndim))
                f.write(struct.pack("<%dq" % a.ndim, *a.shape))
                f.write(a.tobytes())


def read_samples(path: str) -> List[List[np.ndarray]]:
    with open(path, "rb") as f:
        data = f.read()
    off = 0

    def take(fmt):
        nonlocal off
        v = struct.unpack_from(fmt, data, off)
        off += struct.calcsize(fmt)
        return v

    n, per = take("<qq")
    out = []
    for _ in range(n):
        ts = []
        for _ in range(per):
            (rank,) = take("<q")
            dims = take("<%dq" % rank)
            vol = int(np.prod(dims))
            ts.append(np.frombuffer(data, np.float32, vol, off).reshape(dims).copy())
            off += 4 * vol
        out.append(ts)
    return out


def reference_predict(model_json_text: str, samples: Sequence[Sequence[np.ndarray]], exe: Optional[str] = None) -> List[List[np.ndarray]]:
    """fdeep::model::predict_multi of the reference itself on the given samples."""
    exe = exe or build(verbose=False)
    if exe is None:
        raise RuntimeError("the reference is not built (oracle/_ref is missing)")
    with tempfile.TemporaryDirectory() as tmp:
        mp, ip, op = os.path.join(tmp, "m.json"), os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
        with open(mp, "w") as f:
            f.write(model_json_text)
        write_samples(ip, samples)
        r = subprocess.run([exe, mp, ip, op], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference driver failed: " + r.stderr[-500:])
        return read_samples(op)


def compare_golden(exe: str) -> int:
    """The restatement against the reference on every fixture under tests/golden/: worst relative difference per file.
    Returns the number of fixtures whose difference exceeds 1e-4 (the tolerance of the parity tests)."""
    sys.path.insert(0, HERE)
    from oracle import OracleModel
    bad = 0
    for path in sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz"))):
        z = np.load(path, allow_pickle=False)
        text = bytes(z["model_json"]).decode()
        n_in, ns = int(z["n_in"]), int(z["n_samples"])
        samples = [[z[f"in_{s}_{i}"] for i in range(n_in)] for s in range(ns)]
        ref = reference_predict(text, samples, exe)
        mine = OracleModel(json_text=text).predict_multi(samples)
        worst = 0.0
        for a, b in zip(ref, mine):
            for x, y in zip(a, b):
                rms = float(np.sqrt(np.mean(np.square(x.astype(np.float64))))) if x.size else 0.0
                scale = np.maximum(np.abs(x), max(rms, 1e-30))
                worst = max(worst, float((np.abs(x.astype(np.float64) - y.astype(np.float64)) / scale).max()))
        print(f"{os.path.basename(path)}: restatement vs reference, worst relative difference {worst:.3e}")
        bad += worst > 1e-4
    return bad


if __name__ == "__main__":
    exe = build()
    if exe is None:
        print("parity stays unpinned: the restatement is checked against independent float64 computations only")
        sys.exit(0)
    sys.exit(1 if compare_golden(exe) else 0)
