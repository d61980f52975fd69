"""ctypes binding of the CPU oracle (oracle/fdeep_oracle.cpp).  Test infrastructure only: imported by
tests/, the smoke run and the bench's CPU-baseline leg, never by the shipped package."""
from __future__ import annotations

import ctypes as C
import os
import sys
from typing import List, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _HERE)
import build_oracle  # noqa: E402

_libs = {}


def lib(double: bool = False):
    """The fp32 oracle, or (double=True) its double-precision arbiter build; arrays cross the interface in that type."""
    if double not in _libs:
        path = build_oracle.build(double=double)
        L = C.CDLL(path)
        L.fdo_last_error.restype = C.c_char_p
        L.fdo_load.restype = C.c_void_p
        L.fdo_load.argtypes = [C.c_char_p]
        L.fdo_load_string.restype = C.c_void_p
        L.fdo_load_string.argtypes = [C.c_char_p, C.c_size_t]
        L.fdo_free.argtypes = [C.c_void_p]
        for f in ("fdo_num_inputs", "fdo_num_outputs", "fdo_num_tests"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.fdo_predict.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.POINTER(C.c_int)]
        L.fdo_out_shape.argtypes = [C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int)]
        L.fdo_out_copy.argtypes = [C.c_int, C.c_void_p]
        L.fdo_predict_multi.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p), C.c_int]
        L.fdo_run_tests.argtypes = [C.c_void_p, C.c_double if double else C.c_float]
        _libs[double] = L
    return _libs[double]


def _dims5(shape: Sequence[int]) -> List[int]:
    return [1] * (5 - len(shape)) + [int(s) for s in shape]


class OracleModel:
    """One loaded model.  ``predict`` takes one sample (list of arrays without batch dim)."""

    def __init__(self, path: str = None, json_text: str = None, double: bool = False):
        self.double = double
        self.dtype = np.float64 if double else np.float32
        L = lib(double)
        if path is not None:
            self.h = L.fdo_load(path.encode())
        else:
            b = json_text.encode()
            self.h = L.fdo_load_string(b, len(b))
        if not self.h:
            raise RuntimeError(L.fdo_last_error().decode())
        self.n_in = L.fdo_num_inputs(self.h)
        self.n_out = L.fdo_num_outputs(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            lib(self.double).fdo_free(self.h)
            self.h = None

    def predict(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        L = lib(self.double)
        arrs = [np.ascontiguousarray(a, dtype=self.dtype) for a in inputs]
        n = len(arrs)
        ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
        dims = (C.c_int64 * (5 * n))(*[d for a in arrs for d in _dims5(a.shape)])
        ranks = (C.c_int * n)(*[a.ndim for a in arrs])
        if L.fdo_predict(self.h, n, ptrs, dims, ranks) != 0:
            raise RuntimeError(L.fdo_last_error().decode())
        outs = []
        for i in range(L.fdo_out_count()):
            d = (C.c_int64 * 5)()
            r = C.c_int()
            L.fdo_out_shape(i, d, C.byref(r))
            shape = list(d)[5 - r.value:]
            o = np.empty(shape, dtype=self.dtype)
            L.fdo_out_copy(i, o.ctypes.data)
            outs.append(o)
        return outs

    def predict_multi(self, samples: Sequence[Sequence[np.ndarray]], threads: int = 1) -> List[List[np.ndarray]]:
        """samples[s][i] = input i of sample s.  Output shapes are learnt from sample 0."""
        L = lib(self.double)
        if not samples:
            return []
        first = self.predict(samples[0])
        ns, n_in, n_out = len(samples), self.n_in, len(first)
        arrs = [[np.ascontiguousarray(a, dtype=self.dtype) for a in s] for s in samples]
        outs = [[np.empty_like(o) for o in first] for _ in range(ns)]
        # output shapes may differ per sample only when input shapes differ
        for s in range(ns):
            if any(a.shape != b.shape for a, b in zip(arrs[s], arrs[0])):
                outs[s] = [np.empty_like(o) for o in self.predict(arrs[s])]
        in_ptrs = (C.c_void_p * (ns * n_in))(*[a.ctypes.data for s in arrs for a in s])
        dims = (C.c_int64 * (5 * ns * n_in))(*[d for s in arrs for a in s for d in _dims5(a.shape)])
        ranks = (C.c_int * (ns * n_in))(*[a.ndim for s in arrs for a in s])
        out_ptrs = (C.c_void_p * (ns * n_out))(*[o.ctypes.data for s in outs for o in s])
        if L.fdo_predict_multi(self.h, ns, n_in, in_ptrs, dims, ranks, n_out, out_ptrs, threads) != 0:
            raise RuntimeError(L.fdo_last_error().decode())
        return outs

    def run_tests(self, eps: float = 1e-4) -> None:
        L = lib(self.double)
        if L.fdo_run_tests(self.h, eps) != 0:
            raise RuntimeError(L.fdo_last_error().decode())
