"""ctypes binding of libfdeep_b200.so (declared in include/fdeep_b200.h)."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)

# Every symbol include/fdeep_b200.h declares; checked when the library is loaded.
EXPORTS = [
    "fdk_last_error", "fdk_device_count", "fdk_model_load_file", "fdk_model_load_json", "fdk_model_destroy",
    "fdk_model_num_inputs", "fdk_model_num_outputs", "fdk_model_input_shape", "fdk_model_output_shape",
    "fdk_model_name", "fdk_model_hash", "fdk_model_num_devices", "fdk_model_infer_shapes",
    "fdk_model_predict_multi", "fdk_model_predict_multi_u8", "fdk_model_predict_batch_device", "fdk_model_sync", "fdk_model_run_tests",
    "fdk_model_launch_count", "fdk_model_plan_info", "fdk_model_profile", "fdk_plan_describe", "fdk_gemm", "fdk_split_tf32", "fdk_gemm_presplit", "fdk_tc_status", "fdk_shard_block", "fdk_gemm_static", "fdk_gemm_static_max_weight_floats",
    "fdk_session_create", "fdk_session_step", "fdk_session_info", "fdk_session_reset", "fdk_session_destroy",
    "fdk_model_cuda_device", "fdk_device_alloc", "fdk_device_free", "fdk_device_copy", "fdk_transfer_bytes",
]


class FdeepError(RuntimeError):
    """Raised where the reference throws std::runtime_error (include/fdeep/common.hpp:42-57)."""


_lib = None


def library_path() -> str:
    return os.path.join(_ROOT, "libfdeep_b200.so")


def load_library():
    """Loads the in-tree shared library.  Fails loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise FdeepError(f"{path} is missing: build it with `python frugally-deep_b200/build.py` "
                         "(there is no fallback implementation)")
    L = C.CDLL(path)
    missing = [s for s in EXPORTS if not hasattr(L, s)]
    if missing:
        raise FdeepError(f"{path} does not export {missing}")
    vp, i64p, ip = C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int)
    L.fdk_last_error.restype = C.c_size_t
    L.fdk_last_error.argtypes = [C.c_char_p, C.c_size_t]
    L.fdk_device_count.argtypes = [ip]
    L.fdk_model_load_file.argtypes = [C.c_char_p, ip, C.c_int, C.c_uint, C.POINTER(vp)]
    L.fdk_model_load_json.argtypes = [C.c_char_p, C.c_size_t, ip, C.c_int, C.c_uint, C.POINTER(vp)]
    L.fdk_model_destroy.argtypes = [vp]
    L.fdk_model_destroy.restype = None
    for f in ("fdk_model_num_inputs", "fdk_model_num_outputs", "fdk_model_num_devices"):
        getattr(L, f).argtypes = [vp]
    L.fdk_model_input_shape.argtypes = [vp, C.c_int, i64p, ip]
    L.fdk_model_output_shape.argtypes = [vp, C.c_int, i64p, ip]
    L.fdk_model_name.argtypes = [vp]
    L.fdk_model_name.restype = C.c_char_p
    L.fdk_model_hash.argtypes = [vp]
    L.fdk_model_hash.restype = C.c_char_p
    L.fdk_model_infer_shapes.argtypes = [vp, i64p, ip, i64p, ip]
    L.fdk_model_predict_multi.argtypes = [vp, C.c_int64, C.POINTER(vp), i64p, ip, C.POINTER(vp)]
    L.fdk_model_predict_multi_u8.argtypes = [vp, C.c_int64, C.POINTER(vp), i64p, ip, C.c_float, C.c_float, C.POINTER(vp)]
    L.fdk_model_predict_batch_device.argtypes = [vp, C.c_int, C.c_int64, C.POINTER(vp), i64p, ip, C.POINTER(vp), vp]
    L.fdk_model_sync.argtypes = [vp, C.c_int]
    L.fdk_model_run_tests.argtypes = [vp, C.c_float, ip]
    L.fdk_model_launch_count.argtypes = [vp]
    L.fdk_model_launch_count.restype = C.c_int64
    L.fdk_model_plan_info.argtypes = [vp, i64p, ip, C.POINTER(C.c_double), i64p, i64p]
    L.fdk_model_profile.argtypes = [vp, C.c_int, C.c_int64, C.POINTER(vp), i64p, ip, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    L.fdk_plan_describe.argtypes = [C.c_char_p, C.c_size_t, i64p, ip, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    L.fdk_gemm.argtypes = [C.c_int, vp, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int64, C.c_int, C.c_int, vp, C.c_int, vp]
    L.fdk_split_tf32.argtypes = [vp, vp, vp, C.c_int64, vp]
    L.fdk_gemm_presplit.argtypes = [vp, C.c_int64, vp, vp, C.c_int64, vp, C.c_int64, C.c_int64, C.c_int, C.c_int, vp, vp, C.c_int, vp]
    L.fdk_tc_status.argtypes = [vp, ip]
    L.fdk_session_create.argtypes = [vp, vp, C.c_int64, C.c_int64, C.POINTER(vp)]
    L.fdk_session_step.argtypes = [vp, vp, vp, vp]
    L.fdk_session_info.argtypes = [vp, i64p, i64p, i64p]
    L.fdk_session_reset.argtypes = [vp]
    L.fdk_session_destroy.argtypes = [vp]
    L.fdk_session_destroy.restype = None
    L.fdk_gemm_static.argtypes = [vp, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int64, C.c_int, C.c_int, vp, C.c_int, vp]
    L.fdk_gemm_static_max_weight_floats.argtypes = []
    L.fdk_gemm_static_max_weight_floats.restype = C.c_int64
    L.fdk_shard_block.argtypes = [C.c_int64, C.c_int, C.c_int, i64p, i64p]
    L.fdk_model_cuda_device.argtypes = [vp, C.c_int, ip]
    L.fdk_device_alloc.argtypes = [C.c_int, C.c_size_t, C.POINTER(vp)]
    L.fdk_device_free.argtypes = [C.c_int, vp]
    L.fdk_device_copy.argtypes = [C.c_int, vp, vp, C.c_size_t, C.c_int]
    L.fdk_transfer_bytes.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    _lib = L
    return L


def _err() -> str:
    L = load_library()
    n = L.fdk_last_error(None, 0)
    buf = C.create_string_buffer(n + 1)
    L.fdk_last_error(buf, n + 1)
    return buf.value.decode(errors="replace")


def _check(rc: int) -> None:
    if rc != 0:
        raise FdeepError(_err())


def device_count() -> int:
    n = C.c_int(0)
    _check(load_library().fdk_device_count(C.byref(n)))
    return n.value


def _dims5(shape: Sequence[int]) -> List[int]:
    if not 1 <= len(shape) <= 5:
        raise FdeepError("Invalid tensor-shape dimensions")
    return [1] * (5 - len(shape)) + [int(s) for s in shape]


FLAG_NO_TENSOR_CORES = 1
FLAG_SKINNY_PRODUCTS = 2
FLAG_FUSED_CELLS = 4


class Model:
    """Counterpart of fdeep::model (include/fdeep/model.hpp:19-182)."""

    def __init__(self, handle):
        self._h = handle
        L = load_library()
        self.n_inputs = L.fdk_model_num_inputs(handle)
        self.n_outputs = L.fdk_model_num_outputs(handle)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            load_library().fdk_model_destroy(h)
            self._h = None

    # -- metadata -----------------------------------------------------------------
    def name(self) -> str:
        return load_library().fdk_model_name(self._h).decode()

    def hash(self) -> str:
        return load_library().fdk_model_hash(self._h).decode()

    def num_devices(self) -> int:
        return load_library().fdk_model_num_devices(self._h)

    def _var_shape(self, fn, i):
        d = (C.c_int64 * 5)()
        r = C.c_int()
        _check(fn(self._h, i, d, C.byref(r)))
        return [None if v < 0 else int(v) for v in list(d)[5 - r.value:]]

    def get_input_shapes(self):
        L = load_library()
        return [self._var_shape(L.fdk_model_input_shape, i) for i in range(self.n_inputs)]

    def get_output_shapes(self):
        L = load_library()
        return [self._var_shape(L.fdk_model_output_shape, i) for i in range(self.n_outputs)]

    def infer_shapes(self, in_shapes: Sequence[Sequence[int]]) -> List[List[int]]:
        L = load_library()
        n = self.n_inputs
        if len(in_shapes) != n:
            raise FdeepError(f"Invalid number of input tensors for this model: {n} required but {len(in_shapes)} provided")
        dims = (C.c_int64 * (5 * n))(*[d for s in in_shapes for d in _dims5(s)])
        ranks = (C.c_int * n)(*[len(s) for s in in_shapes])
        od = (C.c_int64 * (5 * self.n_outputs))()
        orank = (C.c_int * self.n_outputs)()
        _check(L.fdk_model_infer_shapes(self._h, dims, ranks, od, orank))
        return [list(od[5 * o + 5 - orank[o]:5 * o + 5]) for o in range(self.n_outputs)]

    def plan_info(self, in_shapes: Sequence[Sequence[int]]):
        L = load_library()
        n = self.n_inputs
        dims = (C.c_int64 * (5 * n))(*[d for s in in_shapes for d in _dims5(s)])
        ranks = (C.c_int * n)(*[len(s) for s in in_shapes])
        fl, ab, mb = C.c_double(), C.c_int64(), C.c_int64()
        _check(L.fdk_model_plan_info(self._h, dims, ranks, C.byref(fl), C.byref(ab), C.byref(mb)))
        return {"flops_per_sample": fl.value, "arena_bytes_per_sample": ab.value, "max_batch": mb.value}

    def launch_count(self) -> int:
        return int(load_library().fdk_model_launch_count(self._h))

    # -- prediction ------------------------------------------------------------------
    def predict(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        """model::predict (model.hpp:23-26): one sample, a list of arrays without batch dimension."""
        return self.predict_multi([inputs])[0]

    def predict_multi(self, samples: Sequence[Sequence[np.ndarray]], bytes_range: Optional[Sequence[float]] = None) -> List[List[np.ndarray]]:
        """model::predict_multi (model.hpp:31-42): samples[s][i] is input i of sample s (host arrays).  With
        bytes_range = (low, high) the inputs are uint8 arrays scaled into that range on the GPU."""
        L = load_library()
        ns = len(samples)
        if ns == 0:
            return []
        n_in, n_out = self.n_inputs, self.n_outputs
        arrs = []
        for s in samples:
            if len(s) != n_in:
                raise FdeepError(f"Invalid number of input tensors for this model: {n_in} required but {len(s)} provided")
            arrs.append([np.ascontiguousarray(a, dtype=np.uint8 if bytes_range is not None else np.float32) for a in s])
        shape_cache = {}
        outs = []
        for s in arrs:
            key = tuple(a.shape for a in s)
            if key not in shape_cache:
                shape_cache[key] = self.infer_shapes([a.shape for a in s])
            outs.append([np.empty(sh, dtype=np.float32) for sh in shape_cache[key]])
        in_ptrs = (C.c_void_p * (ns * n_in))(*[a.ctypes.data for s in arrs for a in s])
        dims = (C.c_int64 * (5 * ns * n_in))(*[d for s in arrs for a in s for d in _dims5(a.shape)])
        ranks = (C.c_int * (ns * n_in))(*[a.ndim for s in arrs for a in s])
        out_ptrs = (C.c_void_p * (ns * n_out))(*[o.ctypes.data for s in outs for o in s])
        if bytes_range is not None:
            _check(L.fdk_model_predict_multi_u8(self._h, ns, in_ptrs, dims, ranks, float(bytes_range[0]), float(bytes_range[1]), out_ptrs))
        else:
            _check(L.fdk_model_predict_multi(self._h, ns, in_ptrs, dims, ranks, out_ptrs))
        return outs

    def predict_batch(self, inputs: Sequence[np.ndarray], bytes_range: Optional[Sequence[float]] = None) -> List[np.ndarray]:
        """Convenience for equally shaped samples: inputs[i] has shape (batch, ...); one call of
        predict_multi on views of the batch arrays, outputs stacked the same way.  With bytes_range =
        (low, high) the inputs are uint8 arrays that are scaled into that range on the GPU
        (tensor_from_bytes, tensor.hpp:1230-1245)."""
        L = load_library()
        n_in, n_out = self.n_inputs, self.n_outputs
        arrs = [np.ascontiguousarray(a, dtype=np.uint8 if bytes_range is not None else np.float32) for a in inputs]
        ns = arrs[0].shape[0]
        out_shapes = self.infer_shapes([a.shape[1:] for a in arrs])
        outs = [np.empty([ns] + list(sh), dtype=np.float32) for sh in out_shapes]
        in_ptrs = (C.c_void_p * (ns * n_in))()
        out_ptrs = (C.c_void_p * (ns * n_out))()
        for i, a in enumerate(arrs):
            stride = a.strides[0] if ns > 0 else 0
            base = a.ctypes.data
            for s in range(ns):
                in_ptrs[s * n_in + i] = base + s * stride
        for o, a in enumerate(outs):
            stride = a.strides[0] if ns > 0 else 0
            base = a.ctypes.data
            for s in range(ns):
                out_ptrs[s * n_out + o] = base + s * stride
        one = [d for a in arrs for d in _dims5(a.shape[1:])]
        dims = (C.c_int64 * (5 * ns * n_in))(*(one * ns))
        ranks = (C.c_int * (ns * n_in))(*([a.ndim - 1 for a in arrs] * ns))
        if bytes_range is not None:
            _check(L.fdk_model_predict_multi_u8(self._h, ns, in_ptrs, dims, ranks, float(bytes_range[0]), float(bytes_range[1]), out_ptrs))
        else:
            _check(L.fdk_model_predict_multi(self._h, ns, in_ptrs, dims, ranks, out_ptrs))
        return outs

    def predict_batch_device(self, d_in_ptrs: Sequence[int], in_shapes: Sequence[Sequence[int]], batch: int,
                             d_out_ptrs: Sequence[int], stream: int = 0, device_index: int = 0) -> None:
        """Device-resident batch: raw device pointers (e.g. torch tensor.data_ptr()), per-sample shapes.
        Queued on `stream`; call sync() before reading the outputs."""
        L = load_library()
        n_in, n_out = self.n_inputs, self.n_outputs
        ip = (C.c_void_p * n_in)(*d_in_ptrs)
        op = (C.c_void_p * n_out)(*d_out_ptrs)
        dims = (C.c_int64 * (5 * n_in))(*[d for s in in_shapes for d in _dims5(s)])
        ranks = (C.c_int * n_in)(*[len(s) for s in in_shapes])
        _check(L.fdk_model_predict_batch_device(self._h, device_index, batch, ip, dims, ranks, op, C.c_void_p(stream)))

    def profile(self, d_in_ptrs: Sequence[int], in_shapes: Sequence[Sequence[int]], batch: int, device_index: int = 0):
        """One device-resident batch timed with CUDA events per operation and per contraction kernel.
        Returns a list of dicts: kind ('op' | 'gemm'), layer, ms, flops, M, N, K, path."""
        L = load_library()
        n_in = self.n_inputs
        ip = (C.c_void_p * n_in)(*d_in_ptrs)
        dims = (C.c_int64 * (5 * n_in))(*[d for s in in_shapes for d in _dims5(s)])
        ranks = (C.c_int * n_in)(*[len(s) for s in in_shapes])
        size = 8 << 20
        buf = C.create_string_buffer(size)
        needed = C.c_size_t(0)
        _check(L.fdk_model_profile(self._h, device_index, batch, ip, dims, ranks, buf, size, C.byref(needed)))
        recs = []
        for line in buf.value.decode().strip().split("\n"):
            f = line.split()
            if len(f) == 8:
                recs.append({"kind": f[0], "layer": f[1], "ms": float(f[2]), "flops": float(f[3]), "M": int(f[4]),
                             "N": int(f[5]), "K": int(f[6]), "path": f[7]})
        return recs

    def sync(self, device_index: int = 0) -> None:
        _check(load_library().fdk_model_sync(self._h, device_index))

    def predict_class(self, inputs: Sequence[np.ndarray]) -> int:
        """model::predict_class (model.hpp:48-51)."""
        out = self.predict(inputs)
        if len(out) != 1:
            raise FdeepError("invalid number of outputs")
        return int(np.argmax(out[0].reshape(-1)))

    def run_tests(self, epsilon: float = 1e-4) -> int:
        """The load-time self test of load_model(verify=True) (model.hpp:254-267)."""
        n = C.c_int(0)
        _check(load_library().fdk_model_run_tests(self._h, epsilon, C.byref(n)))
        return n.value


def _devs(devices: Optional[Sequence[int]]):
    if not devices:
        return None, 0
    arr = (C.c_int * len(devices))(*devices)
    return arr, len(devices)


def _flags(tensor_cores: bool, skinny_products: bool, fused_cells: bool = False) -> int:
    return ((0 if tensor_cores else FLAG_NO_TENSOR_CORES) | (FLAG_SKINNY_PRODUCTS if skinny_products else 0) |
            (FLAG_FUSED_CELLS if fused_cells else 0))


def load_model(path: str, verify: bool = True, devices: Optional[Sequence[int]] = None, verify_epsilon: float = 1e-4,
               tensor_cores: bool = True, skinny_products: bool = False, fused_cells: bool = False) -> Model:
    """fdeep::load_model (model.hpp:285-301)."""
    L = load_library()
    h = C.c_void_p()
    arr, n = _devs(devices)
    _check(L.fdk_model_load_file(path.encode(), arr, n, _flags(tensor_cores, skinny_products, fused_cells), C.byref(h)))
    m = Model(h)
    if verify:
        m.run_tests(verify_epsilon)
    return m


def read_model_from_string(text: str, verify: bool = True, devices: Optional[Sequence[int]] = None,
                           verify_epsilon: float = 1e-4, tensor_cores: bool = True, skinny_products: bool = False, fused_cells: bool = False) -> Model:
    """fdeep::read_model_from_string (model.hpp:272-281)."""
    L = load_library()
    h = C.c_void_p()
    arr, n = _devs(devices)
    b = text.encode() if isinstance(text, str) else text
    _check(L.fdk_model_load_json(b, len(b), arr, n, _flags(tensor_cores, skinny_products, fused_cells), C.byref(h)))
    m = Model(h)
    if verify:
        m.run_tests(verify_epsilon)
    return m


def shard_block(n_samples: int, n_parts: int, part: int):
    """Contiguous block [begin, end) of `part` when n_samples are split over n_parts devices or ranks."""
    b, e = C.c_int64(0), C.c_int64(0)
    _check(load_library().fdk_shard_block(n_samples, n_parts, part, C.byref(b), C.byref(e)))
    return b.value, e.value


def split_tf32(dW: int, d_big: int, d_small: int, n: int, stream: int = 0) -> None:
    """fdk_split_tf32 on raw device pointers."""
    _check(load_library().fdk_split_tf32(C.c_void_p(dW), C.c_void_p(d_big), C.c_void_p(d_small), n, C.c_void_p(stream)))


def gemm_presplit(dA: int, lda: int, dW_big: int, dW_small: int, ldw: int, dC: int, ldc: int, M: int, N: int, K: int,
                  d_bias: int = 0, d_residual: int = 0, relu: bool = False, stream: int = 0) -> None:
    """fdk_gemm_presplit on raw device pointers: no allocation, no synchronisation."""
    _check(load_library().fdk_gemm_presplit(C.c_void_p(dA), lda, C.c_void_p(dW_big), C.c_void_p(dW_small), ldw, C.c_void_p(dC), ldc,
                                            M, N, K, C.c_void_p(d_bias), C.c_void_p(d_residual), 1 if relu else 0, C.c_void_p(stream)))


def tc_status(stream: int = 0) -> int:
    st = C.c_int(0)
    _check(load_library().fdk_tc_status(C.c_void_p(stream), C.byref(st)))
    return st.value


def plan_describe(json_text: str, in_shapes: Sequence[Sequence[int]]) -> str:
    """Host-only: compile the plan for `in_shapes` and return its listing (no CUDA device needed)."""
    L = load_library()
    b = json_text.encode() if isinstance(json_text, str) else json_text
    n = len(in_shapes)
    dims = (C.c_int64 * (5 * max(n, 1)))(*[d for s in in_shapes for d in _dims5(s)])
    ranks = (C.c_int * max(n, 1))(*[len(s) for s in in_shapes])
    needed = C.c_size_t(0)
    _check(L.fdk_plan_describe(b, len(b), dims, ranks, n, None, 0, C.byref(needed)))
    buf = C.create_string_buffer(needed.value + 1)
    _check(L.fdk_plan_describe(b, len(b), dims, ranks, n, buf, needed.value + 1, C.byref(needed)))
    return buf.value.decode()


def gemm(path: int, dA: int, lda: int, dW: int, ldw: int, dC: int, ldc: int, M: int, N: int, K: int,
         d_bias: int = 0, relu: bool = False, stream: int = 0) -> None:
    """Kernel-level entry point fdk_gemm on raw device pointers (path 0 = FFMA, 1 = tcgen05 3xTF32, 2 = the split-K
    kernel for at most 64 rows, 3 = the tcgen05 cluster kernel for at most 64 rows)."""
    _check(load_library().fdk_gemm(path, C.c_void_p(dA), lda, C.c_void_p(dW), ldw, C.c_void_p(dC), ldc, M, N, K,
                                   C.c_void_p(d_bias), 1 if relu else 0, C.c_void_p(stream)))


def gemm_static(dA: int, lda: int, dW: int, ldw: int, dC: int, ldc: int, M: int, N: int, K: int,
                d_bias: int = 0, relu: bool = False, stream: int = 0) -> None:
    """fdk_gemm_static on raw device pointers: the tcgen05 contraction with the weight halves kept in a fixed
    array of the library image, for callers that must not allocate device memory (a serving loop that cannot
    take cudaMalloc's device-wide stall, a process whose own pool owns the GPU's memory).  Queued on `stream`,
    not synchronised; calls that can overlap on the GPU share the array and must be serialised."""
    _check(load_library().fdk_gemm_static(C.c_void_p(dA), lda, C.c_void_p(dW), ldw, C.c_void_p(dC), ldc, M, N, K,
                                          C.c_void_p(d_bias), 1 if relu else 0, C.c_void_p(stream)))


def gemm_static_max_weight_floats() -> int:
    """Largest N * ldw that gemm_static accepts."""
    return int(load_library().fdk_gemm_static_max_weight_floats())


class DecodeSession:
    """Device-resident greedy decode loop over the two incremental graphs of a decoder (fdk_session_*): the
    rows that the attention blocks emit stay on the device as the key/value cache."""

    def __init__(self, first: Model, step: Model, batch: int, max_len: int):
        self._h = C.c_void_p()
        self._keep = (first, step)  # the session borrows the models
        _check(load_library().fdk_session_create(first._h, step._h, batch, max_len, C.byref(self._h)))
        b, v, n = C.c_int64(0), C.c_int64(0), C.c_int64(0)
        _check(load_library().fdk_session_info(self._h, C.byref(n), C.byref(b), C.byref(v)))
        self.batch, self.vocab = b.value, v.value

    def step(self, tokens: Optional[np.ndarray] = None, want_logits: bool = False):
        """Feeds one token per sequence (None: the greedy choice of the previous step); returns (next_tokens,
        logits or None)."""
        nxt = np.empty(self.batch, np.float32)
        logits = np.empty((self.batch, self.vocab), np.float32) if want_logits else None
        tok = None if tokens is None else np.ascontiguousarray(tokens, np.float32)
        _check(load_library().fdk_session_step(self._h, None if tok is None else tok.ctypes.data_as(C.c_void_p), nxt.ctypes.data_as(C.c_void_p),
                                               None if logits is None else logits.ctypes.data_as(C.c_void_p)))
        return nxt, logits

    @property
    def length(self) -> int:
        n = C.c_int64(0)
        _check(load_library().fdk_session_info(self._h, C.byref(n), None, None))
        return n.value

    def reset(self):
        """Back to length 0 for a new batch of sequences; buffers and the recorded position are kept."""
        _check(load_library().fdk_session_reset(self._h))

    def close(self):
        if self._h:
            load_library().fdk_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
