"""Python host side of the B200 engine for frugally-deep models.

Thin ctypes layer over the C ABI in include/fdeep_b200.h.  The names mirror the reference's C++
API (include/fdeep/model.hpp): ``load_model``, ``Model.predict``, ``Model.predict_multi``,
``Model.get_input_shapes`` ...  All arithmetic happens in the shared library's CUDA kernels; there is
no CPU path, and loading a model without a CUDA device raises.
"""
from .capi import (DecodeSession, FdeepError, Model, device_count, gemm, library_path, load_library, load_model,  # noqa: F401
                   plan_describe, read_model_from_string, shard_block)
