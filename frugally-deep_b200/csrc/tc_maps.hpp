// Host-side helpers shared by the tcgen05 kernels' launchers: the driver's tensor-map encoder (looked up through the
// runtime, so the library does not link against libcuda) and the 2-D operand map both kernels use.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace fdk {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// cuTensorMapEncodeTiled, or null when the driver does not offer it.
EncodeFn tc_get_encode();
// 2-D map over a row-major [rows][cols] fp32 matrix with row stride ld (floats): box = 32 columns x box_rows, 128-byte
// swizzle, elements outside the matrix read as zero.
CUtensorMap tc_make_map_2d(const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
// SM count of the current device (looked up once per device).
int tc_sm_count();

}  // namespace fdk
