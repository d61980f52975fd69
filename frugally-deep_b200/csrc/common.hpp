// Shared host-side types of the engine: errors, shapes, activation and epilogue descriptors.
#pragma once

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

namespace fdk {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
[[noreturn]] inline void raise(const std::string& msg) { throw Error(msg); }
inline void ensure(bool cond, const std::string& msg) {
    if (!cond) raise(msg);
}
inline void cuda_check(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess)
        raise(std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what + " at " + file + ":" + std::to_string(line));
}
#define FDK_CUDA(x) ::fdk::cuda_check((x), #x, __FILE__, __LINE__)

// Right-aligned rank-5 shape (dim5, dim4, height, width, depth), channels last, row major;
// same convention as the reference's tensor_shape (tensor_shape.hpp:23-170).
struct TShape {
    int64_t d[5] = {1, 1, 1, 1, 1};
    int rank = 1;
    int64_t volume() const { return d[0] * d[1] * d[2] * d[3] * d[4]; }
    int64_t depth() const { return d[4]; }
    int64_t width() const { return d[3]; }
    int64_t height() const { return d[2]; }
    bool same_dims(const TShape& o) const {
        for (int i = 0; i < 5; ++i)
            if (d[i] != o.d[i]) return false;
        return true;
    }
    bool operator==(const TShape& o) const { return rank == o.rank && same_dims(o); }
    bool operator!=(const TShape& o) const { return !(*this == o); }
    int minimal_rank() const {
        for (int i = 0; i < 4; ++i)
            if (d[i] > 1) return 5 - i;
        return 1;
    }
    std::vector<int64_t> dims() const { return std::vector<int64_t>(d + 5 - rank, d + 5); }
    static TShape from_dims(const std::vector<int64_t>& v) {
        ensure(!v.empty() && v.size() <= 5, "Invalid tensor-shape dimensions");
        TShape s;
        s.rank = (int)v.size();
        for (size_t i = 0; i < v.size(); ++i) s.d[5 - v.size() + i] = v[i];
        return s;
    }
    std::string str() const {
        std::string r = "(";
        for (int i = 5 - rank; i < 5; ++i) r += std::to_string(d[i]) + (i < 4 ? ", " : "");
        return r + ")";
    }
};

// Variable shape: -1 marks a dimension that is free at load time (tensor_shape_variable.hpp:97-101).
struct VarShape {
    std::vector<int64_t> dims;
    bool matches(const TShape& s) const {
        if ((int)dims.size() != s.rank) return false;
        for (size_t i = 0; i < dims.size(); ++i)
            if (dims[i] >= 0 && dims[i] != s.d[5 - s.rank + (int)i]) return false;
        return true;
    }
    std::string str() const {
        std::string r = "(";
        for (size_t i = 0; i < dims.size(); ++i) r += (dims[i] < 0 ? std::string("None") : std::to_string(dims[i])) + (i + 1 < dims.size() ? ", " : "");
        return r + ")";
    }
};

// Elementwise activations; numbering shared with the device code (kernels.cuh).
enum ActKind : int {
    ACT_NONE = 0,
    ACT_RELU = 1,        // max(0, x)
    ACT_RELU_GEN = 2,    // p0 max_value, p1 negative_slope, p2 threshold (relu_layer.hpp:40-46)
    ACT_SIGMOID = 3,
    ACT_TANH = 4,
    ACT_GELU = 5,        // exact erf form
    ACT_SWISH = 6,
    ACT_HARD_SIGMOID = 7,
    ACT_SOFTPLUS = 8,
    ACT_ELU = 9,         // p0 alpha
    ACT_SELU = 10,
    ACT_LEAKY_RELU = 11, // p0 slope
    ACT_EXP = 12,
    ACT_SOFTSIGN = 13,
    ACT_CELU = 14,       // p0 alpha
    ACT_HARD_TANH = 15,
    ACT_LOG_SIGMOID = 16,
    ACT_TANH_SHRINK = 17,
    ACT_AFFINE = 18,     // p0 * x + p1 (Rescaling layer, rescaling_layer.hpp:31-34)
    ACT_THRESHOLD = 19,  // x > p0 ? x : p1 (threshold_layer.hpp)
    ACT_HARD_SHRINK = 20,   // |x| > p0 ? x : 0 (hard_shrink_layer.hpp)
    ACT_SOFT_SHRINK = 21,   // x - p0, x + p0 or 0 (soft_shrink_layer.hpp)
    ACT_SPARSE_PLUS = 22,   // 0, (x + 1)^2 / 4 or x (sparse_plus_layer.hpp)
    ACT_SQUARE_PLUS = 23,   // (x + sqrt(x^2 + p0)) / 2 (square_plus_layer.hpp)
    // Not elementwise; never placed in an epilogue:
    ACT_SOFTMAX = 100,
    ACT_LOG_SOFTMAX = 101,
};

struct ActSpec {
    int kind = ACT_NONE;
    float p0 = 0.f, p1 = 0.f, p2 = 0.f;
    bool none() const { return kind == ACT_NONE; }
    bool elementwise() const { return kind < 100; }
};

// Fused tail of a contraction, applied per output element in this order:
//   v = acc (+ bias[n]) -> act1 -> v * scale[n] + shift[n] -> + residual[m, n] -> act2
struct Epilogue {
    const float* bias = nullptr;
    ActSpec act1;
    const float* scale = nullptr;  // scale and shift come together
    const float* shift = nullptr;
    const float* residual = nullptr;
    int64_t ldr = 0;
    ActSpec act2;
};

}  // namespace fdk
