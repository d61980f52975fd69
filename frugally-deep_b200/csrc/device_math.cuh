// Device-side activation and epilogue arithmetic shared by all kernels.
//
// Formulas follow the reference's scalar activations (recurrent_ops.hpp:24-86 and the
// layers/*_layer.hpp transform_input bodies); libdevice expf/erff/tanhf/logf stand in for libm.
#pragma once

#include "common.hpp"

#include <cfloat>

namespace fdk {

struct ActSpecDev {
    int kind;
    float p0, p1, p2;
};
struct EpiDev {
    const float* bias;
    const float* scale;
    const float* shift;
    const float* residual;
    long long ldr;
    ActSpecDev act1, act2;
};

inline ActSpecDev to_dev(const ActSpec& a) { return ActSpecDev{a.kind, a.p0, a.p1, a.p2}; }
inline EpiDev to_dev(const Epilogue& e) {
    return EpiDev{e.bias, e.scale, e.shift, e.residual, (long long)e.ldr, to_dev(e.act1), to_dev(e.act2)};
}

// Activations that need libdevice transcendentals stay out of line: inlined into unrolled epilogues
// they multiplied the code size until instruction fetch, not memory, limited the kernels.
static __device__ __noinline__ float act_apply_general(const ActSpecDev a, float x) {
    switch (a.kind) {
        case ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case ACT_TANH: return tanhf(x);
        case ACT_GELU: return 0.5f * x * (1.0f + erff(x / sqrtf(2.0f)));
        case ACT_SWISH: return x / (1.0f + expf(-x));
        case ACT_HARD_SIGMOID:
            if (x < -3.0f) return 0.0f;
            if (x > 3.0f) return 1.0f;
            return (x / 6.0f) + 0.5f;
        case ACT_SOFTPLUS: {  // softplus_layer.hpp:27-36
            const float th = logf(FLT_EPSILON) + 2.0f;
            if (x > -th) return x;
            if (x < th) return expf(x);
            return log1pf(expf(x));
        }
        case ACT_ELU:
        case ACT_CELU: return x >= 0.0f ? x : a.p0 * (expf(x) - 1.0f);
        case ACT_SELU: {
            const float alpha = 1.6732632423543772848170429916717f, scale = 1.0507009873554804934193349852946f;
            return scale * (x >= 0.0f ? x : alpha * (expf(x) - 1.0f));
        }
        case ACT_LEAKY_RELU: return x > 0.0f ? x : a.p0 * x;
        case ACT_EXP: return expf(x);
        case ACT_SOFTSIGN: return x / (fabsf(x) + 1.0f);
        case ACT_HARD_TANH: return fminf(1.0f, fmaxf(-1.0f, x));
        case ACT_LOG_SIGMOID: return logf(1.0f / (1.0f + expf(-x)));
        case ACT_TANH_SHRINK: return x - tanhf(x);
        case ACT_AFFINE: return __fadd_rn(__fmul_rn(a.p0, x), a.p1);
        case ACT_THRESHOLD: return x > a.p0 ? x : a.p1;
        case ACT_HARD_SHRINK: return fabsf(x) > a.p0 ? x : 0.0f;
        case ACT_SOFT_SHRINK:
            if (x > a.p0) return x - a.p0;
            if (x < -a.p0) return x + a.p0;
            return 0.0f;
        case ACT_SPARSE_PLUS:
            if (x <= -1.0f) return 0.0f;
            if (x < 1.0f) return __fmul_rn(__fmul_rn(0.25f, x + 1.0f), x + 1.0f);
            return x;
        case ACT_SQUARE_PLUS: return (x + sqrtf(__fadd_rn(__fmul_rn(x, x), a.p0))) / 2.0f;
        default: return x;
    }
}
__device__ __forceinline__ float act_apply(const ActSpecDev& a, float x) {
    if (a.kind == ACT_NONE) return x;
    if (a.kind == ACT_RELU) return fmaxf(0.0f, x);
    if (a.kind == ACT_RELU_GEN) {  // relu_layer.hpp:40-46
        if (x >= a.p0) return a.p0;
        if (a.p2 <= x && x < a.p0) return x;
        return a.p1 * (x - a.p2);
    }
    return act_apply_general(a, x);
}

// v = acc + bias -> act1 -> v * scale + shift -> + residual -> act2.  The affine step keeps the
// reference's two roundings (x * inv, then + (beta - mean * inv); tensor.hpp:788-792).
__device__ __forceinline__ float epi_apply(const EpiDev& e, float v, long long row, int col) {
    if (e.bias) v += e.bias[col];
    v = act_apply(e.act1, v);
    if (e.scale) v = __fadd_rn(__fmul_rn(v, e.scale[col]), e.shift[col]);
    if (e.residual) v += e.residual[row * e.ldr + col];
    return act_apply(e.act2, v);
}
// Four consecutive columns; col % 4 == 0 and all vectors 16-byte aligned at col (checked by the caller
// for the residual; bias/scale/shift come from 256-byte aligned weight storage).
__device__ __forceinline__ void epi_apply4(const EpiDev& e, float (&v)[4], long long row, int col) {
    if (e.bias) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(e.bias + col));
        v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    }
    if (e.act1.kind != ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = act_apply(e.act1, v[j]);
    }
    if (e.scale) {
        const float4 s = __ldg(reinterpret_cast<const float4*>(e.scale + col));
        const float4 t = __ldg(reinterpret_cast<const float4*>(e.shift + col));
        v[0] = __fadd_rn(__fmul_rn(v[0], s.x), t.x); v[1] = __fadd_rn(__fmul_rn(v[1], s.y), t.y);
        v[2] = __fadd_rn(__fmul_rn(v[2], s.z), t.z); v[3] = __fadd_rn(__fmul_rn(v[3], s.w), t.w);
    }
    if (e.residual) {
        const float4 r = *reinterpret_cast<const float4*>(e.residual + row * e.ldr + col);
        v[0] += r.x; v[1] += r.y; v[2] += r.z; v[3] += r.w;
    }
    if (e.act2.kind != ACT_NONE) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = act_apply(e.act2, v[j]);
    }
}

}  // namespace fdk
