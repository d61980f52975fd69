// Depthwise 3 x 3 convolution (stride 1 or 2) from input tiles staged in shared memory by TMA.
//
// Replaces, for these shapes, the per-thread global loads of dwconv3x3_kernel: the reference's depthwise
// convolution (include/fdeep/depthwise_convolution.hpp:21-99) reads every input value up to nine times; here a
// persistent CTA pulls one box of the channels-last input [B][H][W][C] per tile — 32 channels x the input columns
// and rows its output tile needs, padding included (coordinates outside the image read as zero) — with one
// cp.async.bulk.tensor.4d into a ring of shared-memory stages, so the loads of the next tiles are in flight while
// the current tile is computed, and the taps come from shared memory with immediate offsets.
//
// Arithmetic per output as in dwconv_kernel (kernels.cu): per filter row a chain of three fused multiply-adds,
// the row sums added top to bottom, then the shared epilogue.  (Taps outside the image add +0.)
#include "common.hpp"
#include "device_math.cuh"
#include "kernels.cuh"
#include "tc_maps.hpp"
#include "tc_ptx.cuh"

#include <algorithm>
#include <cfloat>
#include <string>

namespace fdk {
namespace {

constexpr int DW_CB = 32;                                  // channels per tile: one 128-byte row of the box per pixel
constexpr unsigned long long DW_WAIT_LIMIT_NS = 2000000000ull;
constexpr int DW_MAX_STAGES = 4;

__device__ int g_dw_status = 0;

struct DwParams {
    float* out;
    const float* w;   // [9][C]
    EpiDev epi;
    int C, Ho, Wo;
    int pad_t, pad_l;
    int TH, TW;       // output tile
    int BW;           // input box columns
    int tiles_x, tiles_y, tiles_c;
    int spatial;            // samples x tile rows x tile columns
    int fast1, fast2;       // activation forms of the epilogue: 0 none, 1 ReLU, 2 ReLU clipped at p0, 3 general
    int stages;
    unsigned stage_bytes;   // distance between stages (the box rounded up to 1 KB)
    unsigned box_bytes;     // bytes one TMA load delivers
};

// Bounded wait for a stage's bytes: suspended try_wait, the wall clock looked at between tries; gives up after 2 s,
// records that in the status word and lets the CTA leave.
__device__ __forceinline__ bool dw_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > DW_WAIT_LIMIT_NS) break;
    }
    atomicCAS(&g_dw_status, 0, 1);
    return false;
}

// 16 bytes from shared memory at a 32-bit address plus a constant offset.
template <int OFF>
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(OFF));
    return v;
}

// bias -> act1 -> affine -> residual -> act2 with the per-channel operands already in registers; the activations that
// depthwise layers carry in practice (none, ReLU, clipped ReLU) are two instructions, the rest take the general routine.
__device__ __forceinline__ float dw_act(const ActSpecDev& a, int fast, float v) {
    if (fast == 1) return fmaxf(0.0f, v);
    if (fast == 2) return v >= a.p0 ? a.p0 : (v >= 0.0f ? v : 0.0f * v);   // relu_layer.hpp:40-46 with slope 0, threshold 0
    return act_apply(a, v);
}

template <int S, int TR>
__global__ void __launch_bounds__(256) dwconv_tiles_kernel(const __grid_constant__ CUtensorMap map_in, const DwParams p) {
    extern __shared__ __align__(1024) uint8_t dw_smem[];
    __shared__ __align__(8) uint64_t full_bar[DW_MAX_STAGES];
    __shared__ int gave_up;
    const int tid = threadIdx.x;
    const uint32_t stage0 = smem_u32(dw_smem);
    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) mbar_init(smem_u32(&full_bar[i]), 1);
        gave_up = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // A CTA keeps one block of 32 channels for its whole life (weights and epilogue operands stay in registers) and
    // walks the spatial tiles (sample, tile row, tile column) with the stride of its channel block's CTA group.
    const int cc = (int)(blockIdx.x % p.tiles_c);
    const int first = (int)(blockIdx.x / p.tiles_c);
    const int stride = (int)(gridDim.x / p.tiles_c);
    const int per_image = p.tiles_x * p.tiles_y;

    auto issue = [&](int sp, int st) {  // thread 0 only
        const int b = sp / per_image;
        const int r = sp - b * per_image;
        const int ty = r / p.tiles_x;
        const int tx = r - ty * p.tiles_x;
        const uint32_t bar = smem_u32(&full_bar[st]);
        mbar_arrive_expect_tx(bar, p.box_bytes);
        tma_load_4d(stage0 + (uint32_t)st * p.stage_bytes, &map_in, cc * DW_CB, tx * p.TW * S - p.pad_l, ty * p.TH * S - p.pad_t, b, bar);
    };
    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            const int sp = first + i * stride;
            if (sp < p.spatial) issue(sp, i);
        }
    }

    const int cg = tid & 7;
    const int c = cc * DW_CB + cg * 4;
    const bool has_c = c < p.C;
    float4 wv[9];
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), scale4 = make_float4(1.f, 1.f, 1.f, 1.f), shift4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < 9; ++t) wv[t] = has_c ? __ldg(reinterpret_cast<const float4*>(p.w + t * p.C + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_c && p.epi.bias) bias4 = __ldg(reinterpret_cast<const float4*>(p.epi.bias + c));
    if (has_c && p.epi.scale) {
        scale4 = __ldg(reinterpret_cast<const float4*>(p.epi.scale + c));
        shift4 = __ldg(reinterpret_cast<const float4*>(p.epi.shift + c));
    }
    const bool has_bias = p.epi.bias != nullptr, has_affine = p.epi.scale != nullptr, has_res = p.epi.residual != nullptr;
    const int fast1 = p.fast1, fast2 = p.fast2;

    const int items = (DW_CB / 4) * p.TW * (p.TH / TR);
    const uint32_t row_b = (uint32_t)p.BW * (DW_CB * 4);
    constexpr int ROWS = (TR - 1) * S + 3;
    int it = 0;
    for (int sp = first; sp < p.spatial; sp += stride, ++it) {
        const int st = it % p.stages;
        const uint32_t parity = (uint32_t)(it / p.stages) & 1u;
        if (!dw_wait(smem_u32(&full_bar[st]), parity)) gave_up = 1;
        __syncthreads();           // (a wait that gave up is seen by the whole CTA)
        if (gave_up) return;
        const int b = sp / per_image;
        const int r = sp - b * per_image;
        const int ty = r / p.tiles_x;
        const int tx = r - ty * p.tiles_x;
        const uint32_t box = stage0 + (uint32_t)st * p.stage_bytes;
        for (int item = tid; item < items; item += blockDim.x) {
            const int rest = item >> 3;
            const int g = rest / p.TW;
            const int x = rest - g * p.TW;
            const int ox = tx * p.TW + x;
            const int oy0 = ty * p.TH + g * TR;
            if (!has_c || ox >= p.Wo || oy0 >= p.Ho) continue;
            float4 acc[TR];
#pragma unroll
            for (int t = 0; t < TR; ++t) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
            uint32_t row = box + ((uint32_t)(g * TR * S) * (uint32_t)p.BW + (uint32_t)(x * S)) * (DW_CB * 4) + (uint32_t)cg * 16;
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) {
                const float4 a0 = lds128<0>(row), a1 = lds128<DW_CB * 4>(row), a2 = lds128<2 * DW_CB * 4>(row);
                row += row_b;
#pragma unroll
                for (int t = 0; t < TR; ++t) {
                    const int ky = rr - t * S;
                    if (ky < 0 || ky > 2) continue;  // compile-time after unrolling
                    const float4 f0 = wv[ky * 3], f1 = wv[ky * 3 + 1], f2 = wv[ky * 3 + 2];
                    float4 rs;
                    rs.x = fmaf(a2.x, f2.x, fmaf(a1.x, f1.x, fmaf(a0.x, f0.x, 0.f)));
                    rs.y = fmaf(a2.y, f2.y, fmaf(a1.y, f1.y, fmaf(a0.y, f0.y, 0.f)));
                    rs.z = fmaf(a2.z, f2.z, fmaf(a1.z, f1.z, fmaf(a0.z, f0.z, 0.f)));
                    rs.w = fmaf(a2.w, f2.w, fmaf(a1.w, f1.w, fmaf(a0.w, f0.w, 0.f)));
                    acc[t].x += rs.x; acc[t].y += rs.y; acc[t].z += rs.z; acc[t].w += rs.w;
                }
            }
            const long long m0 = ((long long)b * p.Ho + oy0) * p.Wo + ox;
            float* o = p.out + m0 * p.C + c;
            const float* res = has_res ? p.epi.residual + m0 * p.epi.ldr + c : nullptr;
            const long long o_step = (long long)p.Wo * p.C, r_step = (long long)p.Wo * p.epi.ldr;
#pragma unroll
            for (int t = 0; t < TR; ++t) {
                if (oy0 + t >= p.Ho) break;
                float v[4] = {acc[t].x, acc[t].y, acc[t].z, acc[t].w};
                if (has_bias) { v[0] += bias4.x; v[1] += bias4.y; v[2] += bias4.z; v[3] += bias4.w; }
                if (fast1 != 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = dw_act(p.epi.act1, fast1, v[j]);
                }
                if (has_affine) {
                    v[0] = __fadd_rn(__fmul_rn(v[0], scale4.x), shift4.x); v[1] = __fadd_rn(__fmul_rn(v[1], scale4.y), shift4.y);
                    v[2] = __fadd_rn(__fmul_rn(v[2], scale4.z), shift4.z); v[3] = __fadd_rn(__fmul_rn(v[3], scale4.w), shift4.w);
                }
                if (has_res) {
                    const float4 rv = *reinterpret_cast<const float4*>(res);
                    v[0] += rv.x; v[1] += rv.y; v[2] += rv.z; v[3] += rv.w;
                    res += r_step;
                }
                if (fast2 != 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = dw_act(p.epi.act2, fast2, v[j]);
                }
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                o += o_step;
            }
        }
        __syncthreads();           // every thread has read this stage: it may be refilled
        if (tid == 0) {
            const int next = sp + p.stages * stride;
            if (next < p.spatial) issue(next, st);
        }
    }
}

// ---- 2-D pooling over the same kind of tiles -------------------------------------------------------------------------
// Max or average pooling with a P x P window and stride S whose every tap lies inside the tensor or inside a frame of
// explicit zeros around it (a folded ZeroPadding layer: those taps read 0 and count as values, pooling_3d_layer.hpp:44-79
// on the padded tensor) - exactly what the TMA's out-of-range fill delivers.  Windows that SAME padding would clip are
// not handled here (clipped taps are skipped and do not count).  Taps in (ky, kx) order like pool3d_kernel.
struct PoolTileParams {
    float* out;
    int C, Ho, Wo;
    int off_t, off_l;       // rows / columns of the zero frame in front of the data
    int TH, TW, BW;
    int tiles_x, tiles_y, tiles_c;
    int spatial;
    int stages;
    unsigned stage_bytes, box_bytes;
};

template <int P, int S, int TR, bool IS_MAX>
__global__ void __launch_bounds__(256) pool_tiles_kernel(const __grid_constant__ CUtensorMap map_in, const PoolTileParams p) {
    extern __shared__ __align__(1024) uint8_t dw_smem[];
    __shared__ __align__(8) uint64_t full_bar[DW_MAX_STAGES];
    __shared__ int gave_up;
    const int tid = threadIdx.x;
    const uint32_t stage0 = smem_u32(dw_smem);
    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) mbar_init(smem_u32(&full_bar[i]), 1);
        gave_up = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const int cc = (int)(blockIdx.x % p.tiles_c);
    const int first = (int)(blockIdx.x / p.tiles_c);
    const int stride = (int)(gridDim.x / p.tiles_c);
    const int per_image = p.tiles_x * p.tiles_y;
    auto issue = [&](int sp, int st) {  // thread 0 only
        const int b = sp / per_image;
        const int r = sp - b * per_image;
        const int ty = r / p.tiles_x;
        const int tx = r - ty * p.tiles_x;
        const uint32_t bar = smem_u32(&full_bar[st]);
        mbar_arrive_expect_tx(bar, p.box_bytes);
        tma_load_4d(stage0 + (uint32_t)st * p.stage_bytes, &map_in, cc * DW_CB, tx * p.TW * S - p.off_l, ty * p.TH * S - p.off_t, b, bar);
    };
    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            const int sp = first + i * stride;
            if (sp < p.spatial) issue(sp, i);
        }
    }
    const int cg = tid & 7;
    const int c = cc * DW_CB + cg * 4;
    const bool has_c = c < p.C;
    const int items = (DW_CB / 4) * p.TW * (p.TH / TR);
    const uint32_t row_b = (uint32_t)p.BW * (DW_CB * 4);
    constexpr int ROWS = (TR - 1) * S + P;
    int it = 0;
    for (int sp = first; sp < p.spatial; sp += stride, ++it) {
        const int st = it % p.stages;
        const uint32_t parity = (uint32_t)(it / p.stages) & 1u;
        if (!dw_wait(smem_u32(&full_bar[st]), parity)) gave_up = 1;
        __syncthreads();
        if (gave_up) return;
        const int b = sp / per_image;
        const int r = sp - b * per_image;
        const int ty = r / p.tiles_x;
        const int tx = r - ty * p.tiles_x;
        const uint32_t box = stage0 + (uint32_t)st * p.stage_bytes;
        for (int item = tid; item < items; item += blockDim.x) {
            const int rest = item >> 3;
            const int g = rest / p.TW;
            const int x = rest - g * p.TW;
            const int ox = tx * p.TW + x;
            const int oy0 = ty * p.TH + g * TR;
            if (!has_c || ox >= p.Wo || oy0 >= p.Ho) continue;
            float4 acc[TR];
#pragma unroll
            for (int t = 0; t < TR; ++t) acc[t] = IS_MAX ? make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX) : make_float4(0.f, 0.f, 0.f, 0.f);
            uint32_t row = box + ((uint32_t)(g * TR * S) * (uint32_t)p.BW + (uint32_t)(x * S)) * (DW_CB * 4) + (uint32_t)cg * 16;
#pragma unroll
            for (int rr = 0; rr < ROWS; ++rr) {
                float4 a[P];
                a[0] = lds128<0>(row);
                a[1] = lds128<DW_CB * 4>(row);
                if (P > 2) a[P - 1] = lds128<2 * DW_CB * 4>(row);
                row += row_b;
#pragma unroll
                for (int t = 0; t < TR; ++t) {
                    const int ky = rr - t * S;
                    if (ky < 0 || ky >= P) continue;  // compile-time after unrolling
#pragma unroll
                    for (int kx = 0; kx < P; ++kx) {
                        if (IS_MAX) {
                            acc[t].x = fmaxf(acc[t].x, a[kx].x); acc[t].y = fmaxf(acc[t].y, a[kx].y);
                            acc[t].z = fmaxf(acc[t].z, a[kx].z); acc[t].w = fmaxf(acc[t].w, a[kx].w);
                        } else {
                            acc[t].x += a[kx].x; acc[t].y += a[kx].y; acc[t].z += a[kx].z; acc[t].w += a[kx].w;
                        }
                    }
                }
            }
            float* o = p.out + (((long long)b * p.Ho + oy0) * p.Wo + ox) * p.C + c;
            const long long o_step = (long long)p.Wo * p.C;
#pragma unroll
            for (int t = 0; t < TR; ++t) {
                if (oy0 + t >= p.Ho) break;
                float4 v = acc[t];
                if (!IS_MAX) { v.x = v.x / (float)(P * P); v.y = v.y / (float)(P * P); v.z = v.z / (float)(P * P); v.w = v.w / (float)(P * P); }
                *reinterpret_cast<float4*>(o) = v;
                o += o_step;
            }
        }
        __syncthreads();
        if (tid == 0) {
            const int next = sp + p.stages * stride;
            if (next < p.spatial) issue(next, st);
        }
    }
}

int dw_ctas_per_sm(size_t smem) {
    const size_t per_sm = 227 * 1024;
    return (int)std::max<size_t>(1, std::min<size_t>(4, per_sm / (smem + 1024)));
}

}  // namespace

bool dwconv_tiles_supported(const float* in, const float* w, const float* out, int C, int kh, int kw, int sy, int sx, const Epilogue& e) {
    if (tc_get_encode() == nullptr) return false;
    if (kh != 3 || kw != 3 || sy != sx || (sy != 1 && sy != 2)) return false;
    if (C % 4 != 0 || C < 8) return false;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return false;
    if (e.residual != nullptr && ((e.ldr % 4 != 0) || (reinterpret_cast<uintptr_t>(e.residual) & 15))) return false;
    return true;
}

void launch_dwconv_tiles(const float* in, const float* w, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int stride, int pad_t,
                         int pad_l, const Epilogue& e, cudaStream_t s) {
    if (B * Ho * Wo == 0) return;
    ensure(B <= 0x7fffffff, "depthwise convolution: too many samples");
    DwParams p{};
    p.out = out; p.w = w; p.epi = to_dev(e);
    p.C = C; p.Ho = Ho; p.Wo = Wo; p.pad_t = pad_t; p.pad_l = pad_l;
    const int TR = stride == 1 ? 7 : 4;
    p.TH = stride == 1 ? (Ho > 7 ? 14 : 7) : 4;
    p.TW = Wo >= 14 ? 14 : Wo;
    const int BH = (p.TH - 1) * stride + 3;
    p.BW = (p.TW - 1) * stride + 3;
    p.tiles_x = (Wo + p.TW - 1) / p.TW;
    p.tiles_y = (Ho + p.TH - 1) / p.TH;
    p.tiles_c = (C + DW_CB - 1) / DW_CB;
    const long long spatial = (long long)B * p.tiles_y * p.tiles_x;
    ensure(spatial < (1LL << 30), "depthwise convolution: too many tiles");
    p.spatial = (int)spatial;
    auto form = [](const ActSpec& a) {
        if (a.kind == ACT_NONE) return 0;
        if (a.kind == ACT_RELU) return 1;
        if (a.kind == ACT_RELU_GEN && a.p1 == 0.0f && a.p2 == 0.0f) return 2;   // slope 0, threshold 0: clipped ReLU
        return 3;
    };
    p.fast1 = form(e.act1);
    p.fast2 = form(e.act2);
    p.box_bytes = (unsigned)(BH * p.BW * DW_CB * sizeof(float));
    p.stage_bytes = (p.box_bytes + 1023u) & ~1023u;
    p.stages = 3;

    EncodeFn enc = tc_get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap map;
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)C * sizeof(float), (cuuint64_t)W * C * sizeof(float), (cuuint64_t)H * W * C * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)DW_CB, (cuuint32_t)p.BW, (cuuint32_t)BH, 1u};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (depthwise input) failed with code " + std::to_string((int)r));

    const size_t smem = (size_t)p.stages * p.stage_bytes;
    const int items = (DW_CB / 4) * p.TW * (p.TH / TR);
    const int threads = std::min(256, ((items + 31) / 32) * 32);
    const int per_sm = dw_ctas_per_sm(smem);
    // whole groups of tiles_c CTAs (one per channel block), as many groups as fit on the device at once
    const long long groups = std::max<long long>(1, std::min<long long>(spatial, (long long)tc_sm_count() * per_sm / p.tiles_c));
    const long long grid = groups * p.tiles_c;
    static bool attr_set[64] = {};
    int dev = 0;
    FDK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        FDK_CUDA(cudaFuncSetAttribute(dwconv_tiles_kernel<1, 7>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        FDK_CUDA(cudaFuncSetAttribute(dwconv_tiles_kernel<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    if (stride == 1) dwconv_tiles_kernel<1, 7><<<(unsigned)grid, threads, smem, s>>>(map, p);
    else dwconv_tiles_kernel<2, 4><<<(unsigned)grid, threads, smem, s>>>(map, p);
    FDK_CUDA(cudaGetLastError());
}

namespace {
template <int P, int S, int TR>
void launch_pool_variant(bool is_max, unsigned grid, int threads, size_t smem, const CUtensorMap& map, const PoolTileParams& p, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    FDK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        FDK_CUDA(cudaFuncSetAttribute(pool_tiles_kernel<P, S, TR, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        FDK_CUDA(cudaFuncSetAttribute(pool_tiles_kernel<P, S, TR, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    if (is_max) pool_tiles_kernel<P, S, TR, true><<<grid, threads, smem, s>>>(map, p);
    else pool_tiles_kernel<P, S, TR, false><<<grid, threads, smem, s>>>(map, p);
    FDK_CUDA(cudaGetLastError());
}
}  // namespace

// Windows 2 x 2 / stride 2 and 3 x 3 / stride 1 or 2 whose taps all lie inside the tensor or its zero frame.
// Hz, Wz: the framed sizes; pad_t / pad_l: SAME-padding offsets of the framed tensor (must be 0 here).
bool pool_tiles_supported(const float* in, const float* out, int C, int Hz, int Wz, int Ho, int Wo, int ph, int pw, int sy, int sx, int pad_t,
                          int pad_l) {
    if (tc_get_encode() == nullptr) return false;
    if (ph != pw || sy != sx || !((ph == 2 && sy == 2) || (ph == 3 && (sy == 1 || sy == 2)))) return false;
    if (pad_t != 0 || pad_l != 0) return false;
    if ((Ho - 1) * sy + ph > Hz || (Wo - 1) * sx + pw > Wz) return false;   // a window would leave the framed tensor
    if (C % 4 != 0 || C < 8) return false;
    return (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
}

void launch_pool_tiles(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int window, int stride, int frame_t,
                       int frame_l, bool is_max, cudaStream_t s) {
    if (B * Ho * Wo == 0) return;
    ensure(B <= 0x7fffffff, "pooling: too many samples");
    PoolTileParams p{};
    p.out = out; p.C = C; p.Ho = Ho; p.Wo = Wo; p.off_t = frame_t; p.off_l = frame_l;
    const int TR = stride == 1 ? 7 : 4;
    p.TH = stride == 1 ? (Ho > 7 ? 14 : 7) : 4;
    p.TW = Wo >= 14 ? 14 : Wo;
    const int BH = (p.TH - 1) * stride + window;
    p.BW = (p.TW - 1) * stride + window;
    p.tiles_x = (Wo + p.TW - 1) / p.TW;
    p.tiles_y = (Ho + p.TH - 1) / p.TH;
    p.tiles_c = (C + DW_CB - 1) / DW_CB;
    const long long spatial = (long long)B * p.tiles_y * p.tiles_x;
    ensure(spatial < (1LL << 30), "pooling: too many tiles");
    p.spatial = (int)spatial;
    p.box_bytes = (unsigned)(BH * p.BW * DW_CB * sizeof(float));
    p.stage_bytes = (p.box_bytes + 1023u) & ~1023u;
    p.stages = 3;
    EncodeFn enc = tc_get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap map;
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)C * sizeof(float), (cuuint64_t)W * C * sizeof(float), (cuuint64_t)H * W * C * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)DW_CB, (cuuint32_t)p.BW, (cuuint32_t)BH, 1u};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (pooling input) failed with code " + std::to_string((int)r));
    const size_t smem = (size_t)p.stages * p.stage_bytes;
    const int items = (DW_CB / 4) * p.TW * (p.TH / TR);
    const int threads = std::min(256, ((items + 31) / 32) * 32);
    const int per_sm = dw_ctas_per_sm(smem);
    const long long groups = std::max<long long>(1, std::min<long long>(spatial, (long long)tc_sm_count() * per_sm / p.tiles_c));
    const unsigned grid = (unsigned)(groups * p.tiles_c);
    if (window == 2) launch_pool_variant<2, 2, 4>(is_max, grid, threads, smem, map, p, s);
    else if (stride == 2) launch_pool_variant<3, 2, 4>(is_max, grid, threads, smem, map, p, s);
    else launch_pool_variant<3, 1, 7>(is_max, grid, threads, smem, map, p, s);
}

int dwconv_tiles_take_status(cudaStream_t s) {
    int v = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_dw_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbolAsync(g_dw_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return v;
}

}  // namespace fdk
