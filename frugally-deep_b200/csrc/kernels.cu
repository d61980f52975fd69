// Memory-bound layer kernels and the FFMA contraction for sm_100a.
//
// Every kernel here is a restatement, for batch-major fp32 device tensors, of one reference CPU
// routine; the file:line of that routine is given at each kernel.  The reference processes one
// sample per call; these kernels process the whole batch in one launch and keep each sample's
// arithmetic independent of the batch size and of the sample's position in the batch.
#include "kernels.cuh"
#include "device_math.cuh"
#include "pdl.cuh"

#include <cfloat>
#include <cstdlib>

namespace fdk {

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline unsigned grid_1d(int64_t n, int block) {
    int64_t g = ceil_div64(n, block);
    if (g < 1) g = 1;
    // grid-stride loops below: cap at a few waves over 148 SMs
    const int64_t cap = 148LL * 32;
    return (unsigned)(g > cap ? cap : g);
}

// =====================================================================================================
// FFMA GEMM: C[M,N] = epi(A[M,K] * W[N,K]^T).  128x128x16 tiles, 256 threads, 8x8 per thread,
// double-buffered shared memory.  Replaces the reference's Eigen GEMM call sites
// (convolution.hpp:147,274; dense_layer.hpp:85; recurrent_ops.hpp:144,165) for shapes the tensor-core
// path does not take, and serves as the exact-fp32 arbiter for it.
// =====================================================================================================
namespace {
constexpr int GBM = 128, GBN = 128, GBK = 16, GLD = GBM + 4;

template <int VEC>
__device__ __forceinline__ void gemm_load_tile(const float* __restrict__ P, int64_t ld, int64_t row0, int64_t nrows,
                                               int k0, int K, int tid, float (&r)[8]) {
    // 128 rows x 16 k = 512 float4; thread handles float4 #tid and #tid+256
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * 256;
        const int row = idx >> 2;
        const int kq = (idx & 3) * 4;
        const int64_t gr = row0 + row;
        const int gk = k0 + kq;
        if (VEC == 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr < nrows && gk < K) v = *reinterpret_cast<const float4*>(P + gr * ld + gk);
            r[i * 4 + 0] = v.x; r[i * 4 + 1] = v.y; r[i * 4 + 2] = v.z; r[i * 4 + 3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) r[i * 4 + j] = (gr < nrows && gk + j < K) ? P[gr * ld + gk + j] : 0.f;
        }
    }
}
__device__ __forceinline__ void gemm_store_tile(float (*S)[GLD], int tid, const float (&r)[8]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * 256;
        const int row = idx >> 2;
        const int kq = (idx & 3) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) S[kq + j][row] = r[i * 4 + j];
    }
}

template <int VEC>
__global__ void __launch_bounds__(256) gemm_ffma_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ W,
                                                        int64_t ldw, float* __restrict__ C, int64_t ldc, int64_t M, int N, int K,
                                                        EpiDev epi) {
    __shared__ __align__(16) float As[2][GBK][GLD];
    __shared__ __align__(16) float Bs[2][GBK][GLD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.x * GBM;
    const int n0 = blockIdx.y * GBN;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float ra[8], rb[8];
    gemm_load_tile<VEC>(A, lda, m0, M, 0, K, tid, ra);
    gemm_load_tile<VEC>(W, ldw, n0, N, 0, K, tid, rb);
    gemm_store_tile(As[0], tid, ra);
    gemm_store_tile(Bs[0], tid, rb);
    __syncthreads();

    const int nk = (K + GBK - 1) / GBK;
    for (int kt = 0; kt < nk; ++kt) {
        const int cur = kt & 1;
        if (kt + 1 < nk) {
            gemm_load_tile<VEC>(A, lda, m0, M, (kt + 1) * GBK, K, tid, ra);
            gemm_load_tile<VEC>(W, ldw, n0, N, (kt + 1) * GBK, K, tid, rb);
        }
#pragma unroll
        for (int k = 0; k < GBK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            gemm_store_tile(As[cur ^ 1], tid, ra);
            gemm_store_tile(Bs[cur ^ 1], tid, rb);
        }
        __syncthreads();
    }

    const bool vec_store = ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) &&
                           (epi.residual == nullptr || (((epi.ldr & 3) == 0) && ((reinterpret_cast<uintptr_t>(epi.residual) & 15) == 0)));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int col0 = n0 + jh * 64 + tx * 4;
            if (col0 >= N) continue;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = acc[i][jh * 4 + j];
            if (vec_store && col0 + 3 < N) {
                epi_apply4(epi, v, row, col0);
                *reinterpret_cast<float4*>(C + row * ldc + col0) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (col0 + j < N) C[row * ldc + col0 + j] = epi_apply(epi, v[j], row, col0 + j);
            }
        }
    }
}
}  // namespace

// Skinny product: M <= 64 rows (a few samples against a large weight matrix: one decode position, a dense head).
// 128-row tiles would occupy N / 128 SMs and leave the rest idle while the weights stream in.  Here the matrix is
// cut into 64-column blocks AND into slices of K, one CTA each, so that a few hundred CTAs stream disjoint parts of
// W; the partial 64 x 64 tiles go to a workspace and the CTA that arrives last for a column block adds the slices in a
// fixed order and applies the epilogue (deterministic; with a single slice every CTA applies the epilogue itself).
// Products: three TF32 tensor-core products per fp32 product, or exact fp32 FFMA (template parameter MMA below).
namespace {
constexpr int SK_BK = 32;
constexpr int SK_NB = 2;                       // shared-memory chunk buffers per operand (36.9 KB per CTA: six CTAs per SM)
constexpr int SK_LDK = SK_BK + 4;              // row stride (floats) of a chunk buffer: rows of 32 k values, 16-byte aligned
constexpr int SK_LD = 64 + 4;                  // row stride (floats) of the result tile
constexpr int SK_SMEM = 2 * SK_NB * 64 * SK_LDK * (int)sizeof(float);
// The workspace of a sliced product starts with one arrival counter per column block (zero between launches: the
// workspace is cleared when it is allocated and every launch leaves its counters at zero); partial tiles follow.
constexpr int SK_COUNTERS = 512;
// Up to two more products that ride in the same launch as the first (grid.z): see launch_gemm_skinny_group.
struct SkinnyGroup {
    const float* W[2];
    float* C[2];
    long long ldc[2];
    const float* bias[2];
};
__device__ __forceinline__ void sk_cp_async16(float* smem_dst, const float* gmem_src, bool valid) {
    // 16 bytes global -> shared without passing through registers; an invalid source gives zeros (src-size 0)
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sk_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void sk_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Structure: operands go global -> shared with cp.async (a small rolled loop issues the copies; a slice of two
// chunks has all of them in flight from the start), one rolled product loop over a two-buffer ring, and the result
// tile passes through shared memory so that neither the slice sum nor the epilogue needs the accumulators by index
// (both are rolled loops too: the kernel is short, which keeps instruction fetch out of the picture for launches
// that live 15-30 us).  Measured on B200: these launches are bound by FFMA issue (FMA pipe a third busy, shared-memory
// latency exposed at one or two CTAs per SM), not by how the operands arrive.
// MMA: the products run on the tensor cores as three TF32 products per fp32 product (operands cut into a 10-bit high
// part and the exact remainder, the low x low term dropped: error about 2^-21 of |a||b| per product, the arithmetic of
// the tcgen05 contraction path) with warp-level mma.sync on fragments read straight from the row-major chunk buffers;
// !MMA: exact fp32 FFMA products with a 4 x 4 register tile per thread.
template <bool MMA>
__global__ void __launch_bounds__(256) gemm_skinny_partial_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ W, int64_t ldw,
                                                                  float* out, int64_t ld_out, int64_t slice_stride, int M, int N,
                                                                  int K, int k_per_slice, EpiDev epi, int apply_epi, float* C, int64_t ldc,
                                                                  int* counters, SkinnyGroup grp) {
    extern __shared__ __align__(16) float sk_smem[];
    float (*As)[64][SK_LDK] = reinterpret_cast<float (*)[64][SK_LDK]>(sk_smem);
    float (*Ws)[64][SK_LDK] = reinterpret_cast<float (*)[64][SK_LDK]>(sk_smem + SK_NB * 64 * SK_LDK);
    float (*tile)[SK_LD] = reinterpret_cast<float (*)[SK_LD]>(sk_smem);   // 64 x 64 results, after the products
    // blockIdx.z > 0: a further product of the same A, shape and slicing (other weights, bias and destination)
    if (blockIdx.z > 0) {
        const int z = blockIdx.z == 1 ? 0 : 1;
        W = grp.W[z];
        C = grp.C[z];
        ldc = grp.ldc[z];
        epi.bias = grp.bias[z];
        out += (int64_t)blockIdx.z * gridDim.y * slice_stride;
        counters += blockIdx.z * gridDim.x;
    }
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * 64;
    const int k_begin = blockIdx.y * k_per_slice;
    const int k_end = min(K, k_begin + k_per_slice);
    const int chunks = (k_end - k_begin + SK_BK - 1) / SK_BK;
    // one chunk = 64 rows x 32 k of each operand = 512 float4 each: this thread copies float4 #tid and #tid + 256
    auto issue = [&](int ch, int buf) {
        const int k0 = k_begin + ch * SK_BK;
#pragma unroll 1
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 256;
            const int row = idx >> 3, kq = (idx & 7) * 4;
            const bool kin = k0 + kq < k_end;
            const bool va = kin && row < M, vw = kin && n0 + row < N;
            sk_cp_async16(&As[buf][row][kq], va ? A + (int64_t)row * lda + k0 + kq : A, va);
            sk_cp_async16(&Ws[buf][row][kq], vw ? W + (int64_t)(n0 + row) * ldw + k0 + kq : W, vw);
        }
    };
#pragma unroll 1
    for (int ch = 0; ch < SK_NB; ++ch) {
        if (ch < chunks) issue(ch, ch);
        sk_cp_async_commit();
    }
    // Epilogue operands: the bias of this thread's columns now, the residual rows pulled towards L2
    const int n_epi = n0 + (tid & 15) * 4;
    const bool vec_c = (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
                       (!epi.residual || ((epi.ldr & 3) == 0 && (reinterpret_cast<uintptr_t>(epi.residual) & 15) == 0));
    const bool vec_epi = vec_c && n_epi + 3 < N;
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec_epi && epi.bias) bias4 = __ldg(reinterpret_cast<const float4*>(epi.bias + n_epi));
    if (epi.residual && n_epi < N) {
#pragma unroll 1
        for (int it = 0; it < 4; ++it) {
            const int m = (tid >> 4) + 16 * it;
            if (m < M) asm volatile("prefetch.global.L2 [%0];" ::"l"(epi.residual + (int64_t)m * epi.ldr + n_epi));
        }
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // MMA form: warp w owns rows 16 (w & 3) .. +15 and columns 32 (w >> 2) .. +31 of the tile as four m16n8 accumulators
    // acc[j][0..3]; lane = 4 g + t holds (row g, cols 2t, 2t+1) and (row g + 8, cols 2t, 2t+1) of each
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int mrow = (warp & 3) * 16, ncol = (warp >> 2) * 32;
#pragma unroll 1
    for (int ch = 0; ch < chunks; ++ch) {
        const int cur = ch & (SK_NB - 1);
        sk_cp_async_wait<SK_NB - 1>();   // all but the newest SK_NB - 1 groups: chunk ch has landed
        __syncthreads();
        if (MMA) {
#pragma unroll 2
            for (int k8 = 0; k8 < SK_BK / 8; ++k8) {
                const int k0 = k8 * 8 + t4;
                // fragments (m16n8k8, A row-major, B column-major = rows of W): banks (4 g + t) are all different
                float af[4] = {As[cur][mrow + g][k0], As[cur][mrow + g + 8][k0], As[cur][mrow + g][k0 + 4], As[cur][mrow + g + 8][k0 + 4]};
                unsigned abig[4], asml[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    abig[i] = __float_as_uint(af[i]) & 0xffffe000u;
                    asml[i] = __float_as_uint(af[i] - __uint_as_float(abig[i]));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float bf[2] = {Ws[cur][ncol + 8 * j + g][k0], Ws[cur][ncol + 8 * j + g][k0 + 4]};
                    unsigned bbig[2], bsml[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        bbig[i] = __float_as_uint(bf[i]) & 0xffffe000u;
                        bsml[i] = __float_as_uint(bf[i] - __uint_as_float(bbig[i]));
                    }
                    // small terms first, the large product last
                    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                                 : "r"(asml[0]), "r"(asml[1]), "r"(asml[2]), "r"(asml[3]), "r"(bbig[0]), "r"(bbig[1]));
                    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                                 : "r"(abig[0]), "r"(abig[1]), "r"(abig[2]), "r"(abig[3]), "r"(bsml[0]), "r"(bsml[1]));
                    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                                 : "r"(abig[0]), "r"(abig[1]), "r"(abig[2]), "r"(abig[3]), "r"(bbig[0]), "r"(bbig[1]));
                }
            }
        } else {
#pragma unroll 2
            for (int k4 = 0; k4 < SK_BK / 4; ++k4) {
                float4 a[4], b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(&As[cur][ty * 4 + i][k4 * 4]);
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(&Ws[cur][tx + 16 * j][k4 * 4]);   // columns tx + 16 j: no bank conflicts
                // k ascending within each accumulator, as a sequential dot product
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
                        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
                        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
                        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
                    }
            }
        }
        __syncthreads();                  // everyone is done with this buffer: chunk ch + SK_NB may take it
        if (ch + SK_NB < chunks) issue(ch + SK_NB, cur);
        sk_cp_async_commit();             // one group per turn (possibly empty) keeps the wait count fixed
    }
    // results -> shared tile (the last turn's barrier freed the chunk buffers; no copy is in flight any more)
    sk_cp_async_wait<0>();
    if (MMA) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float2*>(&tile[mrow + g][ncol + 8 * j + 2 * t4]) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2*>(&tile[mrow + g + 8][ncol + 8 * j + 2 * t4]) = make_float2(acc[j][2], acc[j][3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) tile[ty * 4 + i][tx + 16 * j] = acc[i][j];
    }
    __syncthreads();
    if (!apply_epi) {
        // Several slices of K: this CTA's tile goes to the workspace; the CTA that arrives last for the column block
        // adds the tiles, always in slice order (so the result does not depend on which CTA that is).  One thread
        // per CTA orders the block's stores before its arrival and the other slices' stores before the block's loads.
        float* dst = out + (int64_t)blockIdx.y * slice_stride;
        const bool vec_part = (ld_out & 3) == 0 && (slice_stride & 3) == 0;
#pragma unroll 1
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int m = idx >> 4, n = n0 + (idx & 15) * 4;
            if (m >= M || n >= N) continue;
            const float4 q = *reinterpret_cast<const float4*>(&tile[m][(idx & 15) * 4]);
            if (vec_part && n + 3 < N) {
                __stcg(reinterpret_cast<float4*>(dst + (int64_t)m * ld_out + n), q);
            } else {
                const float qv[4] = {q.x, q.y, q.z, q.w};
                for (int j = 0; j < 4 && n + j < N; ++j) __stcg(dst + (int64_t)m * ld_out + n + j, qv[j]);
            }
        }
        __shared__ int is_last;
        __syncthreads();
        if (tid == 0) {
            // release: the block's tile (made visible to this thread by the barrier) before the arrival; acquire: the
            // other slices' tiles before the loads below
            int arrived;
            asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(counters + blockIdx.x) : "memory");
            is_last = arrived == (int)gridDim.y - 1;
        }
        __syncthreads();
        if (!is_last) return;
        const int slices = (int)gridDim.y;
#pragma unroll 1
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int m = idx >> 4, n = n0 + (idx & 15) * 4;
            if (m >= M || n >= N) continue;
            const float* src = out + (int64_t)m * ld_out + n;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            if (vec_part && n + 3 < N) {
#pragma unroll 4
                for (int s2 = 0; s2 < slices; ++s2) {
                    const float4 q = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)s2 * slice_stride));
                    sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
                }
            } else {
                for (int s2 = 0; s2 < slices; ++s2) {
                    const float* ps = src + (int64_t)s2 * slice_stride;
                    sum.x += __ldcg(ps);
                    if (n + 1 < N) sum.y += __ldcg(ps + 1);
                    if (n + 2 < N) sum.z += __ldcg(ps + 2);
                    if (n + 3 < N) sum.w += __ldcg(ps + 3);
                }
            }
            *reinterpret_cast<float4*>(&tile[m][(idx & 15) * 4]) = sum;   // the same thread reads it back below
        }
        if (tid == 0) counters[blockIdx.x] = 0;
    }
    // epilogue, tile -> C
    EpiDev rest = epi;   // the bias was fetched before the products
    if (vec_epi) rest.bias = nullptr;
#pragma unroll 1
    for (int it = 0; it < 4; ++it) {
        const int idx = tid + it * 256;
        const int m = idx >> 4, n = n_epi;
        if (m >= M || n >= N) continue;
        const float4 q = *reinterpret_cast<const float4*>(&tile[m][(idx & 15) * 4]);
        float v[4] = {q.x, q.y, q.z, q.w};
        if (vec_epi) {
            v[0] += bias4.x; v[1] += bias4.y; v[2] += bias4.z; v[3] += bias4.w;
            epi_apply4(rest, v, m, n);   // act1, scale/shift, residual, act2
            *reinterpret_cast<float4*>(C + (int64_t)m * ldc + n) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            for (int j = 0; j < 4 && n + j < N; ++j) C[(int64_t)m * ldc + n + j] = epi_apply(epi, v[j], m, n + j);
        }
    }
}
}  // namespace

bool gemm_skinny_supported(int64_t M, int N, int K, int64_t lda, int64_t ldw, const void* A, const void* W) {
    return M >= 1 && M <= 64 && N >= 1 && K >= 4 && (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) &&
           ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
}
void gemm_skinny_plan(int N, int K, int& slices, int& k_per_slice, int64_t& workspace_floats, int64_t M) {
    const int n_blocks = (N + 63) / 64;
    slices = 1;
    // enough CTAs for about two per SM (the products are bound by FFMA issue with shared-memory latency exposed, so
    // every SM should have warps to choose from), slices of at least 64 values of K (two chunks, both in flight from
    // the start), at most 24 slices (the CTA that arrives last adds them all)
    while (n_blocks * slices < 296 && slices < 24 && K / (slices + 1) >= 64) ++slices;
    k_per_slice = ((K + slices - 1) / slices + SK_BK - 1) / SK_BK * SK_BK;
    slices = (K + k_per_slice - 1) / k_per_slice;
    workspace_floats = slices > 1 ? SK_COUNTERS + (int64_t)slices * M * N : 0;
}
// FDK_SKINNY_MMA=0: exact FFMA products instead of the tensor-core form (read once per process)
static bool skinny_mma() {
    static const bool on = [] { const char* v = getenv("FDK_SKINNY_MMA"); return !(v && *v == '0'); }();
    return on;
}
#define SK_LAUNCH(grid, s) (mma ? gemm_skinny_partial_kernel<true> : gemm_skinny_partial_kernel<false>)<<<grid, 256, SK_SMEM, s>>>
static void skinny_prepare(bool mma) {
    // more than 48 KB of dynamic shared memory needs the opt-in (per device; cheap, so asked for at every launch)
    FDK_CUDA(cudaFuncSetAttribute(mma ? gemm_skinny_partial_kernel<true> : gemm_skinny_partial_kernel<false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM));
}
void launch_gemm_skinny_group(const float* A, int64_t lda, int count, const float* const* W, int64_t ldw, float* const* C, const int64_t* ldc,
                              const float* const* bias, int64_t M, int N, int K, float* workspace, cudaStream_t s, bool tensor_cores) {
    const bool mma = tensor_cores && skinny_mma();
    ensure(count >= 1 && count <= 3, "skinny product group: one to three products");
    Epilogue e;
    e.bias = bias[0];
    const EpiDev epi = to_dev(e);
    int slices = 1, kps = K;
    int64_t ws = 0;
    gemm_skinny_plan(N, K, slices, kps, ws, M);
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)slices, (unsigned)count);
    skinny_prepare(mma);
    SkinnyGroup grp = {};
    for (int i = 1; i < count; ++i) { grp.W[i - 1] = W[i]; grp.C[i - 1] = C[i]; grp.ldc[i - 1] = ldc[i]; grp.bias[i - 1] = bias[i]; }
    if (slices == 1) {
        SK_LAUNCH(grid, s)(A, lda, W[0], ldw, C[0], ldc[0], 0, (int)M, N, K, kps, epi, 1, C[0], ldc[0], nullptr, grp);
        FDK_CUDA(cudaGetLastError());
        return;
    }
    ensure(workspace != nullptr, "skinny product: workspace missing");
    ensure((int)grid.x * count <= SK_COUNTERS, "skinny product: too many column blocks for a sliced launch");
    SK_LAUNCH(grid, s)(A, lda, W[0], ldw, workspace + SK_COUNTERS, N, (int64_t)M * N, (int)M, N, K, kps, epi, 0, C[0],
                                                    ldc[0], reinterpret_cast<int*>(workspace), grp);
    FDK_CUDA(cudaGetLastError());
}
void launch_gemm_skinny(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc, int64_t M, int N, int K,
                        const Epilogue& e, float* workspace, cudaStream_t s, bool tensor_cores) {
    const bool mma = tensor_cores && skinny_mma();
    const EpiDev epi = to_dev(e);
    int slices = 1, kps = K;
    int64_t ws = 0;
    gemm_skinny_plan(N, K, slices, kps, ws, M);
    dim3 grid((unsigned)((N + 63) / 64), (unsigned)slices);
    const SkinnyGroup none = {};
    skinny_prepare(mma);
    if (slices == 1) {
        SK_LAUNCH(grid, s)(A, lda, W, ldw, C, ldc, 0, (int)M, N, K, kps, epi, 1, C, ldc, nullptr, none);
        FDK_CUDA(cudaGetLastError());
        return;
    }
    ensure(workspace != nullptr, "skinny product: workspace missing");
    ensure((int)grid.x <= SK_COUNTERS, "skinny product: too many column blocks for a sliced launch");
    SK_LAUNCH(grid, s)(A, lda, W, ldw, workspace + SK_COUNTERS, N, (int64_t)M * N, (int)M, N, K, kps, epi, 0, C, ldc,
                                                    reinterpret_cast<int*>(workspace), none);
    FDK_CUDA(cudaGetLastError());
}

void launch_gemm_ffma(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc, int64_t M, int N,
                      int K, const Epilogue& e, cudaStream_t s) {
    if (M <= 0 || N <= 0) return;
    const EpiDev epi = to_dev(e);
    dim3 grid((unsigned)ceil_div64(M, GBM), (unsigned)((N + GBN - 1) / GBN));
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
    if (vec) gemm_ffma_kernel<4><<<grid, 256, 0, s>>>(A, lda, W, ldw, C, ldc, M, N, K, epi);
    else gemm_ffma_kernel<1><<<grid, 256, 0, s>>>(A, lda, W, ldw, C, ldc, M, N, K, epi);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// im2col gather (explicit form of the reference's overlapping Eigen::Map, convolution.hpp:86-103, with
// the zero padding of pad_tensor, tensor.hpp:490-517, folded into the bounds test).
// =====================================================================================================
namespace {
template <int VEC>
__global__ void im2col_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int H, int W, int C,
                              int Ho, int Wo, int kh, int kw, int sy, int sx, int dy, int dx, int pad_t, int pad_l, int K,
                              int Kp) {
    const int kpv = Kp / VEC;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int kq = (int)(i % kpv) * VEC;
        const int64_t m = i / kpv;
        const int ox = (int)(m % Wo);
        const int oy = (int)((m / Wo) % Ho);
        const int64_t b = m / ((int64_t)Wo * Ho);
        float v[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = 0.f;
        if (kq < K) {
            const int c = kq % C;
            const int tap = kq / C;
            const int kx = tap % kw, ky = tap / kw;
            const int iy = oy * sy + ky * dy - pad_t;
            const int ix = ox * sx + kx * dx - pad_l;
            if (iy >= 0 && iy < H && ix >= 0 && ix < W) {
                const float* p = in + (((b * H + iy) * W + ix) * (int64_t)C + c);
                if (VEC == 4) {
                    const float4 t = *reinterpret_cast<const float4*>(p);
                    v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
                } else {
                    v[0] = *p;
                }
            }
        }
        if (VEC == 4) *reinterpret_cast<float4*>(out + m * Kp + kq) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
        else out[m * Kp + kq] = v[0];
    }
}

__global__ void im2col_transposed_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int H, int W,
                                         int C, int Ho, int Wo, int kh, int kw, int sy, int sx, int offy, int offx,
                                         int pad_t, int pad_l, int Hd, int Wd, int K, int Kp) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int kq = (int)(i % Kp);
        const int64_t m = i / Kp;
        const int ox = (int)(m % Wo);
        const int oy = (int)((m / Wo) % Ho);
        const int64_t b = m / ((int64_t)Wo * Ho);
        float v = 0.f;
        if (kq < K) {
            const int c = kq % C;
            const int tap = kq / C;
            const int kx = tap % kw, ky = tap / kw;
            // position in the zero-dilated tensor (tensor.hpp:612-640), after pad_tensor
            const int yd = oy + ky - pad_t, xd = ox + kx - pad_l;
            if (yd >= 0 && yd < Hd && xd >= 0 && xd < Wd) {
                const int yy = yd - offy, xx = xd - offx;
                if (yy >= 0 && xx >= 0 && yy % sy == 0 && xx % sx == 0) {
                    const int iy = yy / sy, ix = xx / sx;
                    if (iy < H && ix < W) v = in[((b * H + iy) * W + ix) * (int64_t)C + c];
                }
            }
        }
        out[m * Kp + kq] = v;
    }
}
}  // namespace

void launch_im2col(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int kh, int kw, int sy,
                   int sx, int dy, int dx, int pad_t, int pad_l, int Kp, cudaStream_t s) {
    const int K = kh * kw * C;
    const int64_t M = B * Ho * Wo;
    if (M == 0) return;
    const bool vec = (C % 4 == 0) && (Kp % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    if (vec) {
        const int64_t total = M * (Kp / 4);
        im2col_kernel<4><<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, Ho, Wo, kh, kw, sy, sx, dy, dx, pad_t, pad_l, K, Kp);
    } else {
        const int64_t total = M * Kp;
        im2col_kernel<1><<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, Ho, Wo, kh, kw, sy, sx, dy, dx, pad_t, pad_l, K, Kp);
    }
    FDK_CUDA(cudaGetLastError());
}

void launch_im2col_transposed(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int kh, int kw,
                              int sy, int sx, int offy, int offx, int pad_t, int pad_l, int Hd, int Wd, int Kp, cudaStream_t s) {
    const int K = kh * kw * C;
    const int64_t total = B * Ho * Wo * Kp;
    if (total == 0) return;
    im2col_transposed_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, Ho, Wo, kh, kw, sy, sx, offy, offx,
                                                                pad_t, pad_l, Hd, Wd, K, Kp);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Depthwise convolution (depthwise_convolution.hpp:21-99): per filter row a row-sum over the filter
// width is added to the bias-initialised output; that order is kept.
// =====================================================================================================
namespace {
// One block per output row (b, oy): all index arithmetic inside the row is 32-bit (64-bit divisions per element
// cost more than the taps).  Consecutive threads take consecutive channel groups of one pixel, then the next
// pixel: every warp access covers whole 128-byte lines, and the taps shared by neighbouring pixels hit in L1.
template <int VEC>
__global__ void __launch_bounds__(256) dwconv_kernel(const float* __restrict__ in, const float* __restrict__ w, float* __restrict__ out,
                                                     int H, int W, int C, int Ho, int Wo, int kh, int kw, int sy, int sx, int pad_t,
                                                     int pad_l, EpiDev epi) {
    const int cv = C / VEC;
    const int64_t row = blockIdx.x;           // b * Ho + oy
    const int oy = (int)(row % Ho);
    const int64_t b = row / Ho;
    const float* in_b = in + b * (int64_t)H * W * C;
    const int per_row = Wo * cv;
    for (int e = threadIdx.x; e < per_row; e += blockDim.x) {
        const int ox = e / cv;
        const int c = (e - ox * cv) * VEC;
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
        for (int ky = 0; ky < kh; ++ky) {
            const int iy = oy * sy + ky - pad_t;
            float rs[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) rs[j] = 0.f;
            if (iy >= 0 && iy < H) {
                const float* in_row = in_b + (int64_t)iy * W * C + c;
                for (int kx = 0; kx < kw; ++kx) {
                    const int ix = ox * sx + kx - pad_l;
                    if (ix < 0 || ix >= W) continue;
                    const float* p = in_row + ix * C;
                    const float* q = w + (ky * kw + kx) * C + c;
                    if (VEC == 4) {
                        const float4 a = *reinterpret_cast<const float4*>(p);
                        const float4 f = __ldg(reinterpret_cast<const float4*>(q));
                        rs[0] = fmaf(a.x, f.x, rs[0]); rs[1 % VEC] = fmaf(a.y, f.y, rs[1 % VEC]);
                        rs[2 % VEC] = fmaf(a.z, f.z, rs[2 % VEC]); rs[3 % VEC] = fmaf(a.w, f.w, rs[3 % VEC]);
                    } else {
                        rs[0] = fmaf(*p, __ldg(q), rs[0]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[j] += rs[j];
        }
        const int64_t m = row * Wo + ox;
        if (VEC == 4) {
            float v[4] = {acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]};
            epi_apply4(epi, v, m, c);
            *reinterpret_cast<float4*>(out + m * C + c) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            out[m * C + c] = epi_apply(epi, acc[0], m, c);
        }
    }
}
}  // namespace

namespace {
// 3 x 3 filters, 4 channels per thread, TR output rows per thread in one column: every input row the thread needs
// is loaded once (three taps) and feeds up to three of its outputs, the nine weight vectors stay in registers.
// Same summation order per output as the general kernel (rows top to bottom, taps left to right inside a row).
template <int S, int TR>
__global__ void __launch_bounds__(256) dwconv3x3_kernel(const float* __restrict__ in, const float* __restrict__ w, float* __restrict__ out,
                                                        int H, int W, int C, int Ho, int Wo, int pad_t, int pad_l, int row_tiles, EpiDev epi) {
    const int cv = C >> 2;
    const int64_t b = blockIdx.x / row_tiles;
    const int oy0 = (int)(blockIdx.x % row_tiles) * TR;
    const float* in_b = in + b * (int64_t)H * W * C;
    const int per_row = Wo * cv;
    for (int e = threadIdx.x; e < per_row; e += blockDim.x) {
        const int ox = e / cv;
        const int c = (e - ox * cv) << 2;
        float4 wv[9];
#pragma unroll
        for (int t = 0; t < 9; ++t) wv[t] = __ldg(reinterpret_cast<const float4*>(w + t * C + c));
        float4 acc[TR];
#pragma unroll
        for (int t = 0; t < TR; ++t) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int ix0 = ox * S - pad_l;
        constexpr int ROWS = (TR - 1) * S + 3;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int iy = oy0 * S - pad_t + r;
            float4 a[3];
#pragma unroll
            for (int kx = 0; kx < 3; ++kx) {
                const int ix = ix0 + kx;
                a[kx] = (iy >= 0 && iy < H && ix >= 0 && ix < W) ? *reinterpret_cast<const float4*>(in_b + ((int64_t)iy * W + ix) * C + c)
                                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int t = 0; t < TR; ++t) {
                const int ky = r - t * S;
                if (ky < 0 || ky > 2) continue;  // compile-time after unrolling
                // taps outside the image are skipped by the general kernel; adding their zeros changes nothing
                float4 rs = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const float4 f = wv[ky * 3 + kx];
                    rs.x = fmaf(a[kx].x, f.x, rs.x); rs.y = fmaf(a[kx].y, f.y, rs.y);
                    rs.z = fmaf(a[kx].z, f.z, rs.z); rs.w = fmaf(a[kx].w, f.w, rs.w);
                }
                acc[t].x += rs.x; acc[t].y += rs.y; acc[t].z += rs.z; acc[t].w += rs.w;
            }
        }
#pragma unroll
        for (int t = 0; t < TR; ++t) {
            const int oy = oy0 + t;
            if (oy >= Ho) break;
            const int64_t m = (b * Ho + oy) * Wo + ox;
            float v[4] = {acc[t].x, acc[t].y, acc[t].z, acc[t].w};
            epi_apply4(epi, v, m, c);
            *reinterpret_cast<float4*>(out + m * C + c) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
}
}  // namespace

void launch_dwconv(const float* in, const float* w, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int kh,
                   int kw, int sy, int sx, int pad_t, int pad_l, const Epilogue& e, cudaStream_t s) {
    const int64_t M = B * Ho * Wo;
    if (M == 0) return;
    const EpiDev epi = to_dev(e);
    const bool vec = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(w) & 15) == 0) &&
                     (e.residual == nullptr || ((e.ldr % 4 == 0) && ((reinterpret_cast<uintptr_t>(e.residual) & 15) == 0)));
    const int64_t rows = B * Ho;
    ensure(rows <= 0x7fffffffLL, "depthwise convolution: too many output rows");
    if (dwconv_tiles_supported(in, w, out, C, kh, kw, sy, sx, e)) {
        launch_dwconv_tiles(in, w, out, B, H, W, C, Ho, Wo, sy, pad_t, pad_l, e, s);
        return;
    }
    if (vec && kh == 3 && kw == 3 && sy == sx && (sy == 1 || sy == 2)) {
        constexpr int TR = 4;
        const int row_tiles = (Ho + TR - 1) / TR;
        const int per = Wo * (C / 4);
        const int th = per >= 256 ? 256 : per >= 128 ? 128 : 64;
        const unsigned grid = (unsigned)(B * row_tiles);
        if (sy == 1) dwconv3x3_kernel<1, TR><<<grid, th, 0, s>>>(in, w, out, H, W, C, Ho, Wo, pad_t, pad_l, row_tiles, epi);
        else dwconv3x3_kernel<2, TR><<<grid, th, 0, s>>>(in, w, out, H, W, C, Ho, Wo, pad_t, pad_l, row_tiles, epi);
        FDK_CUDA(cudaGetLastError());
        return;
    }
    const int per_row = Wo * (vec ? C / 4 : C);
    const int threads = per_row >= 256 ? 256 : per_row >= 128 ? 128 : 64;
    if (vec) dwconv_kernel<4><<<(unsigned)rows, threads, 0, s>>>(in, w, out, H, W, C, Ho, Wo, kh, kw, sy, sx, pad_t, pad_l, epi);
    else dwconv_kernel<1><<<(unsigned)rows, threads, 0, s>>>(in, w, out, H, W, C, Ho, Wo, kh, kw, sy, sx, pad_t, pad_l, epi);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Pooling (pooling_3d_layer.hpp:44-79; max: max_pooling_3d_layer.hpp:17-38; average divides by the number
// of taps inside the tensor: average_pooling_3d_layer.hpp:17-42).
// =====================================================================================================
namespace {
// The input may carry a frame of explicit zeros (a ZeroPadding layer folded into the pooling): the window
// walks the framed tensor of size (D + zf + zb, ...); a tap inside the frame reads 0 and counts as a value,
// a tap outside the framed tensor (SAME padding) is skipped.
struct PoolGeom {
    int D, H, W, C, Do, Ho, Wo, pd, ph, pw, sd, sy, sx, pad_f, pad_t, pad_l;
    int zf, zt, zl, Dz, Hz, Wz;  // zero frame before the data and framed sizes
};
// One block per output row (b, od, oy); 32-bit index arithmetic inside the row.
template <int VEC>
__global__ void __launch_bounds__(256) pool3d_kernel(const float* __restrict__ in, float* __restrict__ out, PoolGeom g, bool is_max) {
    const int cv = g.C / VEC;
    int64_t r = blockIdx.x;
    const int oy = (int)(r % g.Ho); r /= g.Ho;
    const int od = (int)(r % g.Do);
    const int64_t b = r / g.Do;
    const int per_row = g.Wo * cv;
    for (int e = threadIdx.x; e < per_row; e += blockDim.x) {
        const int ox = e / cv;
        const int c = (e - ox * cv) * VEC;
        float val[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) val[j] = is_max ? -FLT_MAX : 0.f;
        int cnt = 0;
        for (int a = 0; a < g.pd; ++a) {
            const int vd = od * g.sd + a - g.pad_f;
            if (vd < 0 || vd >= g.Dz) continue;
            const int id = vd - g.zf;
            for (int ky = 0; ky < g.ph; ++ky) {
                const int vy = oy * g.sy + ky - g.pad_t;
                if (vy < 0 || vy >= g.Hz) continue;
                const int iy = vy - g.zt;
                for (int kx = 0; kx < g.pw; ++kx) {
                    const int vx = ox * g.sx + kx - g.pad_l;
                    if (vx < 0 || vx >= g.Wz) continue;
                    const int ix = vx - g.zl;
                    float cur[VEC];
#pragma unroll
                    for (int j = 0; j < VEC; ++j) cur[j] = 0.f;
                    if (id >= 0 && id < g.D && iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) {
                        const float* p = in + ((((b * g.D + id) * g.H + iy) * g.W + ix) * (int64_t)g.C) + c;
                        if (VEC == 4) {
                            const float4 t = *reinterpret_cast<const float4*>(p);
                            cur[0] = t.x; cur[1 % VEC] = t.y; cur[2 % VEC] = t.z; cur[3 % VEC] = t.w;
                        } else {
                            cur[0] = *p;
                        }
                    }
                    ++cnt;
#pragma unroll
                    for (int j = 0; j < VEC; ++j) val[j] = is_max ? fmaxf(val[j], cur[j]) : val[j] + cur[j];
                }
            }
        }
        float* q = out + (((b * g.Do + od) * g.Ho + oy) * g.Wo + ox) * (int64_t)g.C + c;
        if (!is_max) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) val[j] = val[j] / (float)cnt;
        }
        if (VEC == 4) *reinterpret_cast<float4*>(q) = make_float4(val[0], val[1 % VEC], val[2 % VEC], val[3 % VEC]);
        else q[0] = val[0];
    }
}

// global pooling (global_average_pooling_3d_layer.hpp:25-41): sequential sum in (d4, y, x) order, then
// one division.  One thread per (sample, channel); consecutive threads read consecutive channels.
__global__ void global_pool_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t B, int64_t spatial, int C,
                                   bool is_max) {
    const int64_t total = B * C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int64_t b = i / C;
        const float* p = in + b * spatial * C + c;
        float val = is_max ? -FLT_MAX : 0.f;
        for (int64_t sidx = 0; sidx < spatial; ++sidx) {
            const float cur = p[sidx * C];
            val = is_max ? fmaxf(val, cur) : val + cur;
        }
        out[i] = is_max ? val : val / (float)spatial;
    }
}
}  // namespace

void launch_pool3d(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo, int pd, int ph,
                   int pw, int sd, int sy, int sx, int pad_f, int pad_t, int pad_l, const int* zero_frame, bool is_max, cudaStream_t s) {
    if (B * Do * Ho * Wo * C == 0) return;
    PoolGeom g{D, H, W, C, Do, Ho, Wo, pd, ph, pw, sd, sy, sx, pad_f, pad_t, pad_l, 0, 0, 0, D, H, W};
    if (zero_frame) {  // front, back, top, bottom, left, right
        g.zf = zero_frame[0]; g.zt = zero_frame[2]; g.zl = zero_frame[4];
        g.Dz = D + zero_frame[0] + zero_frame[1]; g.Hz = H + zero_frame[2] + zero_frame[3]; g.Wz = W + zero_frame[4] + zero_frame[5];
    }
    if (D == 1 && Do == 1 && pd == 1 && g.zf == 0 && g.Dz == 1 && pad_f == 0 &&
        pool_tiles_supported(in, out, C, g.Hz, g.Wz, Ho, Wo, ph, pw, sy, sx, pad_t, pad_l)) {
        launch_pool_tiles(in, out, B, H, W, C, Ho, Wo, ph, sy, g.zt, g.zl, is_max, s);
        return;
    }
    const bool vec = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    const int64_t rows = B * Do * Ho;
    ensure(rows <= 0x7fffffffLL, "pooling: too many output rows");
    const int per_row = Wo * (vec ? C / 4 : C);
    const int threads = per_row >= 256 ? 256 : per_row >= 128 ? 128 : 64;
    if (vec) pool3d_kernel<4><<<(unsigned)rows, threads, 0, s>>>(in, out, g, is_max);
    else pool3d_kernel<1><<<(unsigned)rows, threads, 0, s>>>(in, out, g, is_max);
    FDK_CUDA(cudaGetLastError());
}
void launch_global_pool(const float* in, float* out, int64_t B, int64_t spatial, int C, bool is_max, cudaStream_t s) {
    if (B * C == 0) return;
    global_pool_kernel<<<grid_1d(B * C, 128), 128, 0, s>>>(in, out, B, spatial, C, is_max);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Elementwise merge with broadcasting (elem_wise_combine_tensors, tensor.hpp:642-660), unary activations
// (transform_tensor, tensor.hpp:190-196) and the per-channel affine form of batch_normalization
// (tensor.hpp:773-793).
// =====================================================================================================
namespace {
struct Dims5 { int64_t d[5]; };

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
    switch (op) {
        case BIN_ADD: return a + b;
        case BIN_SUB: return a - b;
        case BIN_MUL: return a * b;
        case BIN_MAX: return fmaxf(a, b);
        default: return fminf(a, b);
    }
}
__global__ void binary_same_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                   int64_t n4, int64_t n, float post_scale, ActSpecDev act) {
    pdl_launch_dependents();
    pdl_wait();
    const bool scale = post_scale != 1.0f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 x = __ldcg(reinterpret_cast<const float4*>(a) + i);
        const float4 y = __ldcg(reinterpret_cast<const float4*>(b) + i);
        float4 r;
        r.x = bin_apply(op, x.x, y.x); r.y = bin_apply(op, x.y, y.y); r.z = bin_apply(op, x.z, y.z); r.w = bin_apply(op, x.w, y.w);
        if (scale) { r.x *= post_scale; r.y *= post_scale; r.z *= post_scale; r.w *= post_scale; }
        r.x = act_apply(act, r.x); r.y = act_apply(act, r.y); r.z = act_apply(act, r.z); r.w = act_apply(act, r.w);
        reinterpret_cast<float4*>(out)[i] = r;
    }
    // tail
    const int64_t start = n4 * 4;
    for (int64_t i = start + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float r = bin_apply(op, __ldcg(a + i), __ldcg(b + i));
        if (scale) r *= post_scale;
        out[i] = act_apply(act, r);
    }
}
__global__ void binary_bcast_kernel(int op, const float* __restrict__ a, Dims5 ad, const float* __restrict__ b, Dims5 bd,
                                    float* __restrict__ out, Dims5 od, int64_t total, float post_scale, ActSpecDev act) {
    const int64_t ovol = od.d[0] * od.d[1] * od.d[2] * od.d[3] * od.d[4];
    const int64_t avol = ad.d[0] * ad.d[1] * ad.d[2] * ad.d[3] * ad.d[4];
    const int64_t bvol = bd.d[0] * bd.d[1] * bd.d[2] * bd.d[3] * bd.d[4];
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t smp = i / ovol;
        int64_t r = i % ovol;
        int64_t p[5];
#pragma unroll
        for (int k = 4; k >= 0; --k) { p[k] = r % od.d[k]; r /= od.d[k]; }
        int64_t ia = 0, ib = 0;
#pragma unroll
        for (int k = 0; k < 5; ++k) { ia = ia * ad.d[k] + (p[k] % ad.d[k]); ib = ib * bd.d[k] + (p[k] % bd.d[k]); }
        float v = bin_apply(op, a[smp * avol + ia], b[smp * bvol + ib]);
        if (post_scale != 1.0f) v *= post_scale;
        out[i] = act_apply(act, v);
    }
}
__global__ void unary_kernel(ActSpecDev act, const float* __restrict__ in, float* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = act_apply(act, in[i]);
}
__global__ void affine_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ scale,
                              const float* __restrict__ shift, int64_t total, int64_t nc, int64_t inner, ActSpecDev act) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = (i / inner) % nc;
        // x * inv + (beta - mean * inv): two roundings, like the reference (tensor.hpp:788-792)
        out[i] = act_apply(act, __fadd_rn(__fmul_rn(in[i], scale[c]), shift[c]));
    }
}
__global__ void scale_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n, float f) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = in[i] * f;
}
__global__ void fill_kernel(float* p, float v, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}
}  // namespace

void launch_binary(int op, const float* a, const int64_t* adims, const float* b, const int64_t* bdims, float* out,
                   const int64_t* odims, int64_t B, float post_scale, ActSpec act, cudaStream_t s) {
    Dims5 ad, bd, od;
    bool same = true;
    int64_t vol = 1;
    for (int i = 0; i < 5; ++i) {
        ad.d[i] = adims[i]; bd.d[i] = bdims[i]; od.d[i] = odims[i];
        if (adims[i] != odims[i] || bdims[i] != odims[i]) same = false;
        vol *= odims[i];
    }
    const int64_t total = B * vol;
    if (total == 0) return;
    const ActSpecDev ad_act = to_dev(act);
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (same && aligned) {
        const int64_t n4 = total / 4;
        launch_pdl(binary_same_kernel, dim3(grid_1d(n4 > 0 ? n4 : 1, 256)), dim3(256), 0, s, op, a, b, out, n4, total, post_scale, ad_act);
    } else {
        binary_bcast_kernel<<<grid_1d(total, 256), 256, 0, s>>>(op, a, ad, b, bd, out, od, total, post_scale, ad_act);
    }
    FDK_CUDA(cudaGetLastError());
}
void launch_unary(ActSpec act, const float* in, float* out, int64_t n, cudaStream_t s) {
    if (n == 0) return;
    unary_kernel<<<grid_1d(n, 256), 256, 0, s>>>(to_dev(act), in, out, n);
    FDK_CUDA(cudaGetLastError());
}
void launch_affine(const float* in, float* out, const float* scale, const float* shift, int64_t outer, int64_t nc,
                   int64_t inner, ActSpec act, cudaStream_t s) {
    const int64_t total = outer * nc * inner;
    if (total == 0) return;
    affine_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, scale, shift, total, nc, inner, to_dev(act));
    FDK_CUDA(cudaGetLastError());
}
void launch_scale(const float* in, float* out, int64_t n, float f, cudaStream_t s) {
    if (n == 0) return;
    scale_kernel<<<grid_1d(n, 256), 256, 0, s>>>(in, out, n, f);
    FDK_CUDA(cudaGetLastError());
}
void launch_fill(float* p, float v, int64_t n, cudaStream_t s) {
    if (n == 0) return;
    fill_kernel<<<grid_1d(n, 256), 256, 0, s>>>(p, v, n);
    FDK_CUDA(cudaGetLastError());
}

// A decode loop recorded as a CUDA graph keeps its position in device memory: the same launches serve every position.
namespace {
__global__ void fill_from_counter_kernel(float* __restrict__ p, const int* __restrict__ counter, int64_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const float v = (float)__ldcg(counter);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void counter_add_kernel(int* counter, int delta) {
    pdl_launch_dependents();
    pdl_wait();
    atomicAdd(counter, delta);
}
}  // namespace
void launch_fill_from_counter(float* p, const int* counter, int64_t n, cudaStream_t s) {
    if (n == 0) return;
    launch_pdl(fill_from_counter_kernel, dim3(grid_1d(n, 256)), dim3(256), 0, s, p, counter, n);
}
void launch_counter_add(int* counter, int delta, cudaStream_t s) {
    launch_pdl(counter_add_kernel, dim3(1), dim3(1), 0, s, counter, delta);
}

// =====================================================================================================
// Softmax along depth (tensor.hpp:1165-1192): m = max, s = sum exp(x - m), y = exp(x - m - log s),
// inf -> 0.  One warp per row; sums are formed lane-strided then reduced, the reference sums sequentially.
// =====================================================================================================
namespace {
__global__ void softmax_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows_total, int64_t rows_per_sample,
                               int64_t valid_rows, int depth, bool log_form) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row = warp; row < rows_total; row += nwarps) {
        const float* p = in + row * depth;
        float* q = out + row * depth;
        if (row % rows_per_sample >= valid_rows) {
            for (int z = lane; z < depth; z += 32) q[z] = 0.f;
            continue;
        }
        float m = -FLT_MAX;
        for (int z = lane; z < depth; z += 32) m = fmaxf(m, p[z]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float sum = 0.f;
        for (int z = lane; z < depth; z += 32) sum += expf(p[z] - m);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float ls = logf(sum);
        for (int z = lane; z < depth; z += 32) {
            if (log_form) q[z] = p[z] - m - ls;
            else {
                const float r = expf(p[z] - m - ls);
                q[z] = isinf(r) ? 0.f : r;
            }
        }
    }
}

// Layer normalisation over the last axis (layer_normalization_layer.hpp:37-63; moments tensor.hpp:758-771):
// mean = sum / n; var = sum((|x - mean|)^2) / n; y = x * inv + (beta - mean * inv), inv = gamma / sqrt(var + eps).
// RMS form (rms_normalization_layer.hpp:35-69): y = x / sqrt(mean(x^2) + eps) * gamma.
// mode 0: layer normalisation; 1: RMS normalisation; 2: unit (L2) normalisation (l2_normalize, tensor.hpp:801-812:
// x / sqrt(max(sum x^2, machine epsilon))).
// CACHED: rows of at most 1024 values are read once into registers (all loads of a row in flight together; the sums
// run over the same values in the same order as in the streaming form, so both give the same bits).
template <bool CACHED>
__global__ void layernorm_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ gamma,
                                 const float* __restrict__ beta, int64_t rows, int n, float eps, int mode) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const float* p = in + row * n;
        float* q = out + row * n;
        float v[CACHED ? 32 : 1];
        if (CACHED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[CACHED ? i : 0] = lane + 32 * i < n ? p[lane + 32 * i] : 0.f;
        }
        auto at = [&](int i, int z) { return CACHED ? v[CACHED ? i : 0] : p[z]; };
        const int iters = (n - lane + 31) / 32;  // values of this lane: z = lane + 32 i, i < iters
        if (mode != 0) {
            float ss = 0.f;
            if (CACHED) {
#pragma unroll
                for (int i = 0; i < 32; ++i) if (i < iters) ss += at(i, 0) * at(i, 0);
            } else {
                for (int z = lane; z < n; z += 32) ss += p[z] * p[z];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = mode == 1 ? 1.0f / sqrtf(ss / (float)n + eps) : 1.0f / sqrtf(fmaxf(ss, FLT_EPSILON));
            if (CACHED) {
#pragma unroll
                for (int i = 0; i < 32; ++i) if (i < iters) q[lane + 32 * i] = at(i, 0) * inv * (gamma ? gamma[lane + 32 * i] : 1.0f);
            } else {
                for (int z = lane; z < n; z += 32) q[z] = p[z] * inv * (gamma ? gamma[z] : 1.0f);
            }
            continue;
        }
        float sum = 0.f;
        if (CACHED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (i < iters) sum += at(i, 0);
        } else {
            for (int z = lane; z < n; z += 32) sum += p[z];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum / (float)n;
        float var = 0.f;
        if (CACHED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (i < iters) { const float d = fabsf(at(i, 0) - mean); var += d * d; }
        } else {
            for (int z = lane; z < n; z += 32) { const float d = fabsf(p[z] - mean); var += d * d; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
        var = var / (float)n;
        const float rstd = 1.0f / sqrtf(var + eps);
        if (CACHED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i < iters) {
                    const int z = lane + 32 * i;
                    const float inv = rstd * (gamma ? gamma[z] : 1.0f);
                    const float off = (beta ? beta[z] : 0.0f) - __fmul_rn(mean, inv);
                    q[z] = __fadd_rn(__fmul_rn(at(i, 0), inv), off);
                }
            }
        } else {
            for (int z = lane; z < n; z += 32) {
                const float inv = rstd * (gamma ? gamma[z] : 1.0f);
                const float off = (beta ? beta[z] : 0.0f) - __fmul_rn(mean, inv);
                q[z] = __fadd_rn(__fmul_rn(p[z], inv), off);
            }
        }
    }
}
}  // namespace

void launch_softmax(const float* in, float* out, int64_t B, int64_t rows_per_sample, int64_t valid_rows, int depth,
                    bool log_form, cudaStream_t s) {
    const int64_t rows = B * rows_per_sample;
    if (rows == 0 || depth == 0) return;
    softmax_kernel<<<grid_1d(rows * 32, 256), 256, 0, s>>>(in, out, rows, rows_per_sample, valid_rows, depth, log_form);
    FDK_CUDA(cudaGetLastError());
}
// Layer normalisation of short rows with 16-byte loads: a warp per row, NV float4 per lane (n <= 128 NV, n % 4 == 0),
// the row held in registers.  Compact on purpose: a warp runs through this code once, so its length is paid in
// instruction fetch; the scalar kernels above stay for long or unaligned rows and for the RMS / unit forms.
namespace {
template <int NV>
__global__ void layernorm_rows4_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ gamma,
                                       const float* __restrict__ beta, int64_t rows, int n, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    const float4* p = reinterpret_cast<const float4*>(in + row * n);
    float4* q = reinterpret_cast<float4*>(out + row * n);
    const int n4 = n >> 2;
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < n4 ? __ldcg(p + lane + 32 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)n;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < n4) {
            const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
            var += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float rstd = 1.0f / sqrtf(var / (float)n + eps);
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f), zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int z = lane + 32 * i;
        if (z < n4) {
            const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + z) : one;
            const float4 b = beta ? __ldg(reinterpret_cast<const float4*>(beta) + z) : zero;
            float4 y;
            // y = x * inv + (beta - mean * inv), inv = gamma / sqrt(var + eps), each step rounded (tensor.hpp:788-792)
            float inv = rstd * g.x; y.x = __fadd_rn(__fmul_rn(v[i].x, inv), b.x - __fmul_rn(mean, inv));
            inv = rstd * g.y; y.y = __fadd_rn(__fmul_rn(v[i].y, inv), b.y - __fmul_rn(mean, inv));
            inv = rstd * g.z; y.z = __fadd_rn(__fmul_rn(v[i].z, inv), b.z - __fmul_rn(mean, inv));
            inv = rstd * g.w; y.w = __fadd_rn(__fmul_rn(v[i].w, inv), b.w - __fmul_rn(mean, inv));
            q[z] = y;
        }
    }
}
template <int NV>
void launch_layernorm_rows4(const float* in, float* out, const float* gamma, const float* beta, int64_t rows, int n, float eps, cudaStream_t s) {
    const int block = rows <= 4096 ? 64 : 256;   // few rows (one decode position): small blocks, rows spread over many SMs
    const int64_t blocks = (rows * 32 + block - 1) / block;
    launch_pdl(layernorm_rows4_kernel<NV>, dim3((unsigned)blocks), dim3((unsigned)block), 0, s, in, out, gamma, beta, rows, n, eps);
}
bool aligned16_ln(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

void launch_layernorm(const float* in, float* out, const float* gamma, const float* beta, int64_t rows, int n, float eps,
                      int mode, cudaStream_t s) {
    if (rows == 0 || n == 0) return;
    if (mode == 0 && n % 4 == 0 && n <= 1024 && rows * 32 / 64 < (1LL << 31) && aligned16_ln(in) && aligned16_ln(out) && aligned16_ln(gamma) &&
        aligned16_ln(beta)) {
        const int nv = (n / 4 + 31) / 32;
        if (nv <= 2) launch_layernorm_rows4<2>(in, out, gamma, beta, rows, n, eps, s);
        else if (nv <= 4) launch_layernorm_rows4<4>(in, out, gamma, beta, rows, n, eps, s);
        else if (nv <= 6) launch_layernorm_rows4<6>(in, out, gamma, beta, rows, n, eps, s);
        else launch_layernorm_rows4<8>(in, out, gamma, beta, rows, n, eps, s);
        FDK_CUDA(cudaGetLastError());
        return;
    }
    // few rows (one decode position): small blocks, so that the rows spread over many SMs
    const int block = rows <= 4096 ? 64 : 256;
    if (n <= 1024) layernorm_kernel<true><<<grid_1d(rows * 32, block), block, 0, s>>>(in, out, gamma, beta, rows, n, eps, mode);
    else layernorm_kernel<false><<<grid_1d(rows * 32, block), block, 0, s>>>(in, out, gamma, beta, rows, n, eps, mode);
    FDK_CUDA(cudaGetLastError());
}

// Group normalisation over the channel axis (group_normalization_layer.hpp:36-98): one block per (sample, group);
// mean, then variance around it, then (x - mean) * inv_std * gamma[c] + beta[c].
namespace {
__device__ __forceinline__ float block_sum_256(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = threadIdx.x < 8 ? sh[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) sh[8] = t;
    }
    __syncthreads();
    const float r = sh[8];
    __syncthreads();
    return r;
}
__global__ void __launch_bounds__(256) groupnorm_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ gamma,
                                                        const float* __restrict__ beta, int64_t spatial, int C, int groups, float eps) {
    __shared__ float sh[9];
    const int g = blockIdx.x % groups;
    const int64_t b = blockIdx.x / groups;
    const int cpg = C / groups;
    const float* p = in + b * spatial * C + g * cpg;
    float* q = out + b * spatial * C + g * cpg;
    const int64_t n = spatial * cpg;
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += 256) sum += p[(i / cpg) * C + (i % cpg)];
    const float mean = block_sum_256(sum, sh) / (float)n;
    float var = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += 256) { const float d = p[(i / cpg) * C + (i % cpg)] - mean; var += d * d; }
    const float inv = 1.0f / sqrtf(block_sum_256(var, sh) / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += 256) {
        const int cc = (int)(i % cpg);
        const int64_t off = (i / cpg) * C + cc;
        float v = (p[off] - mean) * inv;
        if (gamma) v *= gamma[g * cpg + cc];
        if (beta) v += beta[g * cpg + cc];
        q[off] = v;
    }
}
}  // namespace
void launch_groupnorm(const float* in, float* out, const float* gamma, const float* beta, int64_t B, int64_t spatial, int C, int groups,
                      float eps, cudaStream_t s) {
    if (B * spatial * C == 0) return;
    groupnorm_kernel<<<(unsigned)(B * groups), 256, 0, s>>>(in, out, gamma, beta, spatial, C, groups, eps);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Data movement: window copy (pad_tensor tensor.hpp:490-517 / crop_tensor), slab copy for concatenation
// (tensor.hpp:320-483), permutation (permute_tensor), embedding gather (embedding_layer.hpp:31-57).
// =====================================================================================================
namespace {
__global__ void window_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int D, int H, int W, int C,
                              int Do, int Ho, int Wo, int off_d, int off_y, int off_x) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        int64_t r = i / C;
        const int x = (int)(r % Wo); r /= Wo;
        const int y = (int)(r % Ho); r /= Ho;
        const int d = (int)(r % Do);
        const int64_t b = r / Do;
        const int id = d - off_d, iy = y - off_y, ix = x - off_x;
        float v = 0.f;
        if (id >= 0 && id < D && iy >= 0 && iy < H && ix >= 0 && ix < W) v = in[((((b * D + id) * H + iy) * W + ix) * (int64_t)C) + c];
        out[i] = v;
    }
}
__global__ void slab_copy_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int64_t in_len,
                                 int64_t out_len, int64_t off) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / in_len, j = i % in_len;
        out[o * out_len + off + j] = in[i];
    }
}
struct Perm5 { int p[5]; };
__global__ void permute_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, Dims5 id, Dims5 od, Perm5 perm) {
    const int64_t vol = od.d[0] * od.d[1] * od.d[2] * od.d[3] * od.d[4];
    int64_t istr[5];
    istr[4] = 1;
#pragma unroll
    for (int k = 3; k >= 0; --k) istr[k] = istr[k + 1] * id.d[k + 1];
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t smp = i / vol;
        int64_t r = i % vol;
        int64_t src = 0;
#pragma unroll
        for (int k = 4; k >= 0; --k) { const int64_t pk = r % od.d[k]; r /= od.d[k]; src += pk * istr[perm.p[k]]; }
        out[i] = in[smp * vol + src];
    }
}
__global__ void embedding_kernel(const float* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out,
                                 int64_t total, int dim, int64_t input_dim, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / dim;
        const int j = (int)(i % dim);
        const float f = __ldcg(ids + row);
        const int64_t id = (int64_t)f;  // truncation like static_cast<std::size_t> for non-negative ids
        if (!(f >= 0.f) || id >= input_dim) {
            if (j == 0) atomicExch(err, 1);
            out[i] = 0.f;
        } else {
            out[i] = table[id * dim + j];
        }
    }
}
}  // namespace

void launch_window(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo, int off_d,
                   int off_y, int off_x, cudaStream_t s) {
    const int64_t total = B * Do * Ho * Wo * C;
    if (total == 0) return;
    window_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, D, H, W, C, Do, Ho, Wo, off_d, off_y, off_x);
    FDK_CUDA(cudaGetLastError());
}
namespace {
// out[b, y, x, 0..Cp) = in[b, y - pad_t, x - pad_l, 0..C) padded with zeros in space and in the channels;
// one thread per output pixel (Cp <= 8 in practice: first layers of vision models)
__global__ void pad_channels_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int H, int W, int C, int Hp,
                                    int Wp, int Cp, int pad_t, int pad_l) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % Wp);
        const int y = (int)((i / Wp) % Hp);
        const int64_t b = i / ((int64_t)Wp * Hp);
        const int iy = y - pad_t, ix = x - pad_l;
        const bool inside = iy >= 0 && iy < H && ix >= 0 && ix < W;
        const float* p = in + ((b * H + iy) * W + ix) * (int64_t)C;
        float* q = out + i * Cp;
        for (int c = 0; c < Cp; ++c) q[c] = (inside && c < C) ? p[c] : 0.f;
    }
}
}  // namespace

void launch_pad_channels(const float* in, float* out, int64_t B, int H, int W, int C, int Hp, int Wp, int Cp, int pad_t, int pad_l,
                         cudaStream_t s) {
    const int64_t total = B * Hp * Wp;
    if (total == 0) return;
    pad_channels_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, Hp, Wp, Cp, pad_t, pad_l);
    FDK_CUDA(cudaGetLastError());
}
void launch_slab_copy(const float* in, float* out, int64_t outer, int64_t in_len, int64_t out_len, int64_t off, cudaStream_t s) {
    const int64_t total = outer * in_len;
    if (total == 0) return;
    slab_copy_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, in_len, out_len, off);
    FDK_CUDA(cudaGetLastError());
}
void launch_permute(const float* in, float* out, int64_t B, const int64_t* in_dims, const int* perm, cudaStream_t s) {
    Dims5 id, od;
    Perm5 pp;
    int64_t vol = 1;
    for (int i = 0; i < 5; ++i) { id.d[i] = in_dims[i]; pp.p[i] = perm[i]; vol *= in_dims[i]; }
    for (int i = 0; i < 5; ++i) od.d[i] = in_dims[perm[i]];
    const int64_t total = B * vol;
    if (total == 0) return;
    permute_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, id, od, pp);
    FDK_CUDA(cudaGetLastError());
}
void launch_embedding(const float* ids, const float* table, float* out, int64_t n_ids, int dim, int64_t input_dim, int* err,
                      cudaStream_t s) {
    const int64_t total = n_ids * dim;
    if (total == 0) return;
    launch_pdl(embedding_kernel, dim3(grid_1d(total, 256)), dim3(256), 0, s, ids, table, out, total, dim, input_dim, err);
}

// =====================================================================================================
// Recurrent cells (recurrent_ops.hpp:164-181 LSTM, :262-275 GRU reset_after).
// =====================================================================================================
namespace {
__global__ void lstm_cell_kernel(const float* __restrict__ z, float* __restrict__ c, float* __restrict__ h, float* __restrict__ out,
                                 int64_t out_stride, int64_t total, int U, ActSpecDev act, ActSpecDev ract) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / U;
        const int j = (int)(i % U);
        const float* zr = z + b * 4 * (int64_t)U;
        const float ig = act_apply(ract, zr[j]);
        const float fg = act_apply(ract, zr[U + j]);
        const float cp = act_apply(act, zr[2 * U + j]);
        const float og = act_apply(ract, zr[3 * U + j]);
        // c = f * c + i * c~ as two products and one sum, h = o * act(c)
        const float cn = __fadd_rn(__fmul_rn(fg, c[i]), __fmul_rn(ig, cp));
        const float hn = __fmul_rn(og, act_apply(act, cn));
        c[i] = cn;
        h[i] = hn;
        if (out) out[b * out_stride + j] = hn;
    }
}
// The usual activations (tanh, sigmoid), V = 4 or 2 units per thread with 16- or 8-byte accesses and 32-bit index
// arithmetic; the libdevice calls are those act_apply makes for these kinds, inlined (same results, a third of the
// instructions).  The kernel is bound by instruction issue (about 120 per unit), so what counts is how evenly the
// threads fill the last wave: the launcher picks V by that.
__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
template <int V>
struct CellVec;
template <>
struct CellVec<4> { using type = float4; };
template <>
struct CellVec<2> { using type = float2; };
template <int V>
__global__ void __launch_bounds__(256) lstm_cellv_kernel(const float* __restrict__ z, float* __restrict__ c, float* __restrict__ h,
                                                         float* __restrict__ out, int64_t out_stride, int total_v, int Uv) {
    using Vec = typename CellVec<V>::type;
    // launched with programmatic stream serialisation: the next time step's product may set itself up (and fetch its
    // weights) while this kernel runs; it reads h only after its own wait
    pdl_launch_dependents();
    pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total_v; i += gridDim.x * blockDim.x) {
        const int b = i / Uv;
        const int j = i - b * Uv;
        const Vec* zr = reinterpret_cast<const Vec*>(z) + (int64_t)b * 4 * Uv;
        const Vec zi = zr[j], zf = zr[Uv + j], zc = zr[2 * Uv + j], zo = zr[3 * Uv + j];
        const Vec cv = reinterpret_cast<const Vec*>(c)[i];
        Vec cn, hn;
#define FDK_LSTM_UNIT(f)                                                                          \
        cn.f = __fadd_rn(__fmul_rn(sigmoid_ref(zf.f), cv.f), __fmul_rn(sigmoid_ref(zi.f), tanhf(zc.f))); \
        hn.f = __fmul_rn(sigmoid_ref(zo.f), tanhf(cn.f));
        FDK_LSTM_UNIT(x) FDK_LSTM_UNIT(y)
        if constexpr (V == 4) { FDK_LSTM_UNIT(z) FDK_LSTM_UNIT(w) }
#undef FDK_LSTM_UNIT
        reinterpret_cast<Vec*>(c)[i] = cn;
        reinterpret_cast<Vec*>(h)[i] = hn;
        if (out) *reinterpret_cast<Vec*>(out + (int64_t)b * out_stride + V * j) = hn;
    }
}
__global__ void gru_cell_kernel(const float* __restrict__ xw, int64_t ldx, const float* __restrict__ hu, float* __restrict__ h,
                                float* __restrict__ out, int64_t out_stride, int64_t total, int U, ActSpecDev act, ActSpecDev ract) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / U;
        const int j = (int)(i % U);
        const float* x = xw + b * ldx;
        const float* u = hu + b * 3 * (int64_t)U;
        const float zg = act_apply(ract, x[j] + u[j]);
        const float rg = act_apply(ract, x[U + j] + u[U + j]);
        const float m = act_apply(act, __fadd_rn(x[2 * U + j], __fmul_rn(rg, u[2 * U + j])));
        const float hn = __fadd_rn(__fmul_rn(1.0f - zg, m), __fmul_rn(zg, h[i]));
        h[i] = hn;
        if (out) out[b * out_stride + j] = hn;
    }
}
// GRU with reset_after = false (recurrent_ops.hpp:267-271), first half of a step: hu holds h U_z | h U_r per sample;
// it is overwritten with z | r .* h (the second product's input).
__global__ void gru_gates_kernel(const float* __restrict__ xw, int64_t ldx, float* __restrict__ hu, int64_t ldh, const float* __restrict__ h,
                                 int64_t total, int U, ActSpecDev ract) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / U;
        const int j = (int)(i % U);
        const float* x = xw + b * ldx;
        float* u = hu + b * ldh;
        const float zg = act_apply(ract, x[j] + u[j]);
        const float rg = act_apply(ract, x[U + j] + u[U + j]);
        u[j] = zg;
        u[U + j] = rg * h[i];
    }
}
// second half: m = act(x W_h + b + (r .* h) U_h), h' = (1 - z) m + z h
__global__ void gru_out_kernel(const float* __restrict__ xw, int64_t ldx, const float* __restrict__ zr, int64_t ldh, float* __restrict__ h,
                               float* __restrict__ out, int64_t out_stride, int64_t total, int U, ActSpecDev act) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / U;
        const int j = (int)(i % U);
        const float* u = zr + b * ldh;
        const float zg = u[j];
        const float m = act_apply(act, xw[b * ldx + 2 * U + j] + u[2 * U + j]);
        const float hn = __fadd_rn(__fmul_rn(1.0f - zg, m), __fmul_rn(zg, h[i]));
        h[i] = hn;
        if (out) out[b * out_stride + j] = hn;
    }
}
}  // namespace

void launch_gru_gates(const float* xw, int64_t ldx, float* hu, int64_t ldh, const float* h, int64_t B, int U, ActSpec ract, cudaStream_t s) {
    const int64_t total = B * U;
    if (total == 0) return;
    gru_gates_kernel<<<grid_1d(total, 256), 256, 0, s>>>(xw, ldx, hu, ldh, h, total, U, to_dev(ract));
    FDK_CUDA(cudaGetLastError());
}
void launch_gru_out(const float* xw, int64_t ldx, const float* zr, int64_t ldh, float* h, float* out, int64_t out_stride, int64_t B, int U,
                    ActSpec act, cudaStream_t s) {
    const int64_t total = B * U;
    if (total == 0) return;
    gru_out_kernel<<<grid_1d(total, 256), 256, 0, s>>>(xw, ldx, zr, ldh, h, out, out_stride, total, U, to_dev(act));
    FDK_CUDA(cudaGetLastError());
}

void launch_lstm_cell(const float* z, float* c, float* h, float* out, int64_t out_stride, int64_t B, int U, ActSpec act,
                      ActSpec ract, cudaStream_t s) {
    const int64_t total = B * U;
    if (total == 0) return;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (act.kind == ACT_TANH && ract.kind == ACT_SIGMOID && U % 4 == 0 && total / 4 < 0x7fffffffLL && al16(z) && al16(c) && al16(h) &&
        (out == nullptr || (al16(out) && out_stride % 4 == 0))) {
        // share of the last wave's thread slots that do work (6 blocks of 256 threads per SM at 40 registers)
        auto fill = [&](int64_t threads) {
            const double waves = (double)threads / (148.0 * 1536.0);
            return waves / std::ceil(waves);
        };
        if (fill(total / 2) > fill(total / 4) + 0.05)
            launch_pdl(lstm_cellv_kernel<2>, dim3(grid_1d(total / 2, 256)), dim3(256), 0, s, z, c, h, out, out_stride, (int)(total / 2), U / 2);
        else
            launch_pdl(lstm_cellv_kernel<4>, dim3(grid_1d(total / 4, 256)), dim3(256), 0, s, z, c, h, out, out_stride, (int)(total / 4), U / 4);
        return;
    }
    lstm_cell_kernel<<<grid_1d(total, 256), 256, 0, s>>>(z, c, h, out, out_stride, total, U, to_dev(act), to_dev(ract));
    FDK_CUDA(cudaGetLastError());
}
void launch_gru_cell(const float* xw, int64_t ldx, const float* hu, float* h, float* out, int64_t out_stride, int64_t B, int U,
                     ActSpec act, ActSpec ract, cudaStream_t s) {
    const int64_t total = B * U;
    if (total == 0) return;
    gru_cell_kernel<<<grid_1d(total, 256), 256, 0, s>>>(xw, ldx, hu, h, out, out_stride, total, U, to_dev(act), to_dev(ract));
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Attention core (multi_head_attention_layer.hpp:74-95): per head softmax((q k^T) * scale) v, with the
// reference's softmax form.  One block per (sample, head, query row); scores live in shared memory.
// =====================================================================================================
namespace {
__global__ void attention_kernel(const float* __restrict__ q, int64_t ldq, int64_t q_bs, const float* k, int64_t ldk,
                                 int64_t k_bs, const float* v, int64_t ldv, int64_t v_bs, float* __restrict__ out,
                                 int64_t ldo, int64_t o_bs, int H, int Tq, int Tk, int dk, int dv, float scale, AttnExtra x) {
    extern __shared__ float sm[];
    // cache with its length on the device: row `fresh` comes from this position's projections and enters the cache here
    int fresh = -1;
    if (x.len_ptr) {
        fresh = min(*x.len_ptr, Tk - 1);
        Tk = fresh + 1;
    }
    float* sc = sm;            // Tk scores
    float* qs = sm + Tk;       // dk query values
    __shared__ float red[32];
    const int tq = blockIdx.x % Tq;
    const int h = (blockIdx.x / Tq) % H;
    const int64_t b = blockIdx.x / ((int64_t)Tq * H);
    const float* qp = q + b * q_bs + (int64_t)tq * ldq + (int64_t)h * dk;
    for (int d = threadIdx.x; d < dk; d += blockDim.x) qs[d] = qp[d];
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    // scores: one warp per key row, lanes stride over the head dimension
    const int hk = h / x.group;  // grouped queries: several query heads read one key/value head
    const float* kbase = k + b * k_bs + (int64_t)hk * dk;
    const float* kfresh = fresh >= 0 ? x.k_new + b * ldk + (int64_t)hk * dk : nullptr;
    if (x.mode == ATTN_DOT) {
        // four key rows per warp and turn, their loads in flight together
        for (int t0 = wid * 4; t0 < Tk; t0 += nw * 4) {
            const float* kp[4];
            float s[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = min(t0 + u, Tk - 1);
                kp[u] = t == fresh ? kfresh : kbase + (int64_t)t * ldk;
                s[u] = 0.f;
            }
            for (int d = lane; d < dk; d += 32) {
                const float qd = qs[d];
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] = fmaf(qd, kp[u][d], s[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
                if (lane == 0 && t0 + u < Tk) sc[t0 + u] = s[u] * scale;
            }
        }
        if (fresh >= 0 && wid == 0) {
            float* kc = const_cast<float*>(kbase) + (int64_t)fresh * ldk;
            for (int d = lane; d < dk; d += 32) kc[d] = kfresh[d];
        }
    } else {
        for (int t = wid; t < Tk; t += nw) {
            const float* kp = kbase + (int64_t)t * ldk;
            float s = 0.f;
            if (x.mode == ATTN_CONCAT) {
                for (int d = lane; d < dk; d += 32) s += tanhf(scale * (qs[d] + kp[d]));
            } else {
                for (int d = lane; d < dk; d += 32) s = fmaf(x.svec ? x.svec[x.sn == 1 ? 0 : d] : 1.f, tanhf(qs[d] + kp[d]), s);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) sc[t] = x.mode == ATTN_CONCAT ? s * x.w2 : s;
        }
    }
    __syncthreads();
    float m = -FLT_MAX;
    for (int t = threadIdx.x; t < Tk; t += blockDim.x) m = fmaxf(m, sc[t]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[wid] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nw; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int t = threadIdx.x; t < Tk; t += blockDim.x) sum += expf(sc[t] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[wid] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < nw; ++w) sum += red[w];
    const float ls = logf(sum);
    __syncthreads();
    for (int t = threadIdx.x; t < Tk; t += blockDim.x) {
        const float r = expf(sc[t] - m - ls);
        sc[t] = isinf(r) ? 0.f : r;
    }
    __syncthreads();
    float* op = out + b * o_bs + (int64_t)tq * ldo + (int64_t)h * dv;
    const float* gp = x.gate ? x.gate + b * o_bs + (int64_t)tq * ldo + (int64_t)h * dv : nullptr;
    const int t_cached = fresh >= 0 ? fresh : Tk;   // rows read from k / v themselves
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        const float* vp = v + b * v_bs + (int64_t)hk * dv + d;
        float acc = 0.f;
#pragma unroll 8
        for (int t = 0; t < t_cached; ++t) acc = fmaf(sc[t], vp[(int64_t)t * ldv], acc);
        if (fresh >= 0) {
            const float vn = x.v_new[b * ldv + (int64_t)hk * dv + d];
            acc = fmaf(sc[fresh], vn, acc);
            const_cast<float*>(vp)[(int64_t)fresh * ldv] = vn;
        }
        if (gp) acc *= 1.f / (1.f + expf(-gp[d]));  // sigmoid gate, group_query_attention_layer.hpp:157-164
        op[d] = acc;
    }
}
}  // namespace

// Dot-product scores with 16-byte loads: one THREAD per key row in the score phase (a row's dk values are loaded as
// float4, all in flight together, and summed in rising d), and in the value phase a float4 of output columns per
// thread with the key rows dealt round-robin to 128 / (dv / 4) groups of threads whose partial sums are added in
// group order.  A (sample, head, query row) costs a few memory round trips whatever the key length; the kernel above
// stays for the other score forms and for unaligned operands.  DK: key_dim when known at compile time (else 0).
namespace {
template <int DK>
__global__ void __launch_bounds__(128) attention_rows_kernel(const float* __restrict__ q, int64_t ldq, int64_t q_bs, const float* k, int64_t ldk,
                                                             int64_t k_bs, const float* v, int64_t ldv, int64_t v_bs, float* __restrict__ out,
                                                             int64_t ldo, int64_t o_bs, int H, int Tq, int Tk, int dk_rt, int dv, float scale,
                                                             AttnExtra x) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int dk = DK ? DK : dk_rt;
    int fresh = -1;
    const int cap = Tk;
    if (x.len_ptr) {
        fresh = min(*x.len_ptr, Tk - 1);
        Tk = fresh + 1;
    }
    float* part = sm;                 // 128 float4 partial outputs
    float* qs = sm + 512;             // dk query values
    float* sc = qs + ((dk + 3) & ~3); // scores (capacity `cap`)
    (void)cap;
    __shared__ float red[4];
    const int tid = threadIdx.x;
    const int tq = blockIdx.x % Tq;
    const int h = (blockIdx.x / Tq) % H;
    const int64_t b = blockIdx.x / ((int64_t)Tq * H);
    const float* qp = q + b * q_bs + (int64_t)tq * ldq + (int64_t)h * dk;
    for (int d = tid; d < dk; d += 128) qs[d] = __ldcg(qp + d);
    __syncthreads();
    const int lane = tid & 31, wid = tid >> 5;
    const int hk = h / x.group;
    const float* kbase = k + b * k_bs + (int64_t)hk * dk;
    for (int t = tid; t < Tk; t += 128) {
        const bool is_fresh = t == fresh;
        const float4* kp = reinterpret_cast<const float4*>(is_fresh ? x.k_new + b * ldk + (int64_t)hk * dk : kbase + (int64_t)t * ldk);
        float s = 0.f;
        if (DK) {
            float4 kk[DK ? DK / 4 : 1];
#pragma unroll
            for (int i = 0; i < DK / 4; ++i) kk[i] = __ldcg(kp + i);
#pragma unroll
            for (int i = 0; i < DK / 4; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(qs + 4 * i);
                s = fmaf(qq.x, kk[i].x, s); s = fmaf(qq.y, kk[i].y, s); s = fmaf(qq.z, kk[i].z, s); s = fmaf(qq.w, kk[i].w, s);
            }
            if (is_fresh) {
                float4* kc = reinterpret_cast<float4*>(const_cast<float*>(kbase) + (int64_t)t * ldk);
#pragma unroll
                for (int i = 0; i < DK / 4; ++i) kc[i] = kk[i];
            }
        } else {
#pragma unroll 4
            for (int i = 0; i < dk / 4; ++i) {
                const float4 kk = __ldcg(kp + i);
                const float4 qq = *reinterpret_cast<const float4*>(qs + 4 * i);
                s = fmaf(qq.x, kk.x, s); s = fmaf(qq.y, kk.y, s); s = fmaf(qq.z, kk.z, s); s = fmaf(qq.w, kk.w, s);
                if (is_fresh) reinterpret_cast<float4*>(const_cast<float*>(kbase) + (int64_t)t * ldk)[i] = kk;
            }
        }
        sc[t] = s * scale;
    }
    __syncthreads();
    // softmax in the reference's form (tensor.hpp:1165-1192): exp(x - m - log sum exp(x - m)), inf -> 0
    float m = -FLT_MAX;
    for (int t = tid; t < Tk; t += 128) m = fmaxf(m, sc[t]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[wid] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float sum = 0.f;
    for (int t = tid; t < Tk; t += 128) sum += expf(sc[t] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[wid] = sum;
    __syncthreads();
    sum = ((red[0] + red[1]) + red[2]) + red[3];
    const float ls = logf(sum);
    for (int t = tid; t < Tk; t += 128) {
        const float r = expf(sc[t] - m - ls);
        sc[t] = isinf(r) ? 0.f : r;
    }
    __syncthreads();
    // values
    const int lanes = dv >> 2;            // threads across the head's output columns
    const int groups = 128 / lanes;       // key rows are dealt to the groups round-robin
    const int g = tid / lanes, dl = tid - g * lanes;
    if (g < groups) {
        const float* vbase = v + b * v_bs + (int64_t)hk * dv + 4 * dl;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int t = g; t < Tk; t += groups) {
            const bool is_fresh = t == fresh;
            const float4 vv = __ldcg(reinterpret_cast<const float4*>(is_fresh ? x.v_new + b * ldv + (int64_t)hk * dv + 4 * dl : vbase + (int64_t)t * ldv));
            const float pt = sc[t];
            acc.x = fmaf(pt, vv.x, acc.x); acc.y = fmaf(pt, vv.y, acc.y); acc.z = fmaf(pt, vv.z, acc.z); acc.w = fmaf(pt, vv.w, acc.w);
            if (is_fresh) *reinterpret_cast<float4*>(const_cast<float*>(vbase) + (int64_t)t * ldv) = vv;
        }
        *reinterpret_cast<float4*>(part + 4 * tid) = acc;
    }
    __syncthreads();
    float* op = out + b * o_bs + (int64_t)tq * ldo + (int64_t)h * dv;
    const float* gp = x.gate ? x.gate + b * o_bs + (int64_t)tq * ldo + (int64_t)h * dv : nullptr;
    for (int d = tid; d < dv; d += 128) {
        float acc = 0.f;
        for (int gg = 0; gg < groups; ++gg) acc += part[4 * (gg * lanes + (d >> 2)) + (d & 3)];
        if (gp) acc *= 1.f / (1.f + expf(-__ldcg(gp + d)));  // sigmoid gate, group_query_attention_layer.hpp:157-164
        op[d] = acc;
    }
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- decode positions on a short key/value cache: the rows of a (sample, head) pair staged in shared memory ----
// Same arithmetic as attention_rows_kernel with one query row (scores by one thread per key row, softmax in the
// reference's form, values by 8 groups of key rows added in group order), but a CTA is persistent: it walks the
// (sample, head) pairs with a stride of the grid and copies the NEXT pair's query, key and value rows into the other
// half of its shared memory (cp.async, 16 bytes each, all in flight at once) while it computes the current pair, so
// the key and value rows of a pair cost one trip to memory instead of two dependent ones and the trips of
// consecutive pairs overlap.  16-byte chunk c of row r sits at chunk c ^ (r & 7): a warp's threads read their own
// rows without bank conflicts.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(128) attention_stream_kernel(const float* __restrict__ q, int64_t ldq, int64_t q_bs, const float* k, int64_t ldk,
                                                               int64_t k_bs, const float* v, int64_t ldv, int64_t v_bs, float* __restrict__ out,
                                                               int64_t ldo, int64_t o_bs, int H, int cap, float scale, AttnExtra x, int pairs) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int CH = D / 4;                       // 16-byte chunks per row
    const int cap_r = (cap + 7) & ~7;
    const int buf_floats = 2 * cap_r * D + D;       // keys, values, query
    float* part = sm + 2 * buf_floats;              // 128 float4 partial outputs
    float* sc = part + 512;                         // scores
    __shared__ float red[4];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int fresh = min(*x.len_ptr, cap - 1);
    const int Tk = fresh + 1;

    auto stage = [&](int pair, int half) {
        const int h = pair % H;
        const int64_t b = pair / H;
        const int hk = h / x.group;
        float* kb = sm + half * buf_floats;
        const uint32_t k_s = (uint32_t)__cvta_generic_to_shared(kb), v_s = k_s + (uint32_t)(cap_r * D * 4), q_s = v_s + (uint32_t)(cap_r * D * 4);
        const float* kg = k + b * k_bs + (int64_t)hk * D;
        const float* vg = v + b * v_bs + (int64_t)hk * D;
        for (int e = tid; e < Tk * CH; e += 128) {
            const int r = e / CH, c = e - r * CH;
            const uint32_t off = (uint32_t)(r * D * 4 + ((c ^ (r & 7)) << 4));
            const bool is_fresh = r == fresh;
            cp_async16(k_s + off, (is_fresh ? x.k_new + b * ldk + (int64_t)hk * D : kg + (int64_t)r * ldk) + 4 * c);
            cp_async16(v_s + off, (is_fresh ? x.v_new + b * ldv + (int64_t)hk * D : vg + (int64_t)r * ldv) + 4 * c);
        }
        if (tid < CH) cp_async16(q_s + (uint32_t)(tid << 4), q + b * q_bs + (int64_t)h * D + 4 * tid);
    };

    int pair = blockIdx.x;
    if (pair < pairs) stage(pair, 0);
    cp_async_commit();
    for (int it = 0; pair < pairs; pair += gridDim.x, ++it) {
        const int half = it & 1;
        const int next = pair + gridDim.x;
        if (next < pairs) stage(next, half ^ 1);
        cp_async_commit();
        cp_async_wait<1>();        // everything but the newest group (the next pair) has landed
        __syncthreads();
        const int h = pair % H;
        const int64_t b = pair / H;
        const int hk = h / x.group;
        const float* kb = sm + half * buf_floats;
        const float* vb = kb + cap_r * D;
        const float* qs = vb + cap_r * D;
        // the new row goes into the cache
        if (tid < 2 * CH) {
            const int c = tid % CH;
            const float4 val = *reinterpret_cast<const float4*>((tid < CH ? kb : vb) + fresh * D + ((c ^ (fresh & 7)) << 2));
            float* dst = tid < CH ? const_cast<float*>(k) + b * k_bs + (int64_t)hk * D + (int64_t)fresh * ldk
                                  : const_cast<float*>(v) + b * v_bs + (int64_t)hk * D + (int64_t)fresh * ldv;
            *reinterpret_cast<float4*>(dst + 4 * c) = val;
        }
        for (int t = tid; t < Tk; t += 128) {
            const float* kr = kb + t * D;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const float4 kk = *reinterpret_cast<const float4*>(kr + ((i ^ (t & 7)) << 2));
                const float4 qq = *reinterpret_cast<const float4*>(qs + 4 * i);
                s = fmaf(qq.x, kk.x, s); s = fmaf(qq.y, kk.y, s); s = fmaf(qq.z, kk.z, s); s = fmaf(qq.w, kk.w, s);
            }
            sc[t] = s * scale;
        }
        __syncthreads();
        // softmax in the reference's form (tensor.hpp:1165-1192): exp(x - m - log sum exp(x - m)), inf -> 0
        float m = -FLT_MAX;
        for (int t = tid; t < Tk; t += 128) m = fmaxf(m, sc[t]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[wid] = m;
        __syncthreads();
        m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        __syncthreads();
        float sum = 0.f;
        for (int t = tid; t < Tk; t += 128) sum += expf(sc[t] - m);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) red[wid] = sum;
        __syncthreads();
        sum = ((red[0] + red[1]) + red[2]) + red[3];
        const float ls = logf(sum);
        for (int t = tid; t < Tk; t += 128) {
            const float r = expf(sc[t] - m - ls);
            sc[t] = isinf(r) ? 0.f : r;
        }
        __syncthreads();
        // values: CH threads across the head's columns, 128 / CH groups of key rows dealt round-robin
        constexpr int GROUPS = 128 / CH;
        const int g = tid / CH, dl = tid - g * CH;
        {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int t = g; t < Tk; t += GROUPS) {
                const float4 vv = *reinterpret_cast<const float4*>(vb + t * D + ((dl ^ (t & 7)) << 2));
                const float pt = sc[t];
                acc.x = fmaf(pt, vv.x, acc.x); acc.y = fmaf(pt, vv.y, acc.y); acc.z = fmaf(pt, vv.z, acc.z); acc.w = fmaf(pt, vv.w, acc.w);
            }
            *reinterpret_cast<float4*>(part + 4 * tid) = acc;
        }
        __syncthreads();
        float* op = out + b * o_bs + (int64_t)h * D;
        const float* gp = x.gate ? x.gate + b * o_bs + (int64_t)h * D : nullptr;
        for (int d = tid; d < D; d += 128) {
            float acc = 0.f;
#pragma unroll
            for (int gg = 0; gg < GROUPS; ++gg) acc += part[4 * (gg * CH + (d >> 2)) + (d & 3)];
            if (gp) acc *= 1.f / (1.f + expf(-__ldcg(gp + d)));  // sigmoid gate, group_query_attention_layer.hpp:157-164
            op[d] = acc;
        }
        __syncthreads();           // the pair's buffers, scores and partial sums are free again
    }
    cp_async_wait<0>();
}
}  // namespace

void launch_attention(const float* q, int64_t ldq, int64_t q_bstride, const float* k, int64_t ldk, int64_t k_bstride,
                      const float* v, int64_t ldv, int64_t v_bstride, float* out, int64_t ldo, int64_t o_bstride, int64_t B,
                      int H, int Tq, int Tk, int dk, int dv, float scale, cudaStream_t s, const AttnExtra& x) {
    const int64_t blocks = B * H * Tq;
    if (blocks == 0) return;
    const bool rows_form = x.mode == ATTN_DOT && dk % 4 == 0 && dv % 4 == 0 && dv <= 512 && ldk % 4 == 0 && ldv % 4 == 0 && k_bstride % 4 == 0 &&
                           v_bstride % 4 == 0 && aligned16(k) && aligned16(v) && (!x.len_ptr || (aligned16(x.k_new) && aligned16(x.v_new)));
    // one query row over a short device-resident cache: the streaming form, when both halves of its staging area fit
    if (rows_form && x.len_ptr && Tq == 1 && dk == 64 && dv == 64 && aligned16(q) && ldq % 4 == 0 && q_bstride % 4 == 0 && ldk % 4 == 0 &&
        B * H <= 0x7fffffff) {
        const int cap_r = (Tk + 7) & ~7;
        const size_t smem_s = (size_t)(2 * (2 * cap_r * 64 + 64) + 512 + cap_r) * sizeof(float);
        if (smem_s <= 200 * 1024) {
            static bool attr_set[64] = {};
            int dev = 0;
            FDK_CUDA(cudaGetDevice(&dev));
            if (dev < 0 || dev >= 64 || !attr_set[dev]) {
                FDK_CUDA(cudaFuncSetAttribute(attention_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                if (dev >= 0 && dev < 64) attr_set[dev] = true;
            }
            int sms = 0;
            FDK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(4, (227 * 1024) / (smem_s + 1024)));
            const int pairs = (int)(B * H);
            const int grid = std::min(pairs, sms * per_sm);
            launch_pdl(attention_stream_kernel<64>, dim3((unsigned)grid), dim3(128), smem_s, s, q, ldq, q_bstride, k, ldk, k_bstride, v, ldv, v_bstride,
                       out, ldo, o_bstride, H, Tk, scale, x, pairs);
            FDK_CUDA(cudaGetLastError());
            return;
        }
    }
    if (rows_form) {
        const size_t smem_r = (size_t)(512 + ((dk + 3) & ~3) + Tk) * sizeof(float);
        ensure(smem_r <= 200 * 1024, "attention: key length too large for the shared-memory score buffer");
        if (dk == 64) {
            if (smem_r > 48 * 1024) FDK_CUDA(cudaFuncSetAttribute(attention_rows_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_r));
            launch_pdl(attention_rows_kernel<64>, dim3((unsigned)blocks), dim3(128), smem_r, s, q, ldq, q_bstride, k, ldk, k_bstride, v, ldv, v_bstride, out,
                       ldo, o_bstride, H, Tq, Tk, dk, dv, scale, x);
        } else {
            if (smem_r > 48 * 1024) FDK_CUDA(cudaFuncSetAttribute(attention_rows_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_r));
            launch_pdl(attention_rows_kernel<0>, dim3((unsigned)blocks), dim3(128), smem_r, s, q, ldq, q_bstride, k, ldk, k_bstride, v, ldv, v_bstride, out,
                       ldo, o_bstride, H, Tq, Tk, dk, dv, scale, x);
        }
        FDK_CUDA(cudaGetLastError());
        return;
    }
    const size_t smem = (size_t)(Tk + dk) * sizeof(float);
    ensure(smem <= 200 * 1024, "attention: key length too large for the shared-memory score buffer");
    if (smem > 48 * 1024) FDK_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attention_kernel<<<(unsigned)blocks, 128, smem, s>>>(q, ldq, q_bstride, k, ldk, k_bstride, v, ldv, v_bstride, out, ldo,
                                                        o_bstride, H, Tq, Tk, dk, dv, scale, x);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Greedy token choice of a decode loop: out[b] = index of the first largest value of row b, as a float
// (token ids travel as floats through the model, embedding_layer.hpp:49).  One block per row.
// =====================================================================================================
namespace {
template <int THREADS>
__global__ void __launch_bounds__(THREADS) argmax_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const float* row = in + (int64_t)blockIdx.x * n;
    float best = -FLT_MAX;
    int best_i = 0x7fffffff;
    // a thread meets its candidates in rising index order, so `>` keeps the first of equal values
    int i = threadIdx.x;
    for (; i + 7 * THREADS < n; i += 8 * THREADS) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcg(row + i + u * THREADS);
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (v[u] > best) { best = v[u]; best_i = i + u * THREADS; }
    }
    for (; i < n; i += THREADS) {
        const float v = __ldcg(row + i);
        if (v > best) { best = v; best_i = i; }
    }
    // warp stage, then one value per warp
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, o);
        const int j = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (v > best || (v == best && j < best_i)) { best = v; best_i = j; }
    }
    __shared__ float sv[THREADS / 32];
    __shared__ int si[THREADS / 32];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
        out[blockIdx.x] = (float)(best_i == 0x7fffffff ? 0 : best_i);
    }
}
}  // namespace

namespace {
__global__ void publish_position_kernel(const float* __restrict__ tokens, int n, const int* status_a, const int* status_b,
                                        float* __restrict__ host_tokens, int* __restrict__ host_status) {
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < n; i += blockDim.x) host_tokens[i] = __ldcg(tokens + i);
    if (threadIdx.x == 0) {
        host_status[0] = __ldcg(status_a);
        host_status[1] = __ldcg(status_b);
    }
    __threadfence_system();
}
}  // namespace
void launch_publish_position(const float* tokens, int n, const int* status_a, const int* status_b, float* host_tokens, int* host_status,
                             cudaStream_t s) {
    launch_pdl(publish_position_kernel, dim3(1), dim3(128), 0, s, tokens, n, status_a, status_b, host_tokens, host_status);
}

void launch_argmax_rows(const float* in, float* out, int64_t rows, int n, cudaStream_t s) {
    if (rows <= 0 || n <= 0) return;
    if (n >= 8192) launch_pdl(argmax_rows_kernel<1024>, dim3((unsigned)rows), dim3(1024), 0, s, in, out, n);
    else launch_pdl(argmax_rows_kernel<256>, dim3((unsigned)rows), dim3(256), 0, s, in, out, n);
}

// =====================================================================================================
// PReLU (prelu_layer.hpp:30-68): y = x > 0 ? x : alpha[pos] * x, alpha indexed over (height, width, depth)
// with an index of 0 on every shared axis.
// =====================================================================================================
namespace {
__global__ void prelu_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ alpha, int64_t total,
                             int H, int W, int C, int hs, int ws, int cs) {
    const int aw = ws ? 1 : W, ad = cs ? 1 : C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = in[i];
        const int z = (int)(i % C);
        const int xx = (int)((i / C) % W);
        const int y = (int)((i / ((int64_t)C * W)) % H);
        const int pos = (hs ? 0 : y) * aw * ad + (ws ? 0 : xx) * ad + (cs ? 0 : z);
        out[i] = v > 0.f ? v : alpha[pos] * v;
    }
}
}  // namespace

void launch_prelu(const float* in, float* out, const float* alpha, int64_t B, int H, int W, int C, bool hs, bool ws, bool cs, cudaStream_t s) {
    const int64_t total = B * H * W * C;
    if (total == 0) return;
    const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 16);
    prelu_kernel<<<(unsigned)blocks, 256, 0, s>>>(in, out, alpha, total, H, W, C, hs, ws, cs);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// EinsumDense, general form: one thread per output element walks the summed letters.
// =====================================================================================================
namespace {
__global__ void einsum_kernel(const float* __restrict__ in, const float* __restrict__ kernel, const float* __restrict__ bias,
                              float* __restrict__ out, int64_t total, EinsumGeom g) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / g.out_volume;
        int64_t r = i - b * g.out_volume;
        int64_t io = b * g.in_volume, ko = 0, bo = 0;
        for (int l = g.n_out - 1; l >= 0; --l) {
            const int64_t c = r % g.out_size[l];
            r /= g.out_size[l];
            io += c * g.out_in[l]; ko += c * g.out_k[l]; bo += c * g.out_b[l];
        }
        float acc = 0.f;
        for (int64_t sidx = 0; sidx < g.sum_volume; ++sidx) {
            int64_t q = sidx, is = io, ks = ko;
            for (int l = g.n_sum - 1; l >= 0; --l) {
                const int64_t c = q % g.sum_size[l];
                q /= g.sum_size[l];
                is += c * g.sum_in[l]; ks += c * g.sum_k[l];
            }
            acc = fmaf(in[is], kernel[ks], acc);
        }
        out[i] = bias ? acc + bias[bo] : acc;
    }
}
}  // namespace

void launch_einsum(const float* in, const float* kernel, const float* bias, float* out, int64_t B, const EinsumGeom& g, cudaStream_t s) {
    const int64_t total = B * g.out_volume;
    if (total == 0) return;
    const int64_t blocks = std::min<int64_t>((total + 127) / 128, 148 * 32);
    einsum_kernel<<<(unsigned)blocks, 128, 0, s>>>(in, kernel, bias, out, total, g);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Patch matrix of Conv3D / Conv3DTranspose.
// =====================================================================================================
namespace {
__global__ void im2col3d_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, Conv3dGeom g) {
    const int K = g.k[0] * g.k[1] * g.k[2] * g.C;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int kq = (int)(i % g.Kp);
        int64_t m = i / g.Kp;
        float v = 0.f;
        if (kq < K) {
            const int c = kq % g.C;
            int tap = kq / g.C;
            int f[3], o[3];
            f[2] = tap % g.k[2]; tap /= g.k[2];
            f[1] = tap % g.k[1];
            f[0] = tap / g.k[1];
            o[2] = (int)(m % g.out[2]); m /= g.out[2];
            o[1] = (int)(m % g.out[1]); m /= g.out[1];
            o[0] = (int)(m % g.out[0]);
            const int64_t b = m / g.out[0];
            int src[3];
            bool inside = true;
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                const int p = o[a] * g.stride[a] + f[a] - g.pad_lo[a];
                const int q = p - g.off[a];
                inside = inside && p >= 0 && p < g.spread[a] && q >= 0 && q % g.inner[a] == 0 && q / g.inner[a] < g.in[a];
                src[a] = q / g.inner[a];
            }
            if (inside) v = in[(((b * g.in[0] + src[0]) * g.in[1] + src[1]) * g.in[2] + src[2]) * (int64_t)g.C + c];
        }
        out[i] = v;
    }
}
}  // namespace

void launch_im2col3d(const float* in, float* out, int64_t B, const Conv3dGeom& g, cudaStream_t s) {
    const int64_t total = B * g.out[0] * g.out[1] * g.out[2] * g.Kp;
    if (total == 0) return;
    im2col3d_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, g);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Bytes to floats (tensor_from_bytes): memory-bound, 16 bytes in and 64 bytes out per thread and step.
// =====================================================================================================
namespace {
__global__ void __launch_bounds__(256) bytes_to_float_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, int64_t n, float scale,
                                                             float low) {
    const int64_t n16 = n / 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(in)[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float4* o = reinterpret_cast<float4*>(out) + i * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float4 r;
            r.x = __fadd_rn(__fmul_rn((float)(w[q] & 0xFFu), scale), low);
            r.y = __fadd_rn(__fmul_rn((float)((w[q] >> 8) & 0xFFu), scale), low);
            r.z = __fadd_rn(__fmul_rn((float)((w[q] >> 16) & 0xFFu), scale), low);
            r.w = __fadd_rn(__fmul_rn((float)(w[q] >> 24), scale), low);
            o[q] = r;
        }
    }
    for (int64_t i = n16 * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __fadd_rn(__fmul_rn((float)in[i], scale), low);
}
}  // namespace

void launch_bytes_to_float(const uint8_t* in, float* out, int64_t n, float low, float high, cudaStream_t s) {
    if (n <= 0) return;
    ensure((reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "bytes_to_float: unaligned buffers");
    const float scale = (high - low) / 255.0f;
    bytes_to_float_kernel<<<grid_1d((n + 15) / 16, 256), 256, 0, s>>>(in, out, n, scale, low);
    FDK_CUDA(cudaGetLastError());
}

// =====================================================================================================
// Normalization layer and UpSampling2D.
// =====================================================================================================
namespace {
__global__ void normalization_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ mean,
                                     const float* __restrict__ var, int64_t total, int64_t n, int64_t inner, int invert) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t idx = (i / inner) % n;
        const double den = fmax((double)sqrtf(var[idx]), 1e-7);
        out[i] = invert ? (float)((double)mean[idx] + (double)in[i] * den) : (float)((double)(in[i] - mean[idx]) / den);
    }
}
__global__ void upsample2d_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int H, int W, int C, int fy, int fx,
                                  int bilinear) {
    const int Ho = H * fy, Wo = W * fx;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int z = (int)(i % C);
        const int x = (int)((i / C) % Wo);
        const int y = (int)((i / ((int64_t)C * Wo)) % Ho);
        const int64_t b = i / ((int64_t)C * Wo * Ho);
        const float* img = in + b * (int64_t)H * W * C;
        if (!bilinear) {
            out[i] = img[((int64_t)(y / fy) * W + x / fx) * C + z];
            continue;
        }
        // half-pixel centres, clamped to the image (interpolate_2d_value_bilinearly, tensor.hpp:997-1017); the lower
        // and right weights are 1.0 - w in double there, so the sum is formed in double
        const float scale_y = (float)Ho / (float)H, scale_x = (float)Wo / (float)W;
        const float yc = fminf(fmaxf(0.0f, ((float)y + 0.5f) / scale_y - 0.5f), (float)H);
        const float xc = fminf(fmaxf(0.0f, ((float)x + 0.5f) / scale_x - 0.5f), (float)W);
        const int yt = min((int)floorf(yc), H - 1), yb = min(H - 1, (int)floorf(yc) + 1);
        const int xl = min((int)floorf(xc), W - 1), xr = min(W - 1, (int)floorf(xc) + 1);
        const float fyt = (float)yb - yc, fxl = (float)xr - xc;
        const double fyb = 1.0 - (double)fyt, fxr = 1.0 - (double)fxl;
        const float tl = img[((int64_t)yt * W + xl) * C + z], tr = img[((int64_t)yt * W + xr) * C + z];
        const float bl = img[((int64_t)yb * W + xl) * C + z], br = img[((int64_t)yb * W + xr) * C + z];
        out[i] = (float)((double)(fyt * fxl * tl) + (double)fyt * fxr * (double)tr + fyb * (double)fxl * (double)bl + fyb * fxr * (double)br);
    }
}
}  // namespace

void launch_normalization(const float* in, float* out, const float* mean, const float* var, int64_t outer, int64_t n, int64_t inner,
                          bool invert, cudaStream_t s) {
    const int64_t total = outer * n * inner;
    if (total == 0) return;
    normalization_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, mean, var, total, n, inner, invert ? 1 : 0);
    FDK_CUDA(cudaGetLastError());
}

void launch_upsample2d(const float* in, float* out, int64_t B, int H, int W, int C, int fy, int fx, bool bilinear, cudaStream_t s) {
    const int64_t total = B * H * fy * W * fx * C;
    if (total == 0) return;
    upsample2d_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, fy, fx, bilinear ? 1 : 0);
    FDK_CUDA(cudaGetLastError());
}


// =====================================================================================================
// Resizing (tensor.hpp:959-1111), Dot (tensor.hpp:814-884), adaptive pooling (adaptive_pooling_3d_layer.hpp:53-113)
// and the preprocessing look-ups (discretization_layer.hpp, integer_lookup_layer.hpp, category_encoding_layer.hpp).
// None of them is on a hot path: one thread per output element, arithmetic in the reference's order.
// =====================================================================================================
namespace {
__device__ __forceinline__ float area_value(const float* img, int W, int C, int z, float top, float bottom, float left, float right, int Hs, int Ws) {
    // interpolate_2d_value_area (tensor.hpp:1037-1092).  Border rows / columns whose weight is zero are not read: for the
    // last output row or column they lie one past the image.
    const int top_outer = (int)floorf(top), left_outer = (int)floorf(left);
    const int top_inner = (int)ceilf(top), bottom_inner = (int)floorf(bottom), left_inner = (int)ceilf(left), right_inner = (int)floorf(right);
    const float top_w = (float)top_inner - top, left_w = (float)left_inner - left;
    const float bottom_w = bottom - (float)bottom_inner, right_w = right - (float)right_inner;
    auto at = [&](int y, int x) { return (y >= 0 && y < Hs && x >= 0 && x < Ws) ? img[((int64_t)y * W + x) * C + z] : 0.0f; };
    float inner_sum = 0.f, top_sum = 0.f, bottom_sum = 0.f, left_sum = 0.f, right_sum = 0.f;
    int inner_px = 0, row_px = 0, col_px = 0;
    for (int y = top_inner; y < bottom_inner; ++y)
        for (int x = left_inner; x < right_inner; ++x) { inner_sum += at(y, x); ++inner_px; }
    for (int x = left_inner; x < right_inner; ++x) { top_sum += at(top_outer, x); bottom_sum += at(bottom_inner, x); ++row_px; }
    for (int y = top_inner; y < bottom_inner; ++y) { left_sum += at(y, left_outer); right_sum += at(y, right_inner); ++col_px; }
    const float tl = top_w * left_w, tr = top_w * right_w, bl = bottom_w * left_w, br = bottom_w * right_w;
    const float weighted = inner_sum + top_w * top_sum + bottom_w * bottom_sum + left_w * left_sum + right_w * right_sum +
                           tl * at(top_outer, left_outer) + tr * at(top_outer, right_inner) + bl * at(bottom_inner, left_outer) +
                           br * at(bottom_inner, right_inner);
    const float pixels = (float)inner_px + top_w * (float)row_px + bottom_w * (float)row_px + left_w * (float)col_px + right_w * (float)col_px +
                         tl + tr + bl + br;
    return weighted / pixels;
}
__global__ void resize2d_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int H, int W, int C, int Ho, int Wo, int mode,
                                int y0, int x0, int Hs, int Ws) {
    const float scale_y = (float)Ho / (float)Hs, scale_x = (float)Wo / (float)Ws;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int z = (int)(i % C);
        const int x = (int)((i / C) % Wo);
        const int y = (int)((i / ((int64_t)C * Wo)) % Ho);
        const int64_t b = i / ((int64_t)C * Wo * Ho);
        const float* img = in + (b * H + y0) * (int64_t)W * C + (int64_t)x0 * C;   // the (cropped) source image, row stride W
        if (mode == 0) {
            const int yi = min(Hs - 1, (int)fmaxf(0.0f, roundf(((float)y + 0.5f) / scale_y - 0.5f)));
            const int xi = min(Ws - 1, (int)fmaxf(0.0f, roundf(((float)x + 0.5f) / scale_x - 0.5f)));
            out[i] = img[((int64_t)yi * W + xi) * C + z];
        } else if (mode == 1) {
            // interpolate_2d_value_bilinearly (tensor.hpp:997-1017): the lower and right weights are 1.0 - w in double
            const float yc = fminf(fmaxf(0.0f, ((float)y + 0.5f) / scale_y - 0.5f), (float)Hs);
            const float xc = fminf(fmaxf(0.0f, ((float)x + 0.5f) / scale_x - 0.5f), (float)Ws);
            const int yt = min((int)floorf(yc), Hs - 1), yb = min(Hs - 1, (int)floorf(yc) + 1);
            const int xl = min((int)floorf(xc), Ws - 1), xr = min(Ws - 1, (int)floorf(xc) + 1);
            const float fyt = (float)yb - yc, fxl = (float)xr - xc;
            const double fyb = 1.0 - (double)fyt, fxr = 1.0 - (double)fxl;
            const float tl = img[((int64_t)yt * W + xl) * C + z], tr = img[((int64_t)yt * W + xr) * C + z];
            const float bl = img[((int64_t)yb * W + xl) * C + z], br = img[((int64_t)yb * W + xr) * C + z];
            out[i] = (float)((double)(fyt * fxl * tl) + (double)fyt * fxr * (double)tr + fyb * (double)fxl * (double)bl + fyb * fxr * (double)br);
        } else {
            out[i] = area_value(img, W, C, z, (float)y / scale_y, (float)(y + 1) / scale_y, (float)x / scale_x, (float)(x + 1) / scale_x, Hs, Ws);
        }
    }
}
__global__ void dot_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t total, int64_t a_outer,
                           int64_t a_inner, int64_t b_outer, int64_t b_inner, int64_t K, int normalize) {
    const int64_t a_rem = a_outer * a_inner, b_rem = b_outer * b_inner;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ib = i % b_rem, ia = (i / b_rem) % a_rem, smp = i / (b_rem * a_rem);
        const float* pa = a + smp * a_rem * K + (ia / a_inner) * K * a_inner + ia % a_inner;
        const float* pb = b + smp * b_rem * K + (ib / b_inner) * K * b_inner + ib % b_inner;
        float na = 1.f, nb = 1.f;
        if (normalize) {   // l2_normalize (tensor.hpp:801-812): x * (1 / sqrt(max(sum x^2, machine epsilon)))
            float sa = 0.f, sb = 0.f;
            for (int64_t k = 0; k < K; ++k) { const float x = pa[k * a_inner], y = pb[k * b_inner]; sa += x * x; sb += y * y; }
            na = 1.0f / sqrtf(fmaxf(sa, FLT_EPSILON));
            nb = 1.0f / sqrtf(fmaxf(sb, FLT_EPSILON));
        }
        float acc = 0.f;
        for (int64_t k = 0; k < K; ++k) acc = fmaf(__fmul_rn(pa[k * a_inner], na), __fmul_rn(pb[k * b_inner], nb), acc);
        out[i] = acc;
    }
}
__device__ __forceinline__ void adapt_range(int i, int in_size, int out_size, int& lo, int& hi) {
    if (in_size == 1) { lo = 0; hi = 1; return; }
    lo = (int)floor((double)((int64_t)i * in_size) / (double)out_size);
    hi = (int)ceil((double)((int64_t)(i + 1) * in_size) / (double)out_size);
}
__global__ void adaptive_pool_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t total, int D, int H, int W, int C, int Do,
                                     int Ho, int Wo, int is_max) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int z = (int)(i % C);
        const int ox = (int)((i / C) % Wo);
        const int oy = (int)((i / ((int64_t)C * Wo)) % Ho);
        const int od = (int)((i / ((int64_t)C * Wo * Ho)) % Do);
        const int64_t b = i / ((int64_t)C * Wo * Ho * Do);
        int d0, d1, h0, h1, w0, w1;
        adapt_range(od, D, Do, d0, d1);
        adapt_range(oy, H, Ho, h0, h1);
        adapt_range(ox, W, Wo, w0, w1);
        const float* img = in + b * (int64_t)D * H * W * C;
        float acc = is_max ? -FLT_MAX : 0.f;
        int count = 0;
        for (int d = d0; d < d1; ++d)
            for (int y = h0; y < h1; ++y)
                for (int x = w0; x < w1; ++x) {
                    const float v = img[(((int64_t)d * H + y) * W + x) * C + z];
                    acc = is_max ? fmaxf(acc, v) : acc + v;
                    ++count;
                }
        if (!is_max && count > 0) acc /= (float)count;
        out[i] = acc;
    }
}
__global__ void lookup_kernel(int mode, const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ table, int64_t total,
                              int size, int has_mask) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float x = in[i];
        if (mode == 0) {   // std::upper_bound over the sorted boundaries
            int lo = 0, hi = size;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (x < table[mid]) hi = mid; else lo = mid + 1;
            }
            out[i] = (float)lo;
        } else {
            const long long v = (long long)x;
            const float key = (float)v;   // exact for every integer a float can hold
            float r = has_mask ? 1.0f : 0.0f;   // out of vocabulary: bucket 0, after the mask token's slot if there is one
            if (has_mask && v == (long long)table[2 * size]) {
                r = 0.0f;
            } else {
                int lo = 0, hi = size;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (table[mid] < key) lo = mid + 1; else hi = mid;
                }
                if (lo < size && table[lo] == key && (long long)table[lo] == v) r = table[size + lo];
            }
            out[i] = r;
        }
    }
}
__global__ void category_kernel(int mode, const float* __restrict__ in, float* __restrict__ out, int64_t B, int64_t n, int size, int* err) {
    // out is zero-filled by the launcher; one thread per input value
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < B * n; i += (int64_t)gridDim.x * blockDim.x) {
        const float x = in[i];
        const float fl = floorf(x);
        if (!(fl >= 0.f) || fl >= (float)size) { atomicExch(err, 2); continue; }
        float* slot = out + (i / n) * size + (int64_t)fl;
        if (mode == 4) atomicAdd(slot, 1.0f);   // counts are whole numbers: the order of the additions does not matter
        else *slot = 1.0f;
    }
}
}  // namespace

namespace {
__global__ void convlstm_cell_kernel(const float* __restrict__ x, const float* __restrict__ u, const float* __restrict__ c_prev,
                                     float* __restrict__ h, float* __restrict__ c, int64_t total, int U, ActSpecDev act, ActSpecDev ract) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % U);
        const int64_t base = (i / U) * 4 * U + k;
        const float zi = x[base] + (u ? u[base] : 0.f), zf = x[base + U] + (u ? u[base + U] : 0.f);
        const float zc = x[base + 2 * U] + (u ? u[base + 2 * U] : 0.f), zo = x[base + 3 * U] + (u ? u[base + 3 * U] : 0.f);
        const float iv = act_apply(ract, zi), fv = act_apply(ract, zf), cp = act_apply(act, zc), ov = act_apply(ract, zo);
        const float cn = __fadd_rn(__fmul_rn(fv, c_prev ? c_prev[i] : 0.f), __fmul_rn(iv, cp));
        c[i] = cn;
        h[i] = ov * act_apply(act, cn);
    }
}
}  // namespace
void launch_convlstm_cell(const float* x, const float* u, const float* c_prev, float* h, float* c, int64_t positions, int U, ActSpec act,
                          ActSpec ract, cudaStream_t s) {
    const int64_t total = positions * U;
    if (total == 0) return;
    convlstm_cell_kernel<<<grid_1d(total, 256), 256, 0, s>>>(x, u, c_prev, h, c, total, U, to_dev(act), to_dev(ract));
    FDK_CUDA(cudaGetLastError());
}

void launch_resize2d(const float* in, float* out, int64_t images, int H, int W, int C, int Ho, int Wo, int mode, int y0, int x0, int ch, int cw,
                     cudaStream_t s) {
    const int64_t total = images * Ho * Wo * C;
    if (total == 0) return;
    resize2d_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, H, W, C, Ho, Wo, mode, y0, x0, ch, cw);
    FDK_CUDA(cudaGetLastError());
}
void launch_dot(const float* a, const float* b, float* out, int64_t B, int64_t a_outer, int64_t a_inner, int64_t b_outer, int64_t b_inner, int64_t K,
                bool normalize, cudaStream_t s) {
    const int64_t total = B * a_outer * a_inner * b_outer * b_inner;
    if (total == 0) return;
    dot_kernel<<<grid_1d(total, 256), 256, 0, s>>>(a, b, out, total, a_outer, a_inner, b_outer, b_inner, K, normalize ? 1 : 0);
    FDK_CUDA(cudaGetLastError());
}
void launch_adaptive_pool(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo, bool is_max, cudaStream_t s) {
    const int64_t total = B * Do * Ho * Wo * C;
    if (total == 0) return;
    adaptive_pool_kernel<<<grid_1d(total, 256), 256, 0, s>>>(in, out, total, D, H, W, C, Do, Ho, Wo, is_max ? 1 : 0);
    FDK_CUDA(cudaGetLastError());
}
void launch_lookup(int mode, const float* in, float* out, const float* table, int64_t B, int64_t n, int size, bool has_mask, int* err,
                   cudaStream_t s) {
    if (B * n == 0) return;
    if (mode <= 1) {
        lookup_kernel<<<grid_1d(B * n, 256), 256, 0, s>>>(mode, in, out, table, B * n, size, has_mask ? 1 : 0);
    } else {
        FDK_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)(B * size), s));
        category_kernel<<<grid_1d(B * n, 256), 256, 0, s>>>(mode, in, out, B, n, size, err);
    }
    FDK_CUDA(cudaGetLastError());
}

}  // namespace fdk
