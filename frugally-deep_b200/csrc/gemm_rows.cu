// Products with at most 64 rows on the 5th-generation tensor cores: C[M <= 64, N] = epilogue(X[M, K] * W[N, K]^T).
//
// This is the shape of one decode position (a handful of sequences against every weight matrix of the model) and of
// a dense head on a few samples: dense_layer.hpp:44-96 and the projections of multi_head_attention_layer.hpp:74-110
// in the reference, which runs them as one GEMV per row.  The arithmetic is trivial; what counts is streaming W from
// HBM once, over all SMs, and keeping the chain "launch -> operands -> products -> reduction -> epilogue" short,
// because a decode position is sixty such launches, one after the other.
//
// Layout of the work.  W is cut into blocks of BN = 128 (or 64) rows and K into S slices; one CTA per (block, slice),
// the S CTAs of a block forming a thread-block cluster.  A CTA computes D[BN, 64] = W_blk[BN, Ks] * X[:, Ks]^T with
// tcgen05.mma.kind::tf32 (weight rows on the 128 TMEM lanes, the X rows as the 64 columns), both operands from
// shared memory, fetched by TMA in 32-wide k blocks through a ring of stages.  FP32 semantics through 3xTF32: the
// tensor core reads only the leading 10 mantissa bits of an fp32 operand, so the raw tile IS the "big" half; converter
// warps write the exact remainders (x - trunc(x)) beside it and every k step issues W_small*X_big, W_big*X_small
// (into one accumulator) and W_big*X_big (into another: the tensor core truncates when it adds, so the small terms
// are kept out of the large sums; big terms of even and odd k blocks go to two accumulators for the same reason).
// Reduction over the K slices stays on chip: every CTA parks its partial tile in shared memory, the cluster meets at
// a hardware barrier, and each CTA then sums a share of the tile's rows over all S partial tiles with 16-byte loads
// through distributed shared memory, in slice order (deterministic, independent of M), applies the epilogue and stores.
// (Pushing the values to the owning CTA with scalar remote stores instead measured 4 us slower per launch.)
// Optionally the kernel normalises X first (LayerNormalization over K fused in front of the product: the cluster
// spans K, so row sums are exchanged the same way), which saves the separate normalisation launch and its output.
//
// Launch chain.  The kernel is launched with programmatic stream serialisation: it may start while its predecessor
// still runs, fetches its first W tiles, pulls the later ones into L2 and writes the first tiles' remainders (weights
// never depend on the predecessor), and only then executes griddepcontrol.wait, after which it touches X, the
// residual and C.  Every mbarrier wait is bounded; a wait that
// gives up sets a status word that the host reads, and the CTA still passes every cluster barrier so that its
// peers are not left waiting.
#include "kernels.cuh"
#include "device_math.cuh"
#include "pdl.cuh"
#include "tc_maps.hpp"
#include "tc_ptx.cuh"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace fdk {

namespace {

constexpr int RW_BK = 32;                       // fp32 values per k block = one 128-byte swizzle row
constexpr int RW_M = 64;                        // most rows of X
constexpr int RW_BN = 128;                      // weight rows of a full block (TMEM lanes)
constexpr int RW_STAGES = 4;
constexpr int RW_W_BYTES = RW_BN * RW_BK * 4;   // 16 KB: raw W tile; the same again for its remainders
constexpr int RW_X_BYTES = RW_M * RW_BK * 4;    // 8 KB
constexpr int RW_STAGE_BYTES = 2 * RW_W_BYTES + 2 * RW_X_BYTES;   // W_raw | W_small | X_raw | X_small = 48 KB
constexpr int RW_THREADS = 192;                 // warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 converters / epilogue
constexpr int RW_TMEM_COLS = 256;               // accumulators: big (even k blocks) | big (odd) | small | unused
constexpr int RW_MAX_CLUSTER = 8;
constexpr int RW_XCH_BYTES = RW_M * RW_BN * 4;  // exchange area of the reduction: this CTA's partial tile, read by its peers
constexpr int RW_TAIL_BYTES = 1536;             // barriers, flags, LayerNormalization row statistics
constexpr int RW_SMEM = RW_STAGES * RW_STAGE_BYTES + RW_XCH_BYTES + RW_TAIL_BYTES;
static_assert(RW_SMEM <= 227 * 1024, "shared memory budget");
constexpr int RW_PREFETCH = 12;                 // k blocks whose W tiles are pulled into L2 ahead of the ring
constexpr unsigned long long RW_WAIT_LIMIT_NS = 2000000000ull;   // 2 s: far beyond any legitimate wait

__device__ int g_rows_status = 0;

struct RowsParams {
    float* C[3];
    long long ldc[3];
    const float* bias[3];
    EpiDev epi;               // bias is taken from bias[z]
    int M, N, K;
    int bn;                   // weight rows per block: 64 or 128
    int kb_total;             // ceil(K / 32)
    int kb_per_cta;           // k blocks per slice
    int cluster;              // S: CTAs (K slices) per block
    // LayerNormalization over K in front of the product (layer_normalization_layer.hpp:37-63): off when ln == 0
    int ln;
    const float* gamma;
    const float* beta;
    float eps;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of all CTAs of the cluster; orders shared-memory accesses across the cluster.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of the same barrier, for a rendezvous that need not block where it is announced.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster1(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cluster4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
// Pulls a tile of a tensor map into L2 without a destination in shared memory.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y) : "memory");
}
// Bounded wait.  The kernel lives for a few microseconds and every hand-off is on its critical path, so the waiters
// poll (mbarrier.test_wait) instead of suspending; the wall clock is looked at every 64 polls.
__device__ __forceinline__ bool rows_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_test(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
#pragma unroll 1
        for (int it = 0; it < 64; ++it)
            if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > RW_WAIT_LIMIT_NS) break;
    }
    *abort_flag = 1;
    atomicCAS(&g_rows_status, 0, code);
    return false;
}

// D[128 x 64] (+)= A[128 x 8] * B[64 x 8]^T, both operands K-major tiles in shared memory.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 z;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "mov.b32 z, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {z, z, z, z}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// x - trunc_tf32(x): what the tensor core drops when it reads x (exact).  Infinities and NaNs have no remainder.
__device__ __forceinline__ float tf32_remainder(float x) {
    const float big = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    const float r = x - big;
    return (fabsf(x) < __int_as_float(0x7f800000)) ? r : 0.0f;
}
__device__ __forceinline__ float4 tf32_remainder4(const float4 v) {
    return make_float4(tf32_remainder(v.x), tf32_remainder(v.y), tf32_remainder(v.z), tf32_remainder(v.w));
}

__global__ void __launch_bounds__(RW_THREADS, 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW0,
                 const __grid_constant__ CUtensorMap mapW1, const __grid_constant__ CUtensorMap mapW2, const RowsParams prm) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    const uint32_t base = smem_u32(smem_raw);
    // layout: ring of stages | exchange area of the reduction | barriers, flags, row statistics
    float* xch = reinterpret_cast<float*>(smem + RW_STAGES * RW_STAGE_BYTES);
    uint8_t* tail = smem + RW_STAGES * RW_STAGE_BYTES + RW_XCH_BYTES;
    const uint32_t bar_base = smem_u32(tail);
    auto wfull_bar = [&](int s) { return bar_base + (uint32_t)s * 8u; };                      // TMA landed: raw W tile
    auto xfull_bar = [&](int s) { return bar_base + (uint32_t)(RW_STAGES + s) * 8u; };        // TMA landed: raw X tile
    auto conv_bar = [&](int s) { return bar_base + (uint32_t)(2 * RW_STAGES + s) * 8u; };     // remainders written (4 warps)
    auto empty_bar = [&](int s) { return bar_base + (uint32_t)(3 * RW_STAGES + s) * 8u; };    // MMAs of the stage done
    const uint32_t acc_bar = bar_base + (uint32_t)(4 * RW_STAGES) * 8u;                       // all MMAs done
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 200);
    float* ln_sum = reinterpret_cast<float*>(tail + 256);     // this CTA's partial row sums (read by the cluster)
    float* ln_sq = ln_sum + RW_M;                             // partial sums of squared deviations
    float* ln_mean = ln_sq + RW_M;
    float* ln_rstd = ln_mean + RW_M;
    static_assert(256 + 4 * RW_M * 4 <= RW_TAIL_BYTES && (4 * RW_STAGES + 1) * 8 <= 192, "tail layout");

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int S = prm.cluster;
    const int rank = (int)cluster_rank();
    const int z = blockIdx.z;
    const int n0 = blockIdx.y * prm.bn;
    const int kb0 = rank * prm.kb_per_cta;
    const int my_nkb = max(0, min(prm.kb_per_cta, prm.kb_total - kb0));
    const CUtensorMap* mapW = z == 0 ? &mapW0 : (z == 1 ? &mapW1 : &mapW2);

    if (tid == 0) {
        pdl_launch_dependents();
        for (int s = 0; s < RW_STAGES; ++s) {
            mbar_init(wfull_bar(s), 1);
            mbar_init(xfull_bar(s), 1);
            mbar_init(conv_bar(s), 4);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = (base & 1023u) != 0 ? 1 : 0;   // cannot happen: the kernel has no static shared memory
        if (*abort_flag) atomicCAS(&g_rows_status, 0, 99);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), (uint32_t)RW_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    cluster_arrive();   // "this CTA runs": awaited below, before anyone touches a peer's shared memory

    auto stage_ptr = [&](int s) { return base + (uint32_t)(s * RW_STAGE_BYTES); };
    const uint32_t w_bytes = (uint32_t)(prm.bn * RW_BK * 4);
    const int n_pre = min(RW_STAGES, my_nkb);
    const int w4 = prm.bn * 8;   // float4s of a W tile

    // remainders of the raw W tile of stage s (converter threads)
    auto convert_w = [&](int s, int ct) {
        const float4* w_raw = reinterpret_cast<const float4*>(smem + (size_t)s * RW_STAGE_BYTES);
        float4* w_small = reinterpret_cast<float4*>(smem + (size_t)s * RW_STAGE_BYTES + RW_W_BYTES);
        for (int idx = ct; idx < w4; idx += 128) w_small[idx] = tf32_remainder4(w_raw[idx]);
    };

    // ---- before the dependency wait: everything that only needs the weights (they are never written) ----
    bool conv_ok = !*abort_flag;
    if (tid == 0 && conv_ok) {
        for (int i = 0; i < n_pre; ++i) {
            mbar_arrive_expect_tx(wfull_bar(i), w_bytes);
            tma_load_2d(stage_ptr(i), mapW, (kb0 + i) * RW_BK, n0, wfull_bar(i));
        }
        // later tiles of this CTA are pulled towards L2 now, so that the ring only ever waits for L2
        for (int i = n_pre; i < min(my_nkb, n_pre + RW_PREFETCH); ++i) tma_prefetch_2d(mapW, (kb0 + i) * RW_BK, n0);
    }
    if (warp >= 2) {
        for (int i = 0; i < n_pre && conv_ok; ++i) {
            conv_ok = rows_wait(wfull_bar(i), 0u, abort_flag, 5);
            if (conv_ok) convert_w(i, tid - 64);
        }
    }
    pdl_wait();       // every thread: X, the residual and C belong to the chain of launches
    cluster_wait();   // every CTA of the cluster has started: its shared memory may be addressed from now on
    if (tid == 0 && !*abort_flag) {
        for (int i = 0; i < n_pre; ++i) {
            mbar_arrive_expect_tx(xfull_bar(i), (uint32_t)RW_X_BYTES);
            tma_load_2d(stage_ptr(i) + 2 * RW_W_BYTES, &mapX, (kb0 + i) * RW_BK, 0, xfull_bar(i));
        }
    }

    // ---- LayerNormalization statistics of the rows of X over all of K (the cluster spans K) ----
    // The CTA's whole K slice of X sits in the ring (the host plans at most RW_STAGES k blocks per slice for this form):
    // two threads per row add up alternate 16-byte chunks of the row in every tile, the cluster exchanges the partial
    // sums, then the same for the squared deviations from the mean (the reference's two passes, tensor.hpp:758-771).
    if (prm.ln) {
        const int m = (tid >> 1) & (RW_M - 1), half = tid & 1;
        const bool worker = tid < 2 * RW_M;
        bool ln_ok = !*abort_flag;
        if (worker)
            for (int i = 0; i < my_nkb && ln_ok; ++i) ln_ok = rows_wait(xfull_bar(i), 0u, abort_flag, 6);
        // chunk p (position in the 128-byte row) holds the values k0 + 4 (p ^ (m & 7)) ..; chunks beyond K were zero-filled
        auto row_chunk = [&](int i, int p, int& k) {
            k = (kb0 + i) * RW_BK + 4 * (p ^ (m & 7));
            return *reinterpret_cast<const float4*>(smem + (size_t)i * RW_STAGE_BYTES + 2 * RW_W_BYTES + m * 128 + p * 16);
        };
        float part = 0.f;
        if (worker && ln_ok && m < prm.M)
            for (int i = 0; i < my_nkb; ++i)
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    int k;
                    const float4 v = row_chunk(i, 2 * p + half, k);
                    if (k < prm.K) part += (v.x + v.y) + (v.z + v.w);
                }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        if (worker && half == 0) ln_sum[m] = part;
        cluster_sync_all();
        float mean = 0.f;
        if (worker) {
            float total = 0.f;
            for (int s = 0; s < S; ++s) total += ld_cluster1(map_to_cta(smem_u32(ln_sum + m), (uint32_t)s));
            mean = total / (float)prm.K;
        }
        part = 0.f;
        if (worker && ln_ok && m < prm.M)
            for (int i = 0; i < my_nkb; ++i)
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    int k;
                    const float4 v = row_chunk(i, 2 * p + half, k);
                    if (k < prm.K) {
                        const float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
                        part += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                    }
                }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        if (worker && half == 0) ln_sq[m] = part;
        cluster_sync_all();
        if (worker && half == 0) {
            float total = 0.f;
            for (int s = 0; s < S; ++s) total += ld_cluster1(map_to_cta(smem_u32(ln_sq + m), (uint32_t)s));
            ln_mean[m] = m < prm.M ? mean : 0.f;
            ln_rstd[m] = m < prm.M ? 1.0f / sqrtf(total / (float)prm.K + prm.eps) : 0.f;
        }
        __syncthreads();
    }

    // rows of the output tile this CTA sums and stores, and where a row's partial values go (see the reduction below)
    const int rows_per = (prm.M + S - 1) / S;

    if (warp == 0) {
        // ---------------- TMA producer: the k blocks beyond the first ring ----------------
        bool ok = !*abort_flag;
        for (int i = n_pre; i < my_nkb && ok; ++i) {
            const int s = i % RW_STAGES;
            if (!rows_wait(empty_bar(s), (uint32_t)(((i / RW_STAGES) - 1) & 1), abort_flag, 1)) { ok = false; break; }
            if (lane == 0) {
                mbar_arrive_expect_tx(wfull_bar(s), w_bytes);
                tma_load_2d(stage_ptr(s), mapW, (kb0 + i) * RW_BK, n0, wfull_bar(s));
                mbar_arrive_expect_tx(xfull_bar(s), (uint32_t)RW_X_BYTES);
                tma_load_2d(stage_ptr(s) + 2 * RW_W_BYTES, &mapX, (kb0 + i) * RW_BK, 0, xfull_bar(s));
                if (i + RW_PREFETCH < my_nkb) tma_prefetch_2d(mapW, (kb0 + i + RW_PREFETCH) * RW_BK, n0);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) {
            // gave up: leave copies already issued a bounded time to land before the CTA exits
            for (int s = 0; s < RW_STAGES; ++s)
                for (uint32_t it = 0; it < 4096 && !mbar_test(wfull_bar(s), 0) && !mbar_test(wfull_bar(s), 1); ++it) __nanosleep(64);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t idesc = make_idesc(RW_BN, RW_M);
        bool ok = !*abort_flag;
        for (int i = 0; i < my_nkb && ok; ++i) {
            const int s = i % RW_STAGES;
            if (!rows_wait(conv_bar(s), (uint32_t)((i / RW_STAGES) & 1), abort_flag, 2)) { ok = false; break; }
            tc_fence_after();
            if (lane == 0) {
                const uint64_t w_big = make_smem_desc(stage_ptr(s));
                const uint64_t w_small = make_smem_desc(stage_ptr(s) + RW_W_BYTES);
                const uint64_t x_big = make_smem_desc(stage_ptr(s) + 2 * RW_W_BYTES);
                const uint64_t x_small = make_smem_desc(stage_ptr(s) + 2 * RW_W_BYTES + RW_X_BYTES);
                const uint32_t d_big = tmem_base + (uint32_t)((i & 1) * RW_M);
                const uint32_t d_small = tmem_base + (uint32_t)(2 * RW_M);
#pragma unroll
                for (int j = 0; j < RW_BK / 8; ++j) {
                    const uint64_t step = (uint64_t)(2 * j);   // 8 values = 32 bytes = 2 descriptor units
                    umma_ss(d_small, w_small + step, x_big + step, idesc, (i > 0 || j > 0) ? 1u : 0u);
                    umma_ss(d_small, w_big + step, x_small + step, idesc, 1u);
                    umma_ss(d_big, w_big + step, x_big + step, idesc, (i > 1 || j > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));
                if (i == my_nkb - 1) umma_commit(acc_bar);
            }
            __syncwarp();
        }
    } else {
        // ---------------- converters: remainders of the raw tiles (and the normalisation of X) ----------------
        const int ct = tid - 64;   // 0..127
        bool ok = conv_ok && !*abort_flag;
        for (int i = 0; i < my_nkb && ok; ++i) {
            const int s = i % RW_STAGES;
            const uint32_t parity = (uint32_t)((i / RW_STAGES) & 1);
            if (i >= n_pre) {   // the first ring's W tiles were converted before the dependency wait
                if (!rows_wait(wfull_bar(s), parity, abort_flag, 3)) { ok = false; break; }
                convert_w(s, ct);
            }
            if (!rows_wait(xfull_bar(s), parity, abort_flag, 3)) { ok = false; break; }
            uint8_t* st = smem + (size_t)s * RW_STAGE_BYTES;
            float4* x_raw = reinterpret_cast<float4*>(st + 2 * RW_W_BYTES);
            float4* x_small = reinterpret_cast<float4*>(st + 2 * RW_W_BYTES + RW_X_BYTES);
            // X: 64 rows of eight 16-byte chunks; chunk c of row r sits at position c ^ (r & 7) (128-byte swizzle)
#pragma unroll
            for (int it = 0; it < (RW_M * 8) / 128; ++it) {
                const int idx = ct + it * 128;
                float4 v = x_raw[idx];
                if (prm.ln) {
                    const int r = idx >> 3, c = (idx & 7) ^ (r & 7);
                    const int k = (kb0 + i) * RW_BK + 4 * c;
                    if (k < prm.K) {   // K % 4 == 0: a chunk is inside or outside as a whole
                        const float mean = ln_mean[r], rstd = ln_rstd[r];
                        const float4 g = prm.gamma ? __ldg(reinterpret_cast<const float4*>(prm.gamma + k)) : make_float4(1.f, 1.f, 1.f, 1.f);
                        const float4 b = prm.beta ? __ldg(reinterpret_cast<const float4*>(prm.beta + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        // y = x * inv + (beta - mean * inv), inv = gamma / sqrt(var + eps), each step rounded (tensor.hpp:788-792)
                        float inv = rstd * g.x; v.x = __fadd_rn(__fmul_rn(v.x, inv), b.x - __fmul_rn(mean, inv));
                        inv = rstd * g.y; v.y = __fadd_rn(__fmul_rn(v.y, inv), b.y - __fmul_rn(mean, inv));
                        inv = rstd * g.z; v.z = __fadd_rn(__fmul_rn(v.z, inv), b.z - __fmul_rn(mean, inv));
                        inv = rstd * g.w; v.w = __fadd_rn(__fmul_rn(v.w, inv), b.w - __fmul_rn(mean, inv));
                    } else {
                        v = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    x_raw[idx] = v;
                }
                x_small[idx] = tf32_remainder4(v);
            }
            fence_proxy_async();   // these generic-proxy stores are read by the tensor core (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(conv_bar(s));
        }
        // ---- the partial tile: TMEM -> registers -> this CTA's exchange area, P[m][n] with n the weight row inside the block ----
        if (ok && my_nkb > 0) ok = rows_wait(acc_bar, 0u, abort_flag, 4);
        tc_fence_after();
        const int q = warp & 3;                      // the TMEM lane quadrant this warp may read
        const int n_local = q * 32 + lane;
        if (n_local < prm.bn) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v[32];
                if (ok && my_nkb > 0) {
                    uint32_t b0[32], sm[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(32 * h);
                    tmem_ld32(taddr, b0);
                    tmem_ld32(taddr + (uint32_t)(2 * RW_M), sm);
                    if (my_nkb > 1) {
                        uint32_t b1[32];
                        tmem_ld32(taddr + (uint32_t)RW_M, b1);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = (__uint_as_float(b0[j]) + __uint_as_float(b1[j])) + __uint_as_float(sm[j]);
                    } else {
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(b0[j]) + __uint_as_float(sm[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) xch[(32 * h + j) * RW_BN + n_local] = v[j];
            }
        }
        tc_fence_before();
    }

    // ---- reduction over the K slices through distributed shared memory: the rows of the tile are dealt to the CTAs of
    // the cluster; each sums its rows over all S partial tiles with 16-byte loads from its peers, then epilogue and store ----
    cluster_sync_all();
    {
        const int m_lo = rank * rows_per, m_hi = min(prm.M, m_lo + rows_per);
        const int bn4 = prm.bn >> 2;
        const int items = m_hi > m_lo ? (m_hi - m_lo) * bn4 : 0;
        const uint32_t p_addr = smem_u32(xch);
        float* C = prm.C[z];
        const long long ldc = prm.ldc[z];
        const float* bias = prm.bias[z];
        const EpiDev& e = prm.epi;
        const bool vec = (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
                         (!e.residual || ((e.ldr & 3) == 0 && (reinterpret_cast<uintptr_t>(e.residual) & 15) == 0));
        for (int t = tid; t < items; t += RW_THREADS) {
            const int m = m_lo + t / bn4, n4 = t % bn4;
            const int n = n0 + 4 * n4;
            if (n >= prm.N) continue;
            const uint32_t off = p_addr + (uint32_t)((m * RW_BN + 4 * n4) * 4);
            // all slices' loads in flight together, then the sum in slice order (it does not depend on which CTA adds it)
            float4 part[RW_MAX_CLUSTER];
#pragma unroll
            for (int s = 0; s < RW_MAX_CLUSTER; ++s)
                part[s] = s < S ? ld_cluster4(map_to_cta(off, (uint32_t)s)) : make_float4(0.f, 0.f, 0.f, 0.f);
            float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < RW_MAX_CLUSTER; ++s)
                if (s < S) { v[0] += part[s].x; v[1] += part[s].y; v[2] += part[s].z; v[3] += part[s].w; }
            const bool full4 = n + 3 < prm.N;
            if (bias) {
                if (full4) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(bias + n));
                    v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
                } else {
                    for (int j = 0; j < 4 && n + j < prm.N; ++j) v[j] += __ldg(bias + n + j);
                }
            }
            if (e.act1.kind != ACT_NONE) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = act_apply(e.act1, v[j]);
            }
            if (e.scale) {
                for (int j = 0; j < 4 && n + j < prm.N; ++j) v[j] = __fadd_rn(__fmul_rn(v[j], __ldg(e.scale + n + j)), __ldg(e.shift + n + j));
            }
            if (e.residual) {
                const float* res = e.residual + (long long)m * e.ldr + n;
                if (vec && full4) {
                    const float4 p = __ldcg(reinterpret_cast<const float4*>(res));
                    v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                } else {
                    for (int j = 0; j < 4 && n + j < prm.N; ++j) v[j] += __ldcg(res + j);
                }
            }
            if (e.act2.kind != ACT_NONE) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = act_apply(e.act2, v[j]);
            }
            float* dst = C + (long long)m * ldc + n;
            if (vec && full4) {
                *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
                for (int j = 0; j < 4 && n + j < prm.N; ++j) dst[j] = v[j];
            }
        }
    }
    cluster_sync_all();   // nobody leaves while a peer may still read its partial tile
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)RW_TMEM_COLS);
    }
}

// Per device: the shared-memory opt-in of the kernel, and how many clusters of each size the device can hold at once
// (a CTA takes a whole SM, and a cluster must fit inside one GPC, so clusters of 8 do not cover all SMs).
struct RowsDevice {
    bool ready = false;
    int max_clusters[RW_MAX_CLUSTER + 1] = {};
};
const RowsDevice& rows_device() {
    static std::mutex mu;
    static RowsDevice table[64];
    static RowsDevice fallback;
    int dev = 0;
    FDK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    RowsDevice& d = (dev >= 0 && dev < 64) ? table[dev] : fallback;
    if (!d.ready) {
        FDK_CUDA(cudaFuncSetAttribute(gemm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RW_SMEM));
        const int sms = tc_sm_count();
        for (int c = 1; c <= RW_MAX_CLUSTER; ++c) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)c, (unsigned)sms, 1);
            cfg.blockDim = dim3(RW_THREADS, 1, 1);
            cfg.dynamicSmemBytes = RW_SMEM;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)c;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_rows_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = sms / c / 2; }
            d.max_clusters[c] = n;
        }
        d.ready = true;
    }
    return d;
}

}  // namespace

bool gemm_rows_supported(int64_t M, int N, int K, int64_t lda, int64_t ldw, const void* A, const void* W) {
    return M >= 1 && M <= RW_M && N >= 1 && K >= 4 && (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && K <= lda && K <= ldw &&
           ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) && tc_get_encode() != nullptr;
}

// Blocks of weight rows and K slices for `count` products of one shape: as many CTAs as fit one wave over the SMs
// (every CTA streams a different part of W); among equals the taller block (less traffic for X per byte of W).
void gemm_rows_plan(int N, int K, int count, int& bn, int& cluster, int& kb_per_cta, bool normalised) {
    const int kb_total = (K + RW_BK - 1) / RW_BK;
    const RowsDevice& dev = rows_device();
    int best_ctas = -1;
    bn = RW_BN; cluster = 1;
    for (int b : {RW_BN, RW_BN / 2}) {
        const int blocks = ((N + b - 1) / b) * count;
        for (int s = 1; s <= RW_MAX_CLUSTER; ++s) {
            if (s > kb_total) break;
            const int per = (kb_total + s - 1) / s;
            if ((s - 1) * per >= kb_total) continue;      // the last slice would be empty
            if (normalised && per > RW_STAGES) continue;  // the row statistics are taken from the tiles in the ring
            if (blocks > dev.max_clusters[s]) continue;   // all clusters resident at once: one wave
            const int ctas = blocks * s;
            if (ctas > best_ctas) { best_ctas = ctas; bn = b; cluster = s; }
        }
    }
    // more blocks than SMs (a vocabulary projection): tall blocks, no slicing, several waves
    kb_per_cta = (kb_total + cluster - 1) / cluster;
}

bool gemm_rows_norm_supported(int N, int K, int count) {
    int bn = 0, cluster = 0, per = 0;
    gemm_rows_plan(N, K, count, bn, cluster, per, true);
    return per <= RW_STAGES;
}

void launch_gemm_rows(const float* X, int64_t ldx, int count, const float* const* W, int64_t ldw, float* const* C, const int64_t* ldc,
                      const float* const* bias, const Epilogue& e, int64_t M, int N, int K, const RowsNorm* norm, cudaStream_t s) {
    ensure(count >= 1 && count <= 3, "row product: one to three products per launch");
    ensure(M >= 1 && M <= RW_M, "row product: at most 64 rows");
    rows_device();
    RowsParams prm = {};
    int bn = RW_BN, cluster = 1, per = 1;
    gemm_rows_plan(N, K, count, bn, cluster, per, norm != nullptr);
    prm.epi = to_dev(e);
    prm.epi.bias = nullptr;
    prm.M = (int)M; prm.N = N; prm.K = K;
    prm.bn = bn; prm.cluster = cluster; prm.kb_per_cta = per; prm.kb_total = (K + RW_BK - 1) / RW_BK;
    for (int i = 0; i < 3; ++i) {
        const int j = i < count ? i : 0;
        prm.C[i] = C[j]; prm.ldc[i] = ldc[j]; prm.bias[i] = bias ? bias[j] : nullptr;
    }
    if (norm) {
        prm.ln = 1; prm.gamma = norm->gamma; prm.beta = norm->beta; prm.eps = norm->eps;
        ensure(per <= RW_STAGES, "row product: the normalised form needs the whole K slice of a CTA in the ring");
        ensure((!norm->gamma || (reinterpret_cast<uintptr_t>(norm->gamma) & 15) == 0) && (!norm->beta || (reinterpret_cast<uintptr_t>(norm->beta) & 15) == 0),
               "row product: normalisation parameters must be 16-byte aligned");
    }
    const CUtensorMap mX = tc_make_map_2d(X, M, K, ldx, RW_M);
    CUtensorMap mW[3];
    for (int i = 0; i < 3; ++i) mW[i] = tc_make_map_2d(W[i < count ? i : 0], N, K, ldw, bn);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster, (unsigned)((N + bn - 1) / bn), (unsigned)count);
    cfg.blockDim = dim3(RW_THREADS, 1, 1);
    cfg.dynamicSmemBytes = RW_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    FDK_CUDA(cudaLaunchKernelEx(&cfg, gemm_rows_kernel, mX, mW[0], mW[1], mW[2], prm));
}

const int* gemm_rows_status_address() {
    int* p = nullptr;
    FDK_CUDA(cudaGetSymbolAddress((void**)&p, g_rows_status));
    return p;
}

int gemm_rows_take_status(cudaStream_t s) {
    int v = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_rows_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (v != 0) {
        fprintf(stderr, "gemm_rows: a bounded wait gave up (code %d: 1 producer, 2 issuer, 3 converter, 4 accumulator)\n", v);
        const int zero = 0;
        cudaMemcpyToSymbolAsync(g_rows_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return v;
}

}  // namespace fdk
