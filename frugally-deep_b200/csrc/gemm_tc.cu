// tcgen05 contraction for sm_100a: C[M,N] = epilogue(A[M,K] * W[N,K]^T) with FP32 semantics through
// 3xTF32 split products.
//
// Replaces the reference's Eigen GEMM call sites (convolution.hpp:147,274; dense_layer.hpp:85;
// recurrent_ops.hpp:144,165; tensor.hpp:881) for all shapes with 16-byte aligned rows.
//
// Scheme.  Every fp32 operand x is split as x = big + small with big = rna_tf32(x) and
// small = rna_tf32(x - big); the product a*b is accumulated in FP32 as
// a_small*b_big + a_big*b_small + a_big*b_big (the a_small*b_small term, about 2^-22 relative, is dropped).
// Weight halves are precomputed once; activation halves are produced inside the kernel by a group
// of converter warps that rewrite each TMA-loaded tile in shared memory, so that all other layers
// keep working on plain fp32 tensors.
//
// Accumulation.  The tensor core adds into its TMEM accumulator with truncation (measured: the result
// of a long all-positive chain is low by about 3e-8 relative per tcgen05.mma), which over K = 4608 and
// fifty layers would drift far beyond fp32 rounding noise.  So TMEM only ever holds the sum of ONE
// 32-wide k block, built smallest terms first (8 small-term MMAs, then the 4 big-term MMAs), and the
// per-block sums are added into fp32 registers of the epilogue warps with round-to-nearest.  The k
// blocks rotate over several TMEM accumulator sets so that draining a set overlaps the MMAs of the next.
//
// Structure: persistent CTAs (one per SM), 128 x BN output tiles, warp-specialised:
//   warp 0       TMA producer: A tile (raw fp32), W_big tile, W_small tile per 32-wide k block
//   warp 1       MMA issuer: 12 tcgen05.mma.kind::tf32 (128 x BN x 8) per k block into one TMEM set
//   warps 2-5    converters: split the A tile into its TF32 halves in place
//   warps 6-13   accumulate + epilogue: two warps per TMEM lane quadrant, each owning half of the tile's
//                columns in registers: tcgen05.ld every finished k-block sum and add it; after the last
//                block apply bias / activation / BN affine / residual and store
// Every mbarrier wait is bounded; a wait that gives up sets a status word and the CTA drains and exits.
#include "kernels.cuh"
#include "device_math.cuh"

#include <cuda.h>

#include <mutex>

namespace fdk {

namespace {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;                 // fp32 elements per k block = one 128-byte swizzle row
constexpr int TC_THREADS = 448;           // 14 warps: TMA, MMA, 4 converters, 8 accumulate/epilogue
constexpr int TC_CONV_WARP0 = 2;
constexpr int TC_EPI_WARP0 = 6;
constexpr unsigned long long TC_WAIT_LIMIT_NS = 2000000000ull;  // 2 s: far beyond any legitimate wait

__device__ int g_tc_status = 0;

template <int BN>
struct TcCfg {
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;   // 16 KB
    static constexpr int B_BYTES = BN * TC_BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    static constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 6 ? 6 : (200 * 1024) / STAGE_BYTES;
    static constexpr int STG_FLOATS = 32 * 33;           // per epilogue warp: 32 x 32 transpose tile, padded rows
    static constexpr int STG_BYTES = 8 * STG_FLOATS * 4;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static constexpr int TMEM_COLS = 512;                // the whole tensor memory: one CTA per SM
    static constexpr int SETS = 512 / BN > 4 ? 4 : 512 / BN;  // accumulator sets the k blocks rotate over
    static constexpr int COLS_PER_THREAD = BN / 2;       // each epilogue thread owns half a row of the tile
};

// ---- PTX wrappers ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait suspends the warp in hardware until the phase completes or a time limit passes (hint: 20 us),
// so waiting roles do not compete for issue slots with the working ones.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after TC_WAIT_LIMIT_NS of wall time.
// Returns false when the limit ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > TC_WAIT_LIMIT_NS) break;
    }
    *abort_flag = 1;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Tiled 4-D load (no multicast).  c0 is a multiple of 32 floats, so the innermost coordinate is 16-byte
// aligned; the spatial coordinates may be negative or beyond the image: those elements read as zero.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int x, int y, int b, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(x), "r"(y), "r"(b), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t rna_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// Shared-memory matrix descriptor for a K-major tile of 128-byte rows with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor
// version 1, layout type 2 (SWIZZLE_128B).  The tile base is 1024-byte aligned.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: D = F32, A = B = TF32, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// The A operand is always described as a convolution input [B][H][W][C] (a plain matrix product is the
// 1x1 case with H = W = 1 and B = M).  An output tile of 128 rows is a box of Nb x Hb x Wb output pixels
// (powers of two, product 128); the k blocks walk the filter taps and, inside a tap, 32-channel chunks.
struct TcParams {
    float* C;
    long long ldc;
    long long M;          // output rows = B * Ho * Wo
    int N;
    int stages;
    // geometry
    int B, Ho, Wo, Cin;
    int kw, taps, cchunks;            // filter width, kh * kw, ceil(Cin / 32)
    int sy, sx, dy, dx, pad_t, pad_l;
    int wb_log, hb_log, nb_log;       // log2 of the pixel box
    int tiles_w, tiles_h, tiles_n;
    EpiDev epi;
};

// Vector epilogue of one lane: CPT consecutive columns of one output row, no activation before the affine
// step, final activation none / ReLU / clipped ReLU.  Column parameters are read as float4 (every lane reads
// the same addresses: one broadcast transaction each); residual loads of a group of 16 columns are all
// issued before the group's first store (the residual is a different live tensor than the output).
template <int CPT, bool BIAS, bool AFFINE, bool RESID>
__device__ __forceinline__ void epi_row_store(const float (&sum)[CPT], const TcParams& prm, long long row, int n0) {
    const int act2 = prm.epi.act2.kind;
    const float a_max = prm.epi.act2.p0, a_slope = prm.epi.act2.p1, a_thr = prm.epi.act2.p2;
    float* out = prm.C + row * prm.ldc + n0;
    const float* res = RESID ? prm.epi.residual + row * prm.epi.ldr + n0 : nullptr;
    float4 rn[4];  // residual of the next group: loaded one group ahead of its use
    if (RESID) {
#pragma unroll
        for (int i = 0; i < 4; ++i) rn[i] = __ldg(reinterpret_cast<const float4*>(res + 4 * i));
    }
#pragma unroll
    for (int g = 0; g < CPT; g += 16) {
        float4 r4[4];
        if (RESID) {
#pragma unroll
            for (int i = 0; i < 4; ++i) r4[i] = rn[i];
            if (g + 16 < CPT) {
#pragma unroll
                for (int i = 0; i < 4; ++i) rn[i] = __ldg(reinterpret_cast<const float4*>(res + g + 16 + 4 * i));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = g + 4 * i;
            float v[4] = {sum[j], sum[j + 1], sum[j + 2], sum[j + 3]};
            if (BIAS) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(prm.epi.bias + n0 + j));
                v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
            }
            if (AFFINE) {
                const float4 s = __ldg(reinterpret_cast<const float4*>(prm.epi.scale + n0 + j));
                const float4 t = __ldg(reinterpret_cast<const float4*>(prm.epi.shift + n0 + j));
                v[0] = __fadd_rn(__fmul_rn(v[0], s.x), t.x); v[1] = __fadd_rn(__fmul_rn(v[1], s.y), t.y);
                v[2] = __fadd_rn(__fmul_rn(v[2], s.z), t.z); v[3] = __fadd_rn(__fmul_rn(v[3], s.w), t.w);
            }
            if (RESID) { v[0] += r4[i].x; v[1] += r4[i].y; v[2] += r4[i].z; v[3] += r4[i].w; }
            if (act2 == ACT_RELU) {
#pragma unroll
                for (int t = 0; t < 4; ++t) v[t] = fmaxf(0.0f, v[t]);
            } else if (act2 == ACT_RELU_GEN) {  // relu_layer.hpp:40-46
#pragma unroll
                for (int t = 0; t < 4; ++t) v[t] = v[t] >= a_max ? a_max : (a_thr <= v[t] ? v[t] : a_slope * (v[t] - a_thr));
            }
            *reinterpret_cast<float4*>(out + j) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapWb,
               const __grid_constant__ CUtensorMap mapWs, TcParams prm) {
    using Cfg = TcCfg<BN>;
    const int STAGES = prm.stages;  // 2..Cfg::STAGES; fewer stages leave more of the unified L1 to the store path
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw_addr);
    // layout: [stage][A | As | Wb | Ws], then the epilogue staging tiles, then barriers
    uint8_t* bar_mem = smem + STAGES * Cfg::STAGE_BYTES + Cfg::STG_BYTES;
    const uint32_t bar_base = smem_u32(bar_mem);
    auto full_bar = [&](int s) { return bar_base + (uint32_t)s * 8u; };
    auto conv_bar = [&](int s) { return bar_base + (uint32_t)(STAGES + s) * 8u; };
    auto empty_bar = [&](int s) { return bar_base + (uint32_t)(2 * STAGES + s) * 8u; };
    constexpr int SETS = Cfg::SETS;
    auto tfull_bar = [&](int a) { return bar_base + (uint32_t)(3 * STAGES + a) * 8u; };
    auto tempty_bar = [&](int a) { return bar_base + (uint32_t)(3 * STAGES + SETS + a) * 8u; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + (3 * STAGES + 2 * SETS) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + (3 * STAGES + 2 * SETS) * 8 + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(conv_bar(s), 4);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < SETS; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), (uint32_t)Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long m_tiles = (long long)prm.tiles_n * prm.tiles_h * prm.tiles_w;
    const int n_tiles = (prm.N + BN - 1) / BN;
    const long long tiles = m_tiles * n_tiles;
    const int k_blocks = prm.taps * prm.cchunks;

    auto stage_ptr = [&](int s) { return base + (uint32_t)s * (uint32_t)Cfg::STAGE_BYTES; };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const long long mt = tile / n_tiles;
                const int n0 = (int)(tile % n_tiles) * BN;
                const int tw = (int)(mt % prm.tiles_w);
                const int th = (int)((mt / prm.tiles_w) % prm.tiles_h);
                const int tn = (int)(mt / ((long long)prm.tiles_w * prm.tiles_h));
                // first input pixel (before the tap offset) and first image of the tile's pixel box
                const int x0 = (tw << prm.wb_log) * prm.sx - prm.pad_l;
                const int y0 = (th << prm.hb_log) * prm.sy - prm.pad_t;
                const int b0 = tn << prm.nb_log;
                int tap = 0, cc = 0, ky = 0, kx = 0;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 1)) { ok = false; break; }
                    const uint32_t sp = stage_ptr(stage);
                    mbar_arrive_expect_tx(full_bar(stage), (uint32_t)(Cfg::A_BYTES + 2 * Cfg::B_BYTES));
                    // channels [cc*32, +32) of the input pixels under filter tap (ky, kx); zero outside the image
                    tma_load_4d(sp, &mapA, cc * TC_BK, x0 + kx * prm.dx, y0 + ky * prm.dy, b0, full_bar(stage));
                    const int wk = tap * prm.Cin + cc * TC_BK;  // the same slice of every filter
                    tma_load_2d(sp + 2 * Cfg::A_BYTES, &mapWb, wk, n0, full_bar(stage));
                    tma_load_2d(sp + 2 * Cfg::A_BYTES + Cfg::B_BYTES, &mapWs, wk, n0, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    if (++cc == prm.cchunks) {
                        cc = 0;
                        ++tap;
                        if (++kx == prm.kw) { kx = 0; ++ky; }
                    }
                }
            }
            if (!ok) {
                // drain: give copies already issued a bounded time to land before the CTA exits
                for (int s = 0; s < STAGES; ++s)
                    for (uint32_t it = 0; it < 4096 && !mbar_test(full_bar(s), 0) && !mbar_test(full_bar(s), 1); ++it) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(TC_BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < k_blocks; ++kb) {
                    // one TMEM set per k block: it is drained into registers by the epilogue warps
                    if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, 2)) { ok = false; break; }
                    if (!mbar_wait(conv_bar(stage), phase, abort_flag, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                    const uint32_t sp = stage_ptr(stage);
                    const uint64_t da_big = make_smem_desc(sp);
                    const uint64_t da_small = make_smem_desc(sp + Cfg::A_BYTES);
                    const uint64_t db_big = make_smem_desc(sp + 2 * Cfg::A_BYTES);
                    const uint64_t db_small = make_smem_desc(sp + 2 * Cfg::A_BYTES + Cfg::B_BYTES);
                    // small terms first, so that the truncating accumulator rounds against small partial sums
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 8; ++kk) {
                        const uint64_t koff = (uint64_t)((kk * 8 * 4) >> 4);  // 32 bytes per K=8 step, in 16-byte units
                        umma_tf32(d_tmem, da_small + koff, db_big + koff, idesc, kk > 0 ? 1u : 0u);
                        umma_tf32(d_tmem, da_big + koff, db_small + koff, idesc, 1u);
                    }
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 8; ++kk) {
                        const uint64_t koff = (uint64_t)((kk * 8 * 4) >> 4);
                        umma_tf32(d_tmem, da_big + koff, db_big + koff, idesc, 1u);
                    }
                    umma_commit(empty_bar(stage));
                    umma_commit(tfull_bar(acc));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    if (++acc == SETS) { acc = 0; acc_phase ^= 1u; }
                }
            }
        }
    } else if (warp >= TC_EPI_WARP0) {
        // ---------------- accumulate + epilogue ----------------
        constexpr int CPT = Cfg::COLS_PER_THREAD;
        const int q = warp & 3;                           // TMEM lane quadrant this warp may read
        const int half = (warp - TC_EPI_WARP0) >> 2;      // which half of the tile's columns this warp owns
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool fast_epi = ((prm.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(prm.C) & 15) == 0) && prm.epi.act1.kind == ACT_NONE &&
                              prm.epi.act2.kind <= ACT_RELU_GEN &&
                              (prm.epi.residual == nullptr || (((prm.epi.ldr & 3) == 0) && ((reinterpret_cast<uintptr_t>(prm.epi.residual) & 15) == 0)));
        const int epi_mode = (prm.epi.bias ? 1 : 0) | (prm.epi.scale ? 2 : 0) | (prm.epi.residual ? 4 : 0);
        // per-warp staging tile (32 rows x 33 floats) used to turn "one row per lane" into "one column per lane"
        float* stg = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES) + (warp - TC_EPI_WARP0) * Cfg::STG_FLOATS;
        for (long long tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const long long mt = tile / n_tiles;
            const int n0 = (int)(tile % n_tiles) * BN + half * CPT;
            // output row of this lane: tile row r = (image, y, x) inside the pixel box, x fastest
            long long row = -1;
            {
                const int tw = (int)(mt % prm.tiles_w);
                const int th = (int)((mt / prm.tiles_w) % prm.tiles_h);
                const int tn = (int)(mt / ((long long)prm.tiles_w * prm.tiles_h));
                const int r = q * 32 + lane;
                const int ox = (tw << prm.wb_log) + (r & ((1 << prm.wb_log) - 1));
                const int oy = (th << prm.hb_log) + ((r >> prm.wb_log) & ((1 << prm.hb_log) - 1));
                const int bi = (tn << prm.nb_log) + (r >> (prm.wb_log + prm.hb_log));
                if (ox < prm.Wo && oy < prm.Ho && bi < prm.B) row = ((long long)bi * prm.Ho + oy) * prm.Wo + ox;
            }
            // pull this lane's part of the residual tile into L2 while the k loop runs
            if (prm.epi.residual && row >= 0) {
                const float* rp = prm.epi.residual + row * prm.epi.ldr + n0;
#pragma unroll
                for (int j = 0; j < CPT; j += 32)
                    if (n0 + j < prm.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + j));
            }
            float sum[CPT];
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * CPT + c0), r);
                    tmem_ld_wait();
                    if (kb == 0) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) sum[c0 + j] = __uint_as_float(r[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) sum[c0 + j] += __uint_as_float(r[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                if (++acc == SETS) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) break;
            // Epilogue.  A lane holds 32 consecutive columns of ONE row; written like that, every store of a
            // warp would touch 32 different rows.  Each 32 x 32 block goes through the staging tile instead
            // (row stride 33 floats: conflict-free both ways) and comes back with one COLUMN per lane, so that
            // each global access of the warp covers 128 contiguous bytes of one output row.
            if (fast_epi && n0 + CPT <= prm.N) {
                // common case: straight-line vector epilogue, each lane stores its own row as float4s
                if (row >= 0) {
                    switch (epi_mode) {
                        case 0: epi_row_store<CPT, false, false, false>(sum, prm, row, n0); break;
                        case 1: epi_row_store<CPT, true, false, false>(sum, prm, row, n0); break;
                        case 2: epi_row_store<CPT, false, true, false>(sum, prm, row, n0); break;
                        case 3: epi_row_store<CPT, true, true, false>(sum, prm, row, n0); break;
                        case 4: epi_row_store<CPT, false, false, true>(sum, prm, row, n0); break;
                        case 5: epi_row_store<CPT, true, false, true>(sum, prm, row, n0); break;
                        case 6: epi_row_store<CPT, false, true, true>(sum, prm, row, n0); break;
                        default: epi_row_store<CPT, true, true, true>(sum, prm, row, n0); break;
                    }
                }
                continue;
            }
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += 32) {
                if (n0 + c0 >= prm.N) break;  // warp-uniform
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = sum[c0 + j];
                __syncwarp();
                const int col = n0 + c0 + lane;
                // eight rows at a time: all residual loads of a group are issued before anything is stored
                // (the residual never aliases the output: it is a different live tensor of the plan)
                for (int r0 = 0; r0 < 32; r0 += 8) {
                    float res[8];
                    long long orow[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        orow[i] = __shfl_sync(0xffffffffu, row, r0 + i);  // output row of tile row r0 + i (-1: outside)
                        res[i] = (prm.epi.residual && orow[i] >= 0 && col < prm.N) ? __ldg(prm.epi.residual + orow[i] * prm.epi.ldr + col) : 0.f;
                    }
                    if (col < prm.N) {
                        const float b = prm.epi.bias ? __ldg(prm.epi.bias + col) : 0.f;
                        const float sc = prm.epi.scale ? __ldg(prm.epi.scale + col) : 1.f;
                        const float sh = prm.epi.scale ? __ldg(prm.epi.shift + col) : 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            if (orow[i] >= 0) {
                                float v = stg[(r0 + i) * 33 + lane];
                                if (prm.epi.bias) v += b;
                                v = act_apply(prm.epi.act1, v);
                                if (prm.epi.scale) v = __fadd_rn(__fmul_rn(v, sc), sh);
                                if (prm.epi.residual) v += res[i];
                                prm.C[orow[i] * prm.ldc + col] = act_apply(prm.epi.act2, v);
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- converters (warps 2-5): A tile -> TF32 high half in place, low half beside it ----------------
        const int ct = threadIdx.x - TC_CONV_WARP0 * 32;  // 0..127
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, 5)) { ok = false; break; }
                uint8_t* sp = smem + (size_t)stage * Cfg::STAGE_BYTES;
                float4* a_big = reinterpret_cast<float4*>(sp);
                uint4* a_big_u = reinterpret_cast<uint4*>(sp);
                uint4* a_small_u = reinterpret_cast<uint4*>(sp + Cfg::A_BYTES);
#pragma unroll
                for (int it = 0; it < Cfg::A_BYTES / 16 / 128; ++it) {
                    const int idx = it * 128 + ct;
                    const float4 v = a_big[idx];
                    uint4 hi, lo;
                    hi.x = rna_tf32(v.x); hi.y = rna_tf32(v.y); hi.z = rna_tf32(v.z); hi.w = rna_tf32(v.w);
                    lo.x = rna_tf32(v.x - __uint_as_float(hi.x)); lo.y = rna_tf32(v.y - __uint_as_float(hi.y));
                    lo.z = rna_tf32(v.z - __uint_as_float(hi.z)); lo.w = rna_tf32(v.w - __uint_as_float(hi.w));
                    a_big_u[idx] = hi;
                    a_small_u[idx] = lo;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(conv_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)Cfg::TMEM_COLS);
    }
}

__global__ void split_tf32_kernel(const float* __restrict__ w, float* __restrict__ big, float* __restrict__ small, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float x = w[i];
        const float hi = __uint_as_float(rna_tf32(x));
        big[i] = hi;
        small[i] = __uint_as_float(rna_tf32(x - hi));
    }
}

// ---- host side: tensor maps -------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
        else cudaGetLastError();
    });
    return fn;
}

// 2-D map over a row-major [rows][cols] fp32 matrix with row stride ld (floats): box = 32 columns x box_rows.
CUtensorMap make_map_2d(const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeFn enc = get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return m;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// 4-D map over a channels-last input [B][H][W][pix] (pix = floats per pixel, >= C): box = 32 channels x a
// (Wb, Hb, Nb) pixel box; with strides sx / sy only every sx-th / sy-th pixel is fetched.
CUtensorMap make_map_4d(const float* base, const ConvTcGeom& g, int wb, int hb, int nb) {
    EncodeFn enc = get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap m;
    cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.B};
    cuuint64_t strides[3] = {(cuuint64_t)g.pix * sizeof(float), (cuuint64_t)g.W * g.pix * sizeof(float),
                             (cuuint64_t)g.H * g.W * g.pix * sizeof(float)};
    cuuint32_t box[4] = {(cuuint32_t)TC_BK, (cuuint32_t)(wb * g.sx), (cuuint32_t)(hb * g.sy), (cuuint32_t)nb};
    cuuint32_t estr[4] = {1, (cuuint32_t)g.sx, (cuuint32_t)g.sy, 1};
    if (g.win_stride > 0) {
        // overlapping windows: dimension 1 counts output columns, win_stride floats apart, each 32 floats long
        dims[0] = TC_BK; dims[1] = (cuuint64_t)g.Wo;
        strides[0] = (cuuint64_t)g.win_stride * sizeof(float);
        box[1] = (cuuint32_t)wb; estr[1] = 1;
    }
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (4-D) failed with code " + std::to_string((int)r));
    return m;
}

// Pixel box of an output tile: powers of two (Wb, Hb, Nb) with product 128 that need the fewest tiles.
void choose_box(const ConvTcGeom& g, int& wb_log, int& hb_log, int& nb_log) {
    int64_t best = -1;
    for (int w = 0; w <= 7; ++w) {
        if ((1 << w) * g.sx > 256) break;
        for (int h = 0; w + h <= 7; ++h) {
            if ((1 << h) * g.sy > 256) break;
            const int n = 7 - w - h;
            const int64_t t = ((g.Wo + (1 << w) - 1) >> w) * (int64_t)((g.Ho + (1 << h) - 1) >> h) * ((g.B + (1 << n) - 1) >> n);
            if (best < 0 || t < best || (t == best && w > wb_log)) { best = t; wb_log = w; hb_log = h; nb_log = n; }
        }
    }
}

template <int BN>
void launch_tc(const float* in, const ConvTcGeom& g, const float* Wb, const float* Ws, int64_t ldw, float* C, int64_t ldc, int N,
               const Epilogue& e, cudaStream_t s) {
    using Cfg = TcCfg<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        FDK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set = true;
    }
    TcParams prm;
    int wb = 0, hb = 0, nb = 7;
    choose_box(g, wb, hb, nb);
    prm.wb_log = wb; prm.hb_log = hb; prm.nb_log = nb;
    prm.tiles_w = (g.Wo + (1 << wb) - 1) >> wb;
    prm.tiles_h = (g.Ho + (1 << hb) - 1) >> hb;
    prm.tiles_n = (int)((g.B + (1 << nb) - 1) >> nb);
    const bool rowwin = g.win_stride > 0;
    const int64_t K = rowwin ? (int64_t)g.kh * TC_BK : (int64_t)g.kh * g.kw * g.C;
    const CUtensorMap mA = make_map_4d(in, g, 1 << wb, 1 << hb, 1 << nb);
    const CUtensorMap mWb = make_map_2d(Wb, N, K, ldw, BN);
    const CUtensorMap mWs = make_map_2d(Ws, N, K, ldw, BN);
    prm.C = C; prm.ldc = ldc; prm.M = g.B * g.Ho * g.Wo; prm.N = N; prm.epi = to_dev(e);
    prm.B = (int)g.B; prm.Ho = g.Ho; prm.Wo = g.Wo; prm.Cin = g.C;
    prm.kw = g.kw; prm.taps = g.kh * g.kw; prm.cchunks = (g.C + TC_BK - 1) / TC_BK;
    prm.sy = g.sy; prm.sx = g.sx; prm.dy = g.dy; prm.dx = g.dx; prm.pad_t = g.pad_t; prm.pad_l = g.pad_l;
    if (rowwin) {  // one k block per filter row; x coordinates count output columns
        prm.Cin = TC_BK; prm.kw = 1; prm.taps = g.kh; prm.cchunks = 1;
        prm.sx = 1; prm.dx = 1; prm.dy = 1; prm.pad_t = 0; prm.pad_l = 0;
    }
    // Short contractions are bound by the output stream, not by operand staging: two stages suffice.
    const int k_blocks = prm.taps * prm.cchunks;
    prm.stages = k_blocks <= 4 ? 2 : Cfg::STAGES;
    static const int forced = [] { const char* v = getenv("FDK_TC_STAGES"); return v ? atoi(v) : 0; }();
    if (forced >= 2 && forced <= Cfg::STAGES) prm.stages = forced;
    const int smem_bytes = prm.stages * Cfg::STAGE_BYTES + Cfg::STG_BYTES + 1024 + 256;
    const int64_t tiles = (int64_t)prm.tiles_w * prm.tiles_h * prm.tiles_n * ((N + BN - 1) / BN);
    const int grid = (int)std::min<int64_t>(tiles, sm_count());
    gemm_tc_kernel<BN><<<grid, TC_THREADS, smem_bytes, s>>>(mA, mWb, mWs, prm);
    FDK_CUDA(cudaGetLastError());
}

}  // namespace

bool conv_tc_supported(const ConvTcGeom& g, int N, int64_t ldw, const void* in, const void* W) {
    if (g.B <= 0 || N <= 0 || g.C <= 0 || g.Ho <= 0 || g.Wo <= 0) return false;
    if ((g.C & 3) || (g.pix & 3) || (ldw & 3)) return false;
    if (g.win_stride > 0 && ((g.win_stride & 3) || g.kw * g.C > TC_BK)) return false;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return false;
    if (g.sx < 1 || g.sx > 8 || g.sy < 1 || g.sy > 8) return false;
    if (g.B > 0x7fffffffLL || g.B * g.Ho * g.Wo > 0x7fffffffLL) return false;
    return get_encode() != nullptr;
}

void launch_conv_tc(const float* in, const ConvTcGeom& g, const float* Wbig, const float* Wsmall, int64_t ldw, float* C, int64_t ldc,
                    int N, const Epilogue& e, cudaStream_t s) {
    if (N <= 64) launch_tc<64>(in, g, Wbig, Wsmall, ldw, C, ldc, N, e, s);
    else launch_tc<128>(in, g, Wbig, Wsmall, ldw, C, ldc, N, e, s);
}

static ConvTcGeom gemm_geom(int64_t M, int K, int64_t lda) {
    ConvTcGeom g;
    g.B = M; g.H = 1; g.W = 1; g.C = K; g.pix = lda; g.Ho = 1; g.Wo = 1;
    return g;
}

bool gemm_tc_supported(int64_t M, int N, int K, int64_t lda, int64_t ldw, const void* A, const void* W) {
    if (M <= 0 || K <= 0) return false;
    return conv_tc_supported(gemm_geom(M, K, lda), N, ldw, A, W);
}

void launch_gemm_tc(const float* A, int64_t lda, const float* Wbig, const float* Wsmall, int64_t ldw, float* C, int64_t ldc, int64_t M,
                    int N, int K, const Epilogue& e, cudaStream_t s) {
    launch_conv_tc(A, gemm_geom(M, K, lda), Wbig, Wsmall, ldw, C, ldc, N, e, s);
}

int gemm_tc_take_status(cudaStream_t s) {
    int v = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbolAsync(g_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return v;
}

void launch_split_tf32(const float* w, float* big, float* small, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    int64_t g = (n + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    split_tf32_kernel<<<(unsigned)g, 256, 0, s>>>(w, big, small, (long long)n);
    FDK_CUDA(cudaGetLastError());
}

}  // namespace fdk
