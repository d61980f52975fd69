// tcgen05 contraction for sm_100a: C[M,N] = epilogue(A[M,K] * W[N,K]^T) with FP32 semantics through
// 3xTF32 split products.
//
// Replaces the reference's Eigen GEMM call sites (convolution.hpp:147,274; dense_layer.hpp:85;
// recurrent_ops.hpp:144,165; tensor.hpp:881) for all shapes with 16-byte aligned rows.
//
// Scheme.  Every fp32 operand x is split as x = big + small and the product a*b is accumulated in FP32 as
// a_small*b_big + a_big*b_small + a_big*b_big (the a_small*b_small term, about 2^-22 relative, is dropped).
// Weight halves are precomputed once at load with round-to-nearest (big = rna_tf32(w), small = rna_tf32(w - big)).
// Activation halves are produced inside the kernel by converter warps, by masking (big = x with the 13 low
// mantissa bits cleared, small = x - big, exact), and go straight into TENSOR MEMORY: the A operand of every
// MMA is read from TMEM, only W is read from shared memory, so all other layers keep working on plain fp32
// tensors and the shared-memory bandwidth is left to the W tiles.
//
// Accumulation.  The tensor core adds into its TMEM accumulator with truncation (measured: the result of a
// long all-positive chain is low by about 3e-8 relative per tcgen05.mma), which over K = 4608 and fifty layers
// would drift far beyond fp32 rounding noise.  So a TMEM accumulator set only ever holds the sum of TC_GROUP = 2
// 32-wide k blocks (per block: the 8 small-term MMAs first, then the 4 big-term MMAs), and these partial sums
// are added into fp32 registers of the epilogue warps with round-to-nearest.  There are two accumulator sets,
// one per MMA issuer, so that draining one overlaps the MMAs into the other.
//
// Structure: persistent CTAs (one per SM, 512 threads), 128 x BN output tiles (BN = 64 or 128), warp-specialised:
//   warp 0       TMA producer of the raw fp32 A tiles (4-D tensor map over the channels-last input: one k block
//                is one filter tap x 32 channels; zero padding comes from out-of-range coordinates)
//   warps 1-2    MMA issuers: alternate groups of k blocks, issuer i into accumulator set i; per k block 12
//                tcgen05.mma.kind::tf32 (128 x BN x 8), then the commit that frees the block's A slot and W stage
//   warp 3       TMA producer of the W tiles (W_big | W_small per stage; kept resident for short contractions)
//   warps 4-7    converters: one warp per TMEM lane quadrant; a lane reads its row of the raw tile from shared
//                memory and writes big | small into the 64 TMEM columns of the k block's A slot (tcgen05.st)
//   warps 8-15   accumulate + epilogue: two warps per TMEM lane quadrant, each owning half of the tile's columns
//                in registers: tcgen05.ld every finished group sum and add it; after the last group apply
//                bias / BN affine / residual / activation in a shared-memory staging block and store it by TMA
// Registers are re-divided between the roles with setmaxnreg.  Every mbarrier wait is bounded; a wait that gives
// up sets a status word and the CTA drains its copies, frees its tensor memory and exits.
//
// The same walk serves, through the geometry the host passes (ConvTcGeom):
//   * dilated convolutions (the tap walk steps dy, dx pixels) and negative padding;
//   * 3-D convolutions (convolution3d.hpp:437-506): the input is described as B * D images, a tile lies within one
//     output slice, taps run over (kz, ky, kx), and a tap on a slice outside the volume loads an all-zero tile from a
//     row coordinate beyond the image;
//   * transposed convolutions (convolution.hpp:443-469), one launch per output phase: sub-filter, pad = -shift, and
//     output pixels that lie sx * N, sy * Wo * N floats apart (the output and residual tensor maps carry the strides);
//   * an LSTM time step (recurrent_ops.hpp:164-181) as the kernel instance CELL = true, whose epilogue forms the gate
//     pre-activations in the staging buffers and finishes the cell instead of storing them.
#include "kernels.cuh"
#include "device_math.cuh"
#include "pdl.cuh"
#include "tc_ptx.cuh"
#include "tc_maps.hpp"

#include <cuda.h>

#include <mutex>

namespace fdk {

// ---- host side: tensor maps -------------------------------------------------------------------------
EncodeFn tc_get_encode() {
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
CUtensorMap tc_make_map_2d(const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeFn enc = tc_get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};   // 32 floats = one 128-byte swizzle row
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return m;
}

// SM count of the current device (looked up once per device).
int tc_sm_count() {
    static std::mutex mu;
    static int per_device[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    const bool cached = dev >= 0 && dev < 64;
    if (cached && per_device[dev] > 0) return per_device[dev];
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    if (cached) per_device[dev] = n;
    return n;
}

namespace {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;                 // fp32 elements per k block = one 128-byte swizzle row
constexpr int TC_GROUP = 2;               // k blocks summed inside one TMEM accumulator set before it is drained
// Warp roles (on warpgroup boundaries because setmaxnreg works per warpgroup):
//   warps 0-3    TMA producer of raw A tiles, two MMA issuers, TMA producer of W tiles
//   then         converters: TC_TEAMS teams of four warps (one warp per TMEM lane quadrant), taking k blocks in turn
//   last 8       accumulate + epilogue: two warps per TMEM lane quadrant, each owning half of the tile's columns
// The registers are re-divided between the roles, so that the epilogue warps hold their accumulators without
// spilling.  The pool that setmaxnreg draws from is what the CTA was given at launch (threads x the kernel's
// register count), not the SM's whole register file: a split that adds up to more makes setmaxnreg.inc wait
// forever.
constexpr int TC_TEAMS = 1;               // one converter team (a second team measured no faster)
constexpr int TC_CONV_WARP0 = 4;
constexpr int TC_EPI_WARP0 = TC_CONV_WARP0 + 4 * TC_TEAMS;
constexpr int TC_THREADS = (TC_EPI_WARP0 + 8) * 32;
// registers per thread at launch (65536 / threads, rounded down to a multiple of 8) and after the split
constexpr int TC_REGS_LAUNCH = TC_TEAMS == 1 ? 128 : 96;
constexpr int TC_REGS_CONTROL = TC_TEAMS == 1 ? 56 : 48, TC_REGS_CONVERT = 112, TC_REGS_EPILOGUE = TC_TEAMS == 1 ? 168 : 104;
static_assert(128 * TC_REGS_CONTROL + 128 * TC_TEAMS * TC_REGS_CONVERT + 256 * TC_REGS_EPILOGUE <= TC_THREADS * TC_REGS_LAUNCH, "register budget");
constexpr unsigned long long TC_WAIT_LIMIT_NS = 2000000000ull;  // 2 s: far beyond any legitimate wait

__device__ int g_tc_status = 0;
// Diagnostics of the wait that gave up: the launch (written by every launch's first thread) and the waiter.
__device__ int g_tc_launch[8];
__device__ int g_tc_diag[16];

template <int BN>
struct TcCfg {
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;   // 16 KB
    static constexpr int B_BYTES = BN * TC_BK * 4;
    static constexpr int W_BYTES = 2 * B_BYTES;          // one stage of the W ring: W_big | W_small
    static constexpr int A_STAGES = 4;                   // most stages of the raw A ring
    static constexpr int STAGES = BN > 64 ? 4 : 6;       // most stages of the W ring = A slots in tensor memory
    // Epilogue staging: every epilogue warp owns `nbuf` (1 or 2) buffers of 32 rows x 32 floats (4 KB, 128-byte
    // rows in the 128-byte swizzle), the unit of the output TMA stores and residual TMA loads.
    static constexpr int STG_BUF_BYTES = 32 * 32 * 4;
    static constexpr int BAR_BYTES = 640;
    static constexpr int MAX_SMEM = 227 * 1024;
    // epilogue column parameters: bias | scale | shift of BN / 2 columns, one block per epilogue warp, or one per
    // column half when every tile of a CTA has the same columns
    static constexpr int PRM_BLOCK_BYTES = 3 * (BN / 2) * 4;
    static constexpr int smem_bytes(int a_stages, int w_stages, int nbuf, bool shared_prm) {
        return a_stages * A_BYTES + w_stages * W_BYTES + 8 * nbuf * STG_BUF_BYTES + (shared_prm ? 2 : 8) * PRM_BLOCK_BYTES + BAR_BYTES;
    }
    static constexpr int TMEM_COLS = 512;                // the whole tensor memory: one CTA per SM
    static constexpr int SETS = 2;                       // accumulator sets: one per MMA issuer
    static constexpr int A_SLOT_COLS = 2 * TC_BK;        // TF32 halves of one A k block: 32 + 32 columns
    static constexpr int A_COL0 = SETS * BN;             // first column of the A slots (one slot per stage)
    static_assert(A_COL0 + STAGES * A_SLOT_COLS <= TMEM_COLS, "tensor memory budget");
    static constexpr int COLS_PER_THREAD = BN / 2;       // each epilogue thread owns half a row of the tile
};

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
    if (atomicCAS(&g_tc_status, 0, code) == 0) {
        for (int i = 0; i < 8; ++i) g_tc_diag[i] = g_tc_launch[i];
        g_tc_diag[8] = code; g_tc_diag[9] = (int)blockIdx.x; g_tc_diag[10] = (int)threadIdx.x;
        g_tc_diag[11] = (int)bar; g_tc_diag[12] = (int)parity; g_tc_diag[13] = (int)gridDim.x;
    }
    return false;
}
// tcgen05.mma.kind::tf32: D[128 x BN] (+)= A[128 x 8] * B[BN x 8]^T with the A operand read from tensor memory
// (lane = row, one value per 32-bit column) and B from a K-major shared-memory tile.
// The MMAs of one 32-wide k block in two straight-line sequences with all address arithmetic inside (the issuing
// thread is the bottleneck of short MMAs: every instruction it executes between two tcgen05.mma counts).
// b_*_lo / b_hi: low and high words of the shared-memory descriptors of W_big and W_small; a K step of 8 values
// is 8 TMEM columns of A and 2 descriptor units (32 bytes) of W.
// Cross terms, small first: for each K step  D (+)= A_small * W_big,  D += A_big * W_small.
__device__ __forceinline__ void umma_cross8(uint32_t d, uint32_t a_big, uint32_t a_small, uint32_t b_big_lo, uint32_t b_small_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, pt;\n\t.reg .b64 db;\n\t.reg .b32 t0, t1, z;\n\t"
        "setp.ne.b32 p, %7, 0;\n\t"
        "setp.eq.b32 pt, %7, %7;\n\t"
        "mov.b32 z, 0;\n\t"
        "mov.b64 db, {%3, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], db, %6, {z, z, z, z}, p;\n\t"
        "mov.b64 db, {%4, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %2, 8;\n\t add.u32 t1, %3, 2;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 8;\n\t add.u32 t1, %4, 2;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %2, 16;\n\t add.u32 t1, %3, 4;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 16;\n\t add.u32 t1, %4, 4;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %2, 24;\n\t add.u32 t1, %3, 6;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 24;\n\t add.u32 t1, %4, 6;\n\t mov.b64 db, {t1, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %6, {z, z, z, z}, pt;\n\t}"
        ::"r"(d), "r"(a_big), "r"(a_small), "r"(b_big_lo), "r"(b_small_lo), "r"(b_hi), "r"(idesc), "r"(accumulate_first)
        : "memory");
}
// Main terms:  D += A_big * W_big  for the four K steps.
__device__ __forceinline__ void umma_main4(uint32_t d, uint32_t a_big, uint32_t b_big_lo, uint32_t b_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pt;\n\t.reg .b64 db;\n\t.reg .b32 t0, t1, z;\n\t"
        "setp.eq.b32 pt, %4, %4;\n\t"
        "mov.b32 z, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 8;\n\t add.u32 t1, %2, 2;\n\t mov.b64 db, {t1, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %4, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 16;\n\t add.u32 t1, %2, 4;\n\t mov.b64 db, {t1, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %4, {z, z, z, z}, pt;\n\t"
        "add.u32 t0, %1, 24;\n\t add.u32 t1, %2, 6;\n\t mov.b64 db, {t1, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [t0], db, %4, {z, z, z, z}, pt;\n\t}"
        ::"r"(d), "r"(a_big), "r"(b_big_lo), "r"(b_hi), "r"(idesc)
        : "memory");
}
// The A operand is always described as a convolution input [B][H][W][C] (a plain matrix product is the
// 1x1 case with H = W = 1 and B = M).  An output tile of 128 rows is a box of Nb x Hb x Wb output pixels
// (powers of two, product 128); the k blocks walk the filter taps and, inside a tap, 32-channel chunks.
struct TcParams {
    float* C;
    long long ldc;
    long long out_sx, out_sy, out_sb;  // floats between output pixels in x, in y, between samples (dense: ldc, Wo * ldc, Ho * Wo * ldc)
    int spread;                        // 1: the output pixels are not dense; a residual then has the output's layout
    long long M;          // output rows = B * Ho * Wo
    int N;
    int stages;           // A slots in tensor memory (= W ring stages unless the weights are stationary)
    int a_stages;         // raw A ring stages
    int w_stages;         // W stages in shared memory
    int w_stationary;     // 1: the CTA's tiles all use the same W tiles, loaded once into stages 0 .. k_blocks - 1
    // geometry
    int B, Ho, Wo, Cin;
    int kw, taps, cchunks;            // filter width, kd * kh * kw, ceil(Cin / 32)
    int kh;                           // filter rows (after kh * kw taps the walk moves on to the next input slice)
    int Din, Do, sz, pad_f;           // 3-D convolution: input / output slices per sample, slice stride, front padding (2-D: 1, 1, 1, 0)
    int y_none;                       // a row coordinate beyond the input: what a tap on a slice that does not exist loads (zeros)
    int sy, sx, dy, dx, pad_t, pad_l;
    int wb_log, hb_log, nb_log;       // log2 of the pixel box
    int tiles_w, tiles_h, tiles_n;
    int nbuf;                         // staging buffers per epilogue warp (1 or 2)
    int tma_epi;                      // 1: output (and residual) rows are 16-byte aligned: TMA epilogue
    EpiDev epi;
    // LSTM step (kernel instance with CELL = true): state tensors [B][cell_U]; cell_out may be null
    float* cell_c;
    float* cell_h;
    float* cell_out;
    long long cell_out_stride;
    int cell_U;
};

// Epilogue arithmetic of one lane on a block of 32 consecutive columns of its output row, written into the
// lane's 128-byte row of a staging buffer (16-byte chunk c of row r sits at chunk c ^ (r & 7): the 128-byte
// swizzle of the tensor maps, which also makes the warp's float4 accesses conflict-free).  With a residual the
// buffer holds the residual block (brought in by TMA) and is overwritten in place by the result.
// One copy of the code serves every layer: bias, scale and shift always apply (0, 1, 0 when the layer has
// none; they come from the warp's parameter block in shared memory), residual and clipping are warp-uniform
// branches.  (Specialising this by template made the kernel several hundred KB of code and instruction
// fetch its bottleneck.)
template <int CPT, int J0>
__device__ __forceinline__ void epi_block(const float (&sum)[CPT], const float* __restrict__ wprm, uint8_t* __restrict__ row_ptr, int lane,
                                          bool has_res, bool clip, float lo, float hi) {
    // In phases, every phase's shared-memory loads ahead of its arithmetic and all stores last, so that no load
    // has to wait behind a store it might alias.
    float v[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 b = *reinterpret_cast<const float4*>(wprm + J0 + 4 * c);
        v[4 * c + 0] = sum[J0 + 4 * c + 0] + b.x; v[4 * c + 1] = sum[J0 + 4 * c + 1] + b.y;
        v[4 * c + 2] = sum[J0 + 4 * c + 2] + b.z; v[4 * c + 3] = sum[J0 + 4 * c + 3] + b.w;
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 sc = *reinterpret_cast<const float4*>(wprm + CPT + J0 + 4 * c);
        v[4 * c + 0] = __fmul_rn(v[4 * c + 0], sc.x); v[4 * c + 1] = __fmul_rn(v[4 * c + 1], sc.y);
        v[4 * c + 2] = __fmul_rn(v[4 * c + 2], sc.z); v[4 * c + 3] = __fmul_rn(v[4 * c + 3], sc.w);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 sh = *reinterpret_cast<const float4*>(wprm + 2 * CPT + J0 + 4 * c);
        v[4 * c + 0] = __fadd_rn(v[4 * c + 0], sh.x); v[4 * c + 1] = __fadd_rn(v[4 * c + 1], sh.y);
        v[4 * c + 2] = __fadd_rn(v[4 * c + 2], sh.z); v[4 * c + 3] = __fadd_rn(v[4 * c + 3], sh.w);
    }
    if (has_res) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 r = *reinterpret_cast<const float4*>(row_ptr + ((c ^ (lane & 7)) << 4));
            v[4 * c + 0] += r.x; v[4 * c + 1] += r.y; v[4 * c + 2] += r.z; v[4 * c + 3] += r.w;
        }
    }
    if (clip) {
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = fminf(fmaxf(lo, v[t]), hi);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4*>(row_ptr + ((c ^ (lane & 7)) << 4)) = make_float4(v[4 * c + 0], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

// The same block for a tile whose whole contraction sits in ONE accumulator group (at most TC_GROUP k blocks): the
// values come straight from tensor memory, 16 columns at a time, and ONE copy of the code serves both blocks of a
// warp (the column offset is a run-time operand of tcgen05.ld, where the register-array form above needs one copy per
// block).  A short contraction is bound by its epilogue, and the unrolled block above - 64 columns pulled into
// registers first, a kilobyte of straight-line code per 8 columns, run once per tile - spent most of its time waiting
// for its own instructions: the same loads and arithmetic cost nothing as a small loop.  Measured variants of this
// block: 16 columns per tcgen05.ld, unrolled twice (this one) 0.291 ms on a 802816 x 256 x 64 layer; the same as a
// rolled loop 0.303; 8 columns unrolled 0.30-0.32, rolled 0.375; 32 columns at once 0.341; the old block 0.373.
// Arithmetic per value as in epi_block.  wprm_s: shared address of the warp's parameters at the block's first column;
// prm_stride: bytes between the bias, scale and shift rows; row_s: shared address of the lane's 128-byte staging row.
__device__ __forceinline__ float4 tc_lds4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void tc_sts4(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void epi_block_direct(uint32_t taddr, uint32_t wprm_s, uint32_t prm_stride, uint32_t row_s, int lane, bool has_res,
                                                 bool clip, float lo, float hi) {
    const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint32_t r[16];
        tmem_ld16(taddr + 16u * (uint32_t)i, r);
        float4 pb[4], ps[4], pt[4], pr[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t a = wprm_s + (uint32_t)((16 * i + 4 * k) * 4);
            pb[k] = tc_lds4(a);
            ps[k] = tc_lds4(a + prm_stride);
            pt[k] = tc_lds4(a + 2u * prm_stride);
            pr[k] = has_res ? tc_lds4(row_s + ((((uint32_t)(4 * i + k)) ^ sw) << 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float v[4] = {__uint_as_float(r[4 * k + 0]) + pb[k].x, __uint_as_float(r[4 * k + 1]) + pb[k].y,
                          __uint_as_float(r[4 * k + 2]) + pb[k].z, __uint_as_float(r[4 * k + 3]) + pb[k].w};
            v[0] = __fadd_rn(__fmul_rn(v[0], ps[k].x), pt[k].x); v[1] = __fadd_rn(__fmul_rn(v[1], ps[k].y), pt[k].y);
            v[2] = __fadd_rn(__fmul_rn(v[2], ps[k].z), pt[k].z); v[3] = __fadd_rn(__fmul_rn(v[3], ps[k].w), pt[k].w);
            if (has_res) { v[0] += pr[k].x; v[1] += pr[k].y; v[2] += pr[k].z; v[3] += pr[k].w; }
            if (clip) {
#pragma unroll
                for (int t = 0; t < 4; ++t) v[t] = fminf(fmaxf(lo, v[t]), hi);
            }
            tc_sts4(row_s + ((((uint32_t)(4 * i + k)) ^ sw) << 4), make_float4(v[0], v[1], v[2], v[3]));
        }
    }
}

// LSTM cell of one lane's 16 units (recurrent_ops.hpp:164-181), for the kernel instance whose epilogue ends a time
// step instead of storing the gate pre-activations.  The weight columns of that product are ordered so that a
// lane's 64 columns are [i | f | c~ | o] of 16 consecutive units: row0 is the lane's staging row of the block with
// i and f, row1 of the block with c~ and o (both hold z = h U + x W + b after epi_block).  Arithmetic per unit as in
// lstm_cellv_kernel (kernels.cu), which finishes the step when the product ran without this epilogue.
__device__ __forceinline__ float tc_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ void lstm_cell_row(const uint8_t* __restrict__ row0, const uint8_t* __restrict__ row1, int lane, long long idx0,
                                              long long out0, const float4 (&c_prev)[4], float* __restrict__ c, float* __restrict__ h,
                                              float* __restrict__ out) {
    const int sw = lane & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 zi = *reinterpret_cast<const float4*>(row0 + ((i ^ sw) << 4));
        const float4 zf = *reinterpret_cast<const float4*>(row0 + (((4 + i) ^ sw) << 4));
        const float4 zc = *reinterpret_cast<const float4*>(row1 + ((i ^ sw) << 4));
        const float4 zo = *reinterpret_cast<const float4*>(row1 + (((4 + i) ^ sw) << 4));
        const float4 cv = c_prev[i];
        float4 cn, hn;
#define FDK_TC_LSTM_UNIT(f)                                                                     \
        cn.f = __fadd_rn(__fmul_rn(tc_sigmoid(zf.f), cv.f), __fmul_rn(tc_sigmoid(zi.f), tanhf(zc.f))); \
        hn.f = __fmul_rn(tc_sigmoid(zo.f), tanhf(cn.f));
        FDK_TC_LSTM_UNIT(x) FDK_TC_LSTM_UNIT(y) FDK_TC_LSTM_UNIT(z) FDK_TC_LSTM_UNIT(w)
#undef FDK_TC_LSTM_UNIT
        *reinterpret_cast<float4*>(c + idx0 + 4 * i) = cn;
        *reinterpret_cast<float4*>(h + idx0 + 4 * i) = hn;
        if (out) *reinterpret_cast<float4*>(out + out0 + 4 * i) = hn;
    }
}

template <int BN, bool CELL>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapWb,
               const __grid_constant__ CUtensorMap mapWs, const __grid_constant__ CUtensorMap mapC,
               const __grid_constant__ CUtensorMap mapR, TcParams prm) {
    using Cfg = TcCfg<BN>;
    const int STAGES = prm.stages;      // W ring / A slots: 2..Cfg::STAGES
    const int A_STAGES = prm.a_stages;  // raw A ring: 2..Cfg::A_STAGES
    // The swizzled tiles need 1024-byte alignment; the kernel has no static shared memory, so the dynamic part
    // starts at the aligned base of the CTA's window (checked below).
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    const uint32_t base = smem_u32(smem_raw);
    // layout: raw A ring | W ring (W_big | W_small per stage) | epilogue staging buffers | epilogue column parameters | barriers
    const uint32_t w_off = (uint32_t)(A_STAGES * Cfg::A_BYTES);
    const uint32_t stg_off = w_off + (uint32_t)(prm.w_stages * Cfg::W_BYTES);
    const uint32_t prm_off = stg_off + (uint32_t)(8 * prm.nbuf * Cfg::STG_BUF_BYTES);
    uint8_t* bar_mem = smem + prm_off + (prm.w_stationary ? 2 : 8) * Cfg::PRM_BLOCK_BYTES;
    const uint32_t bar_base = smem_u32(bar_mem);
    // barrier slots (fixed indices)
    constexpr int SETS = Cfg::SETS;
    static_assert(Cfg::STAGES <= 6 && Cfg::A_STAGES <= 4 && SETS == 2, "barrier layout");
    auto afull_bar = [&](int s) { return bar_base + (uint32_t)s * 8u; };            // TMA landed: raw A tile
    auto afree_bar = [&](int s) { return bar_base + (uint32_t)(4 + s) * 8u; };      // converters have read the raw A tile
    auto wfull_bar = [&](int s) { return bar_base + (uint32_t)(8 + s) * 8u; };      // TMA landed: W_big, W_small
    auto aconv_bar = [&](int s) { return bar_base + (uint32_t)(14 + s) * 8u; };     // A halves of the k block are in TMEM slot s
    auto empty_bar = [&](int s) { return bar_base + (uint32_t)(20 + s) * 8u; };     // MMAs done: W stage s and A slot s free
    auto tfull_bar = [&](int a) { return bar_base + (uint32_t)(26 + a) * 8u; };     // accumulator set holds a finished group
    auto tempty_bar = [&](int a) { return bar_base + (uint32_t)(28 + a) * 8u; };    // accumulator set drained
    auto turn_bar = [&](int i) { return bar_base + (uint32_t)(30 + i) * 8u; };      // issuer i has passed the waits of its group
    auto res_bar = [&](int w, int b) { return bar_base + (uint32_t)(32 + w * 4 + b) * 8u; };  // per epilogue warp and buffer
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 64 * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 64 * 8 + 8);
    static_assert(64 * 8 + 16 <= Cfg::BAR_BYTES, "barrier region too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if ((base & 1023u) != 0) {  // cannot happen (see above); leave before anything is set up
        if (threadIdx.x == 0) atomicCAS(&g_tc_status, 0, 99);
        return;
    }
    if (threadIdx.x == 0) {
        pdl_launch_dependents();   // the next kernel of the stream may set itself up (and fetch weights) while this one runs
        if (blockIdx.x == 0) {
            g_tc_launch[0] = BN; g_tc_launch[1] = prm.N; g_tc_launch[2] = prm.taps * prm.cchunks; g_tc_launch[3] = STAGES;
            g_tc_launch[4] = prm.nbuf; g_tc_launch[5] = (int)prm.M; g_tc_launch[6] = prm.epi.residual != nullptr; g_tc_launch[7] = (int)bar_base;
        }
        for (int s = 0; s < A_STAGES; ++s) {
            mbar_init(afull_bar(s), 1);
            mbar_init(afree_bar(s), 4);
        }
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(wfull_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(aconv_bar(s), 4);
        }
        for (int a = 0; a < SETS; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);
        }
        for (int w = 0; w < 8; ++w)
            for (int b = 0; b < 4; ++b) mbar_init(res_bar(w, b), 1);
        mbar_init(turn_bar(0), 1);
        mbar_init(turn_bar(1), 1);
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

    // tile indices fit 32 bits (checked by the host): 32-bit divisions keep the code small
    const uint32_t m_tiles = (uint32_t)prm.tiles_n * (uint32_t)prm.tiles_h * (uint32_t)prm.tiles_w;
    const int n_tiles = (prm.N + BN - 1) / BN;
    const uint32_t tiles = m_tiles * (uint32_t)n_tiles;
    const uint32_t tiles_wh = (uint32_t)prm.tiles_w * (uint32_t)prm.tiles_h;
    const int k_blocks = prm.taps * prm.cchunks;

    auto a_ptr = [&](int s) { return base + (uint32_t)s * (uint32_t)Cfg::A_BYTES; };
    auto w_ptr = [&](int s) { return base + w_off + (uint32_t)s * (uint32_t)Cfg::W_BYTES; };

    // Single-lane roles keep the whole warp in the loop (all lanes wait, lane 0 issues): a warp whose other lanes
    // sit suspended in a different wait gets its working lane scheduled late.
    // Programmatic dependent launch: everything above, and the weight tiles fetched by warp 3, are independent of the
    // previous kernel of the stream; every other role reads or writes activations and waits for it to finish first.
    if (warp != 3) pdl_wait();
    if (warp < TC_CONV_WARP0) {
      setmaxnreg_dec<TC_REGS_CONTROL>();
      if (warp == 0 || warp == 3) {
        // ---------------- TMA producers: warp 0 the raw A tiles, warp 3 the W tiles ----------------
        // Two rings: a raw A tile is free again as soon as the converters have read it, a W stage (and the
        // A slot in tensor memory of the same index) only when the MMAs of its k block are done.
        const bool a_role = warp == 0;
        const int ring = a_role ? A_STAGES : STAGES;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            if (!a_role && prm.w_stationary && tile != blockIdx.x) break;  // the weights of the first tile serve all
            const uint32_t mt = tile / (uint32_t)n_tiles;
            const int n0 = (int)(tile % (uint32_t)n_tiles) * BN;
            const int tw = (int)(mt % (uint32_t)prm.tiles_w);
            const int th = (int)((mt / (uint32_t)prm.tiles_w) % (uint32_t)prm.tiles_h);
            const int tn = (int)(mt / tiles_wh);
            // first input pixel (before the tap offset) and first image of the tile's pixel box
            const int x0 = (tw << prm.wb_log) * prm.sx - prm.pad_l;
            const int y0 = (th << prm.hb_log) * prm.sy - prm.pad_t;
            int b0 = tn << prm.nb_log;
            int z0 = 0;   // 3-D: input slice under filter tap kz = 0 (the tile lies in ONE output slice: nb_log is 0 then)
            if (prm.Do > 1 || prm.Din > 1) {
                const int sample = tn / prm.Do;
                z0 = (tn - sample * prm.Do) * prm.sz - prm.pad_f;
                b0 = sample * prm.Din;
            }
            int tap = 0, cc = 0, ky = 0, kx = 0, kz = 0;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(a_role ? afree_bar(stage) : empty_bar(stage), phase ^ 1u, abort_flag, 1)) { ok = false; break; }
                if (lane == 0) {
                    if (a_role) {
                        mbar_arrive_expect_tx(afull_bar(stage), (uint32_t)Cfg::A_BYTES);
                        // channels [cc*32, +32) of the input pixels under filter tap (ky, kx); zero outside the image
                        const int z = z0 + kz;
                        const bool slice = z >= 0 && z < prm.Din;
                        tma_load_4d(a_ptr(stage), &mapA, cc * TC_BK, x0 + kx * prm.dx, slice ? y0 + ky * prm.dy : prm.y_none, slice ? b0 + z : 0,
                                    afull_bar(stage));
                    } else {
                        const int wk = tap * prm.Cin + cc * TC_BK;  // the same slice of every filter
                        mbar_arrive_expect_tx(wfull_bar(stage), (uint32_t)Cfg::W_BYTES);
                        tma_load_2d(w_ptr(stage), &mapWb, wk, n0, wfull_bar(stage));
                        tma_load_2d(w_ptr(stage) + Cfg::B_BYTES, &mapWs, wk, n0, wfull_bar(stage));
                    }
                }
                __syncwarp();
                if (++stage == ring) { stage = 0; phase ^= 1u; }
                if (++cc == prm.cchunks) {
                    cc = 0;
                    ++tap;
                    if (++kx == prm.kw) {
                        kx = 0;
                        if (++ky == prm.kh) { ky = 0; ++kz; }
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            // drain: give copies already issued a bounded time to land before the CTA exits
            for (int s = 0; s < ring; ++s) {
                const uint32_t bar = a_role ? afull_bar(s) : wfull_bar(s);
                for (uint32_t it = 0; it < 4096 && !mbar_test(bar, 0) && !mbar_test(bar, 1); ++it) __nanosleep(64);
            }
        }
      } else {
        // ---------------- MMA issuers (warps 1 and 2) ----------------
        // The k blocks of a tile are taken in groups of TC_GROUP; group g (counted over all tiles of the CTA) is
        // issued by issuer g % 2 into accumulator set g % 2, so that one issuer's barrier round trips and commits
        // overlap the other's instruction issue (one thread issues a tcgen05.mma every ~50 cycles at best, and a
        // 128 x 128 x 8 TF32 MMA keeps the tensor pipe busy for only 64).  The issuers take turns at WAITING: an
        // issuer looks at the barriers of group g only after the other one has seen those of group g - 1
        // complete, so nobody ever tests a barrier phase that is two completions ahead (a parity test cannot
        // tell that from "done").
        const int me = warp - 1;
        constexpr uint32_t idesc = make_idesc(TC_BM, BN);
        const uint32_t d_tmem = tmem_base + (uint32_t)(me * BN);
        int stage = 0;
        uint32_t phase = 0, set_phase = 0;
        uint32_t gg = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < k_blocks; kb += TC_GROUP, ++gg) {
                const int nb = k_blocks - kb < TC_GROUP ? k_blocks - kb : TC_GROUP;
                const int s0 = stage;
                const uint32_t p0 = phase;
                const int s1 = s0 + 1 == STAGES ? 0 : s0 + 1;
                const uint32_t p1 = s0 + 1 == STAGES ? (phase ^ 1u) : phase;
                if ((int)(gg & 1) == me) {
                    // group gg - 1 was the other issuer's ((gg - 1) / 2)-th group
                    if (gg > 0 && !mbar_wait(turn_bar(me ^ 1), (uint32_t)(((gg - 1) >> 1) & 1), abort_flag, 9)) { ok = false; break; }
                    const int sl = nb > 1 ? s1 : s0;      // last block of the group (repeats the first if alone)
                    const uint32_t pl = nb > 1 ? p1 : p0;
                    // W stages: the ring position, or (stationary weights) the k block itself, loaded once
                    const int w0 = prm.w_stationary ? kb : s0, w1 = prm.w_stationary ? kb + 1 : s1;
                    const int wl = nb > 1 ? w1 : w0;
                    const uint32_t wp0 = prm.w_stationary ? 0u : p0, wpl = prm.w_stationary ? 0u : pl;
                    // The group's first k block starts as soon as ITS operands are there (and the accumulator set is
                    // free); the second block's barriers are looked at while the first block's MMAs run.  All barriers
                    // of a block are tested together (one round trip); blocking waits only where needed.
                    if (!mbar_test3(tempty_bar(me), set_phase ^ 1u, wfull_bar(w0), wp0, aconv_bar(s0), p0)) {
                        if (!mbar_wait(tempty_bar(me), set_phase ^ 1u, abort_flag, 2)) { ok = false; break; }
                        if (!mbar_wait(wfull_bar(w0), wp0, abort_flag, 7)) { ok = false; break; }
                        if (!mbar_wait(aconv_bar(s0), p0, abort_flag, 3)) { ok = false; break; }
                    }
                    tc_fence_after();
                    // Per block: the eight small-term MMAs, then the four big-term ones, then the commit that hands the
                    // block's A slot and W stage back (half a group earlier than committing at the end of the group: the
                    // slot ring is only two groups deep, and this slack is what the reload-convert loop lives on).
                    const uint64_t d0 = make_smem_desc(w_ptr(w0)), d1 = make_smem_desc(w_ptr(w1));
                    const uint32_t b_hi = (uint32_t)(d0 >> 32);  // the same for every tile: only the address field differs
                    const uint32_t bb0 = (uint32_t)d0, bs0 = bb0 + (uint32_t)(Cfg::B_BYTES >> 4);
                    const uint32_t bb1 = (uint32_t)d1, bs1 = bb1 + (uint32_t)(Cfg::B_BYTES >> 4);
                    const uint32_t ab0 = tmem_base + (uint32_t)(Cfg::A_COL0 + s0 * Cfg::A_SLOT_COLS);
                    const uint32_t ab1 = tmem_base + (uint32_t)(Cfg::A_COL0 + s1 * Cfg::A_SLOT_COLS);
                    if (lane == 0) {
                        umma_cross8(d_tmem, ab0, ab0 + (uint32_t)TC_BK, bb0, bs0, b_hi, idesc, 0u);
                        umma_main4(d_tmem, ab0, bb0, b_hi, idesc);
                        umma_commit(empty_bar(s0));
                    }
                    __syncwarp();
                    if (nb > 1) {
                        if (!mbar_test2(wfull_bar(w1), wpl, aconv_bar(s1), pl)) {
                            if (!mbar_wait(wfull_bar(w1), wpl, abort_flag, 7)) { ok = false; break; }
                            if (!mbar_wait(aconv_bar(s1), pl, abort_flag, 3)) { ok = false; break; }
                        }
                        tc_fence_after();
                    }
                    if (lane == 0) {
                        mbar_arrive(turn_bar(me));  // every barrier of this group has been seen complete
                        if (nb > 1) {
                            umma_cross8(d_tmem, ab1, ab1 + (uint32_t)TC_BK, bb1, bs1, b_hi, idesc, 1u);
                            umma_main4(d_tmem, ab1, bb1, b_hi, idesc);
                            umma_commit(empty_bar(s1));
                        }
                        umma_commit(tfull_bar(me));
                    }
                    __syncwarp();
                    set_phase ^= 1u;
                }
                for (int b = 0; b < nb; ++b)
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
      }
    } else if (warp >= TC_EPI_WARP0) {
        // ---------------- accumulate + epilogue ----------------
        setmaxnreg_inc<TC_REGS_EPILOGUE>();
        constexpr int CPT = Cfg::COLS_PER_THREAD;
        const int q = warp & 3;                           // TMEM lane quadrant this warp may read
        const int half = (warp - TC_EPI_WARP0) >> 2;      // which half of the tile's columns this warp owns
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool has_res = prm.epi.residual != nullptr;
        // final activation of the TMA epilogue: none, ReLU, or ReLU clipped at max_value (threshold 0, slope 0)
        const bool clip = prm.epi.act2.kind != ACT_NONE;
        const float clip_lo = 0.0f;
        const float clip_hi = prm.epi.act2.kind == ACT_RELU_GEN ? prm.epi.act2.p0 : __int_as_float(0x7f800000);
        constexpr int NSUB = CPT / 32;                    // 32-column blocks per lane and tile
        const int ew = warp - TC_EPI_WARP0;
        const int nbuf = prm.nbuf;                        // staging buffers of this warp (power of two)
        // Residual blocks come in by TMA.  With 2 * NSUB buffers the blocks of the warp's NEXT tile are
        // requested while the current tile is finished (the two halves of the ring alternate between
        // tiles); with NSUB buffers they are requested during the tile's own k loop.
        const bool res_ahead = has_res && nbuf >= 2 * NSUB;
        // this warp's staging buffers: 32 rows x 128 bytes each, 1024-byte aligned
        uint8_t* stg_buf = smem + stg_off + (size_t)ew * nbuf * Cfg::STG_BUF_BYTES;
        const uint32_t stg_addr = smem_u32(stg_buf);
        uint32_t res_phase = 0;                           // bit b: parity to wait for on res_bar(ew, b)
        int ring = 0;                                     // next staging buffer (plain ring, or the current half)
        // bias | scale | shift of this warp's CPT columns, refreshed when the tile's column range changes
        float* wprm = reinterpret_cast<float*>(smem + prm_off) + (prm.w_stationary ? half : ew) * 3 * CPT;
        const uint32_t wprm_s = smem_u32(wprm);
        int prm_n0 = -1;
        // The warp's 32 tile rows are a sub-box of the tile's pixel box (all extents are powers of two).
        const int qx_off = (q * 32) & ((1 << prm.wb_log) - 1);
        const int qy_off = ((q * 32) >> prm.wb_log) & ((1 << prm.hb_log) - 1);
        const int qb_off = (q * 32) >> (prm.wb_log + prm.hb_log);
        struct TileGeom { int n0, tw, th, tn, qx, qy, qb, nsub; bool box_in, tma_tile; };
        auto geom_of = [&](uint32_t tile) {
            TileGeom g;
            const uint32_t mt = tile / (uint32_t)n_tiles;
            g.n0 = (int)(tile % (uint32_t)n_tiles) * BN + half * CPT;
            g.tw = (int)(mt % (uint32_t)prm.tiles_w);
            g.th = (int)((mt / (uint32_t)prm.tiles_w) % (uint32_t)prm.tiles_h);
            g.tn = (int)(mt / tiles_wh);
            g.qx = (g.tw << prm.wb_log) + qx_off; g.qy = (g.th << prm.hb_log) + qy_off; g.qb = (g.tn << prm.nb_log) + qb_off;
            g.box_in = g.qx < prm.Wo && g.qy < prm.Ho && g.qb < prm.B;  // else nothing of this warp's rows exists
            // 32-column blocks of this warp that hold columns of the matrix (the last may be partial: the TMA
            // store clips it, the residual load fills it with zeros)
            g.nsub = g.n0 >= prm.N ? 0 : (prm.N - g.n0 + 31) / 32 < NSUB ? (prm.N - g.n0 + 31) / 32 : NSUB;
            g.tma_tile = prm.tma_epi != 0 && g.nsub > 0;                 // warp-uniform
            return g;
        };
        // lane 0: request the residual blocks of a tile into buffers first, first + 1, ... (free by then)
        auto request_residual = [&](const TileGeom& g, int first) {
#pragma unroll
            for (int j = 0; j < NSUB; ++j) {
                if (j >= g.nsub) break;
                const int b = first + j;
                mbar_arrive_expect_tx(res_bar(ew, b), (uint32_t)Cfg::STG_BUF_BYTES);
                tma_load_4d(stg_addr + (uint32_t)(b * Cfg::STG_BUF_BYTES), &mapR, g.n0 + 32 * j, g.qx, g.qy, g.qb, res_bar(ew, b));
            }
        };
        bool res_ready = false;  // res_ahead: the current tile's residual blocks were requested one tile ago
        if (res_ahead && blockIdx.x < tiles) {
            const TileGeom g0 = geom_of(blockIdx.x);
            if (g0.tma_tile && g0.box_in) {
                if (lane == 0) request_residual(g0, 0);
                res_ready = true;
            }
        }
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const TileGeom g = geom_of(tile);
            const int n0 = g.n0;
            if (g.tma_tile && n0 != prm_n0) {
                __syncwarp();
                for (int c = lane; c < CPT; c += 32) {
                    const bool in = n0 + c < prm.N;
                    wprm[c] = (in && prm.epi.bias) ? __ldg(prm.epi.bias + n0 + c) : 0.0f;
                    wprm[CPT + c] = (in && prm.epi.scale) ? __ldg(prm.epi.scale + n0 + c) : 1.0f;
                    wprm[2 * CPT + c] = (in && prm.epi.scale) ? __ldg(prm.epi.shift + n0 + c) : 0.0f;
                }
                __syncwarp();
                prm_n0 = n0;
            }
            const int groups = (k_blocks + TC_GROUP - 1) / TC_GROUP;
            if (!CELL && groups == 1 && prm.tma_epi != 0) {
                // ---- one accumulator group: the blocks read tensor memory themselves (epi_block_direct) ----
                if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * CPT);
                const int acc_now = acc;
                if (++acc == SETS) { acc = 0; acc_phase ^= 1u; }
                if (has_res && !res_ahead && g.tma_tile && g.box_in && lane == 0) {
                    bulk_wait_read<0>();
                    request_residual(g, 0);
                }
                __syncwarp();
                const bool cur_ready_d = res_ready;
                if (res_ahead) {
                    res_ready = false;
                    const uint32_t next = tile + gridDim.x;
                    if (next < tiles) {
                        const TileGeom gn = geom_of(next);
                        if (gn.tma_tile && gn.box_in) {
                            if (lane == 0) {
                                bulk_wait_read<0>();
                                request_residual(gn, ring ^ NSUB);
                            }
                            __syncwarp();
                            res_ready = true;
                        }
                    }
                }
                if (!g.box_in || !g.tma_tile) {   // nothing of this warp's rows or columns exists: hand the set back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(acc_now));
                    if (res_ahead) ring ^= NSUB;
                    continue;
                }
#pragma unroll 1
                for (int j = 0; j < g.nsub; ++j) {
                    const int b = has_res ? (res_ahead ? ring + j : j) : ring;
                    if (has_res) {
                        if (res_ahead && !cur_ready_d && j == 0 && lane == 0) {
                            bulk_wait_read<0>();
                            request_residual(g, ring);
                        }
                        if (!mbar_wait(res_bar(ew, b), (res_phase >> b) & 1u, abort_flag, 6)) { ok = false; break; }
                        res_phase ^= 1u << b;
                    } else {
                        if (lane == 0) {
                            if (nbuf >= 4) bulk_wait_read<3>();
                            else if (nbuf == 2) bulk_wait_read<1>();
                            else bulk_wait_read<0>();
                        }
                        __syncwarp();
                        ring = (ring + 1) & (nbuf - 1);
                    }
                    const uint32_t row_s = stg_addr + (uint32_t)(b * Cfg::STG_BUF_BYTES + lane * 128);
                    epi_block_direct(taddr0 + 32u * (uint32_t)j, wprm_s + (uint32_t)(32 * j * 4), (uint32_t)(CPT * 4), row_s, lane, has_res, clip,
                                     clip_lo, clip_hi);
                    if (j == g.nsub - 1) {   // the last read of the accumulator set is done
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(acc_now));
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_4d(&mapC, stg_addr + (uint32_t)(b * Cfg::STG_BUF_BYTES), n0 + 32 * j, g.qx, g.qy, g.qb);
                        bulk_commit();
                    }
                    __syncwarp();
                }
                if (!ok) {   // a residual wait gave up: the set still has to go back
                    if (lane == 0) mbar_arrive(tempty_bar(acc_now));
                    break;
                }
                if (res_ahead) ring ^= NSUB;
                continue;
            }
            float sum[CPT];
            // LSTM step: the lane's 16 cell states are fetched while the contraction runs
            float4 c_prev[4];
            if constexpr (CELL) {
                const long long srow = (long long)g.qb + lane;
                if (g.box_in && g.tma_tile && srow < prm.B) {
                    const float4* cp = reinterpret_cast<const float4*>(prm.cell_c + srow * prm.cell_U + ((n0 >> 6) << 4));
#pragma unroll
                    for (int i = 0; i < 4; ++i) c_prev[i] = __ldcg(cp + i);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) c_prev[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            for (int kb = 0; kb < groups; ++kb) {
                if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4)) { ok = false; break; }
                tc_fence_after();
                if (TC_REGS_EPILOGUE >= 160) {
                    // enough registers: all of the lane's columns in flight before the single wait
                    uint32_t r[CPT];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * CPT);
                    tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    if (CPT > 32) tmem_ld32(taddr + 32u, *reinterpret_cast<uint32_t(*)[32]>(&r[CPT - 32]));
                    tmem_ld_wait();
                    if (kb == 0) {
#pragma unroll
                        for (int j = 0; j < CPT; ++j) sum[j] = __uint_as_float(r[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < CPT; ++j) sum[j] += __uint_as_float(r[j]);
                    }
                } else {
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
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                if (++acc == SETS) { acc = 0; acc_phase ^= 1u; }
                if (kb == 0 && has_res && !res_ahead && g.tma_tile && g.box_in && lane == 0) {
                    // in-tile request: by now the previous tile's stores have had a k block's time to drain
                    bulk_wait_read<0>();
                    request_residual(g, 0);
                }
                __syncwarp();  // all lanes enter the next wait together
            }
            if (!ok) break;
            const bool cur_ready = res_ready;
            if (res_ahead) {
                // request the next tile's residual blocks into the other half of the ring
                res_ready = false;
                const uint32_t next = tile + gridDim.x;
                if (next < tiles) {
                    const TileGeom gn = geom_of(next);
                    if (gn.tma_tile && gn.box_in) {
                        if (lane == 0) {
                            bulk_wait_read<0>();  // the stores of the tile before this one used that half
                            request_residual(gn, ring ^ NSUB);
                        }
                        __syncwarp();
                        res_ready = true;
                    }
                }
            }
            if (!g.box_in) {
                if (res_ahead) ring ^= NSUB;
                continue;
            }
            if constexpr (CELL) {
                // LSTM step: both blocks of the lane's row become z in their staging buffers (the residual is x W + b
                // of this time step), then the lane finishes its 16 units; nothing of z leaves the SM.  The host
                // side guarantees the TMA epilogue form, N % 64 == 0 and a plain matrix (row = sample).
                if (!g.tma_tile) {   // the columns of this half lie beyond N
                    if (res_ahead) ring ^= NSUB;
                    continue;
                }
                const int b0 = res_ahead ? ring : 0;
#pragma unroll
                for (int j = 0; j < NSUB; ++j) {
                    const int b = b0 + j;
                    if (res_ahead && !cur_ready && j == 0 && lane == 0) request_residual(g, ring);
                    if (!mbar_wait(res_bar(ew, b), (res_phase >> b) & 1u, abort_flag, 6)) { ok = false; break; }
                    res_phase ^= 1u << b;
                    uint8_t* buf = stg_buf + b * Cfg::STG_BUF_BYTES;
                    if (j == 0) epi_block<CPT, 0>(sum, wprm, buf + lane * 128, lane, true, false, 0.f, 0.f);
                    else epi_block<CPT, (NSUB > 1 ? 32 : 0)>(sum, wprm, buf + lane * 128, lane, true, false, 0.f, 0.f);
                }
                if (!ok) break;
                const long long srow = (long long)g.qb + lane;
                if (srow < prm.B) {
                    const int unit0 = (n0 >> 6) << 4;
                    lstm_cell_row(stg_buf + b0 * Cfg::STG_BUF_BYTES + lane * 128, stg_buf + (b0 + NSUB - 1) * Cfg::STG_BUF_BYTES + lane * 128, lane,
                                  srow * prm.cell_U + unit0, srow * prm.cell_out_stride + unit0, c_prev, prm.cell_c, prm.cell_h, prm.cell_out);
                }
                // the next residual copy into these buffers (async proxy) comes after the lanes' own accesses
                fence_proxy_async();
                __syncwarp();
                if (res_ahead) ring ^= NSUB;
                continue;
            }
            if (g.tma_tile) {
                // Epilogue through shared memory and TMA: each lane finishes its row block by block in a
                // staging buffer, one thread stores the 32 x 32 block with a tiled bulk copy (whole 128-byte
                // lines, clipped at the tensor's edges, no L1 traffic), and the warp goes on while it drains.
#pragma unroll
                for (int j = 0; j < NSUB; ++j) {
                    if (j >= g.nsub) break;  // warp-uniform
                    const int b = has_res ? (res_ahead ? ring + j : j) : ring;
                    uint8_t* buf = stg_buf + b * Cfg::STG_BUF_BYTES;
                    if (has_res) {
                        if (res_ahead && !cur_ready && j == 0 && lane == 0) {  // not requested ahead (cannot happen): do it now
                            bulk_wait_read<0>();
                            request_residual(g, ring);
                        }
                        if (!mbar_wait(res_bar(ew, b), (res_phase >> b) & 1u, abort_flag, 6)) { ok = false; break; }
                        res_phase ^= 1u << b;
                    } else {
                        // plain ring: the store that last used this buffer is nbuf stores back
                        if (lane == 0) {
                            if (nbuf >= 4) bulk_wait_read<3>();
                            else if (nbuf == 2) bulk_wait_read<1>();
                            else bulk_wait_read<0>();
                        }
                        __syncwarp();
                        ring = (ring + 1) & (nbuf - 1);
                    }
                    if (j == 0) epi_block<CPT, 0>(sum, wprm, buf + lane * 128, lane, has_res, clip, clip_lo, clip_hi);
                    else epi_block<CPT, (NSUB > 1 ? 32 : 0)>(sum, wprm, buf + lane * 128, lane, has_res, clip, clip_lo, clip_hi);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_4d(&mapC, stg_addr + (uint32_t)(b * Cfg::STG_BUF_BYTES), n0 + 32 * j, g.qx, g.qy, g.qb);
                        bulk_commit();
                    }
                    __syncwarp();
                }
                if (res_ahead) ring ^= NSUB;
                continue;
            }
            // Generic epilogue (rows not 16-byte aligned, or the ragged last column tile).  A lane holds 32
            // consecutive columns of ONE row; each 32 x 32 block goes through the staging buffer (column index
            // XORed with the row: conflict-free both ways) and comes back with one COLUMN per lane, so that each
            // global access of the warp covers 128 contiguous bytes of one output row.
            // this lane's tile row (image, y, x) inside the pixel box, x fastest: float offset of its output pixel
            // (-1: outside); a residual has the same layout as the output, with ldr for ldc when the output is dense
            long long row = -1, res_row = -1;
            {
                const int r = q * 32 + lane;
                const int ox = (g.tw << prm.wb_log) + (r & ((1 << prm.wb_log) - 1));
                const int oy = (g.th << prm.hb_log) + ((r >> prm.wb_log) & ((1 << prm.hb_log) - 1));
                const int bi = (g.tn << prm.nb_log) + (r >> (prm.wb_log + prm.hb_log));
                if (ox < prm.Wo && oy < prm.Ho && bi < prm.B) {
                    row = (long long)bi * prm.out_sb + (long long)oy * prm.out_sy + (long long)ox * prm.out_sx;
                    res_row = prm.spread ? row : (((long long)bi * prm.Ho + oy) * prm.Wo + ox) * prm.epi.ldr;
                }
            }
            // scratch: a buffer that no residual request targets (the current half of the ring)
            float* stg = reinterpret_cast<float*>(stg_buf + (res_ahead ? ring : 0) * Cfg::STG_BUF_BYTES);
            if (res_ahead) ring ^= NSUB;
            if (lane == 0) bulk_wait_read<0>();  // an earlier tile's bulk store may still read the buffer
            __syncwarp();
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += 32) {
                if (n0 + c0 >= prm.N) break;  // warp-uniform
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 32 + (j ^ lane)] = sum[c0 + j];
                __syncwarp();
                const int col = n0 + c0 + lane;
                // four rows at a time: all residual loads of a group are issued before anything is stored
                // (the residual never aliases the output: it is a different live tensor of the plan).  Kept as a
                // rolled loop: this path is rare and must not crowd the instruction cache.
#pragma unroll 1
                for (int r0 = 0; r0 < 32; r0 += 4) {
                    float res[4];
                    long long orow[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        orow[i] = __shfl_sync(0xffffffffu, row, r0 + i);  // output offset of tile row r0 + i (-1: outside)
                        const long long rrow = __shfl_sync(0xffffffffu, res_row, r0 + i);
                        res[i] = (prm.epi.residual && orow[i] >= 0 && col < prm.N) ? __ldg(prm.epi.residual + rrow + col) : 0.f;
                    }
                    if (col < prm.N) {
                        const float b = prm.epi.bias ? __ldg(prm.epi.bias + col) : 0.f;
                        const float sc = prm.epi.scale ? __ldg(prm.epi.scale + col) : 1.f;
                        const float sh = prm.epi.scale ? __ldg(prm.epi.shift + col) : 0.f;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (orow[i] >= 0) {
                                float v = stg[(r0 + i) * 32 + (lane ^ (r0 + i))];
                                if (prm.epi.bias) v += b;
                                v = act_apply(prm.epi.act1, v);
                                if (prm.epi.scale) v = __fadd_rn(__fmul_rn(v, sc), sh);
                                if (prm.epi.residual) v += res[i];
                                prm.C[orow[i] + col] = act_apply(prm.epi.act2, v);
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (!ok) {
            // gave up: leave residual copies that may still be in flight a bounded time to land
            for (int it = 0; it < 4096; ++it) __nanosleep(256);
        }
        if (lane == 0) bulk_wait_all();  // the staging buffers must outlive the stores that read them
    } else {
        // ---------------- converters: raw A tile -> TF32 halves in tensor memory ----------------
        // Two teams of four warps take alternate k blocks (counted over all tiles of the CTA; both rings have an
        // even number of stages, so a stage always belongs to the same team).  Lane l of a warp owns tile row
        // r = 32 * (warp % 4) + l (the TMEM lanes this warp may write): it reads the row's 128 bytes from the
        // swizzled tile and writes big | small into the 64 columns of the k block's A slot, 16 columns at a time.
        // big = x with the 13 low mantissa bits cleared (one AND), small = x - big (exact; the tensor core reads
        // its 10 leading mantissa bits, so the split keeps 21 bits of x): two instructions per element where the
        // rounding split took five, which matters because this stage shares the SM's issue slots and shared-memory
        // bandwidth with everything else.  Half rows holding Inf or NaN take the conversion instruction so that
        // those values keep their meaning (Inf - Inf would turn an Inf into NaN).
        if (TC_REGS_CONVERT > TC_REGS_LAUNCH) setmaxnreg_inc<TC_REGS_CONVERT>();
        else setmaxnreg_dec<TC_REGS_CONVERT>();
        const int team = (warp - TC_CONV_WARP0) >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)Cfg::A_COL0;
        int stage = 0, astage = 0;
        uint32_t phase = 0, aphase = 0, kg = 0;
        bool ok = true;
        // The stores of a k block are confirmed (wait, fence, arrive on the block's "converted" barrier) only after
        // the NEXT block's row has been loaded and split, so that their latency is covered by that work.  A warp
        // never blocks with a confirmation pending: the MMAs that free the slot it waits for may need it.
        int pending = -1;  // A slot whose stores are issued but not confirmed
        auto confirm = [&]() {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(aconv_bar(pending));
            __syncwarp();
            pending = -1;
        };
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < k_blocks; ++kb, ++kg) {
                if ((int)(kg & (uint32_t)(TC_TEAMS - 1)) == team) {
                    // the raw tile has landed
                    if (!mbar_try(afull_bar(astage), aphase)) {
                        if (pending >= 0) confirm();
                        if (!mbar_wait(afull_bar(astage), aphase, abort_flag, 5)) { ok = false; break; }
                    }
                    const uint8_t* row = smem + (size_t)astage * Cfg::A_BYTES + r * 128;
                    uint32_t hi[32], lo[32];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float finite = 0.0f;  // becomes NaN if the half row holds an Inf or a NaN
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float4 v = *reinterpret_cast<const float4*>(row + (((4 * h + c) ^ (r & 7)) << 4));
                            const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                finite = fmaf(x[t], 0.0f, finite);
                                const uint32_t b = __float_as_uint(x[t]) & 0xFFFFE000u;
                                hi[16 * h + 4 * c + t] = b;
                                lo[16 * h + 4 * c + t] = __float_as_uint(x[t] - __uint_as_float(b));
                            }
                        }
                        if (finite != finite) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const float4 v = *reinterpret_cast<const float4*>(row + (((4 * h + c) ^ (r & 7)) << 4));
                                const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                for (int t = 0; t < 4; ++t) {
                                    hi[16 * h + 4 * c + t] = rna_tf32(x[t]);
                                    lo[16 * h + 4 * c + t] = rna_tf32(x[t] - __uint_as_float(hi[16 * h + 4 * c + t]));
                                }
                            }
                        }
                    }
                    // the whole row has been read: hand the raw stage back to the producer
                    __syncwarp();
                    if (lane == 0) mbar_arrive(afree_bar(astage));
                    if (pending >= 0) confirm();
                    // the MMAs that read this A slot last time are done
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 8)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t dst = lane_addr + (uint32_t)(stage * Cfg::A_SLOT_COLS);
                    tmem_st16(dst, *reinterpret_cast<const uint32_t(*)[16]>(&hi[0]));
                    tmem_st16(dst + 16u, *reinterpret_cast<const uint32_t(*)[16]>(&hi[16]));
                    tmem_st16(dst + (uint32_t)TC_BK, *reinterpret_cast<const uint32_t(*)[16]>(&lo[0]));
                    tmem_st16(dst + (uint32_t)TC_BK + 16u, *reinterpret_cast<const uint32_t(*)[16]>(&lo[16]));
                    pending = stage;
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                if (++astage == A_STAGES) { astage = 0; aphase ^= 1u; }
            }
        }
        if (ok && pending >= 0) confirm();
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

// 4-D map over a channels-last input [B][H][W][pix] (pix = floats per pixel, >= C): box = 32 channels x a
// (Wb, Hb, Nb) pixel box; with strides sx / sy only every sx-th / sy-th pixel is fetched.
CUtensorMap make_map_4d(const float* base, const ConvTcGeom& g, int wb, int hb, int nb) {
    EncodeFn enc = tc_get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap m;
    cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)(g.B * g.D)};  // images: samples x input slices
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

// 4-D map over a channels-last output or residual tensor of B x Ho x Wo pixels, sx / sy / sb floats apart in x, in y
// and between samples (dense: ld, Wo * ld, Ho * Wo * ld): box = 32 channels x the pixels of one epilogue warp (32 of
// the tile's 128 rows, x fastest).
CUtensorMap make_map_out(const float* base, int64_t B, int Ho, int Wo, int N, int64_t sx, int64_t sy, int64_t sb, int wb, int hb) {
    EncodeFn enc = tc_get_encode();
    ensure(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    const int qw = std::min(wb, 32), qh = std::min(hb, 32 / qw), qn = 32 / (qw * qh);
    CUtensorMap m;
    const cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)Wo, (cuuint64_t)Ho, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)sx * sizeof(float), (cuuint64_t)sy * sizeof(float), (cuuint64_t)sb * sizeof(float)};
    const cuuint32_t box[4] = {(cuuint32_t)TC_BK, (cuuint32_t)qw, (cuuint32_t)qh, (cuuint32_t)qn};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ensure(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (output) failed with code " + std::to_string((int)r));
    return m;
}

// Pixel box of an output tile: powers of two (Wb, Hb, Nb) with product 128 that need the fewest tiles.
void choose_box(const ConvTcGeom& g, int& wb_log, int& hb_log, int& nb_log, int max_nb_log = 7) {
    int64_t best = -1;
    const int64_t images = g.B * g.Do;
    for (int w = 0; w <= 7; ++w) {
        if ((1 << w) * g.sx > 256) break;
        for (int h = 0; w + h <= 7; ++h) {
            if ((1 << h) * g.sy > 256) break;
            const int n = 7 - w - h;
            if (n > max_nb_log) continue;
            const int64_t t = ((g.Wo + (1 << w) - 1) >> w) * (int64_t)((g.Ho + (1 << h) - 1) >> h) * ((images + (1 << n) - 1) >> n);
            if (best < 0 || t < best || (t == best && w > wb_log)) { best = t; wb_log = w; hb_log = h; nb_log = n; }
        }
    }
}

struct CellState {
    float* c = nullptr;
    float* h = nullptr;
    float* out = nullptr;
    int64_t out_stride = 0;
    int U = 0;
};

template <int BN, bool CELL = false>
void launch_tc(const float* in, const ConvTcGeom& g, const float* Wb, const float* Ws, int64_t ldw, float* C, int64_t ldc, int N,
               const Epilogue& e, cudaStream_t s, const CellState* cell = nullptr) {
    using Cfg = TcCfg<BN>;
    {
        // the attribute belongs to the function on one device: set it once per device
        static std::mutex mu;
        static bool attr_set[64] = {};
        int dev = 0;
        FDK_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            FDK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, CELL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::MAX_SMEM));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    TcParams prm;
    int wb = 0, hb = 0, nb = 7;
    const bool volume = g.D > 1 || g.Do > 1 || g.kd > 1;
    if (!CELL) choose_box(g, wb, hb, nb, volume ? 0 : 7);  // the LSTM step wants tile row = sample
    const int64_t out_slices = g.B * g.Do;  // output "images": samples x output slices
    prm.wb_log = wb; prm.hb_log = hb; prm.nb_log = nb;
    prm.tiles_w = (g.Wo + (1 << wb) - 1) >> wb;
    prm.tiles_h = (g.Ho + (1 << hb) - 1) >> hb;
    prm.tiles_n = (int)((out_slices + (1 << nb) - 1) >> nb);
    const bool rowwin = g.win_stride > 0;
    const int64_t K = rowwin ? (int64_t)g.kh * TC_BK : (int64_t)g.kd * g.kh * g.kw * g.C;
    const CUtensorMap mA = make_map_4d(in, g, 1 << wb, 1 << hb, 1 << nb);
    const CUtensorMap mWb = tc_make_map_2d(Wb, N, K, ldw, BN);
    const CUtensorMap mWs = tc_make_map_2d(Ws, N, K, ldw, BN);
    prm.C = C; prm.ldc = ldc; prm.M = out_slices * g.Ho * g.Wo; prm.N = N; prm.epi = to_dev(e);
    prm.cell_c = cell ? cell->c : nullptr; prm.cell_h = cell ? cell->h : nullptr; prm.cell_out = cell ? cell->out : nullptr;
    prm.cell_out_stride = cell ? (long long)cell->out_stride : 0; prm.cell_U = cell ? cell->U : 0;
    prm.B = (int)out_slices; prm.Ho = g.Ho; prm.Wo = g.Wo; prm.Cin = g.C;
    prm.kw = g.kw; prm.kh = g.kh; prm.taps = g.kd * g.kh * g.kw; prm.cchunks = (g.C + TC_BK - 1) / TC_BK;
    prm.Din = g.D; prm.Do = g.Do; prm.sz = g.sz; prm.pad_f = g.pad_f;
    prm.y_none = g.H + 1024;
    prm.sy = g.sy; prm.sx = g.sx; prm.dy = g.dy; prm.dx = g.dx; prm.pad_t = g.pad_t; prm.pad_l = g.pad_l;
    if (rowwin) {  // one k block per filter row; x coordinates count output columns
        prm.Cin = TC_BK; prm.kw = 1; prm.kh = g.kh; prm.taps = g.kh; prm.cchunks = 1;
        prm.sx = 1; prm.dx = 1; prm.dy = 1; prm.pad_t = 0; prm.pad_l = 0;
    }
    // Epilogue through TMA when the rows of the output (and of the residual) start on 16-byte boundaries.
    const bool plain_act = e.act1.kind == ACT_NONE &&
                           (e.act2.kind == ACT_NONE || e.act2.kind == ACT_RELU ||
                            (e.act2.kind == ACT_RELU_GEN && e.act2.p1 == 0.0f && e.act2.p2 == 0.0f));  // clipped ReLU: slope 0, threshold 0
    const bool spread = g.out_sx > 0;  // output pixels are not dense
    prm.out_sx = spread ? g.out_sx : ldc;
    prm.out_sy = spread ? g.out_sy : (long long)g.Wo * ldc;
    prm.out_sb = spread ? g.out_sb : (long long)g.Ho * g.Wo * ldc;
    prm.spread = spread ? 1 : 0;
    ensure(!spread || e.residual == nullptr || e.ldr == ldc, "internal: spread output pixels need a residual of the same layout");
    prm.tma_epi = (plain_act && (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
                   ((prm.out_sx | prm.out_sy | prm.out_sb) & 3) == 0 &&
                   (e.residual == nullptr || ((e.ldr & 3) == 0 && (reinterpret_cast<uintptr_t>(e.residual) & 15) == 0))) ? 1 : 0;
    CUtensorMap mC = mA, mR = mA;  // placeholders when the TMA epilogue is off (never dereferenced then)
    if (prm.tma_epi) {
        mC = make_map_out(C, out_slices, g.Ho, g.Wo, N, prm.out_sx, prm.out_sy, prm.out_sb, 1 << wb, 1 << hb);
        if (e.residual) {
            if (spread) mR = make_map_out(e.residual, out_slices, g.Ho, g.Wo, N, prm.out_sx, prm.out_sy, prm.out_sb, 1 << wb, 1 << hb);
            else mR = make_map_out(e.residual, out_slices, g.Ho, g.Wo, N, e.ldr, (int64_t)g.Wo * e.ldr, (int64_t)g.Ho * g.Wo * e.ldr, 1 << wb, 1 << hb);
        }
    }
    const int64_t tiles = (int64_t)prm.tiles_w * prm.tiles_h * prm.tiles_n * ((N + BN - 1) / BN);
    ensure(tiles < (int64_t)1 << 31, "tensor-core kernel: too many tiles");
    const int grid = (int)std::min<int64_t>(tiles, tc_sm_count());
    // Shared memory plan (227 KB): staging buffers per epilogue warp (ring of 4 KB blocks), W stages and the raw A
    // ring.  Short contractions are bound by the output stream: deep staging (with a residual, the blocks of the
    // warp's next tile are prefetched: 2 * NSUB buffers); if all tiles of a CTA use the same weight tiles (its
    // tile indices share the column tile), the weights are loaded once and stay.  Long contractions: as many W
    // stages as fit (they cover the latency of reloading a stage after its MMAs).
    const int k_blocks = prm.taps * prm.cchunks;
    const int n_tiles = (N + BN - 1) / BN;
    constexpr int NSUB = BN / 64;
    const bool thin = k_blocks <= 4;
    if (!prm.tma_epi) prm.nbuf = 1;
    else if (e.residual) prm.nbuf = (thin || NSUB == 1) ? 2 * NSUB : NSUB;
    else prm.nbuf = thin ? (BN == 64 ? 4 : 2) : (BN == 64 ? 2 : 1);
    prm.stages = Cfg::STAGES;
    prm.a_stages = Cfg::A_STAGES;
    const int k_even = (k_blocks + 1) & ~1;
    prm.w_stationary = (k_even <= Cfg::STAGES && (tiles <= grid || grid % n_tiles == 0)) ? 1 : 0;
    prm.w_stages = prm.w_stationary ? k_even : prm.stages;
    // Shrink until it fits, keeping both rings at three stages or more as long as possible (a ring of two leaves
    // the ~1 us of a TMA load exposed at every other k block): A to 3, W to 3, then A to 2, W to 2, then the staging.
    // With one converter team any ring size works (every role walks the k blocks in order and tracks the phase of
    // each stage itself); two teams need even rings.
    auto need = [&] { return Cfg::smem_bytes(prm.a_stages, prm.w_stages, prm.nbuf, prm.w_stationary != 0); };
    constexpr int step = TC_TEAMS == 1 ? 1 : 2;
    while (need() > Cfg::MAX_SMEM) {
        if (prm.a_stages > 3) prm.a_stages -= step;
        else if (!prm.w_stationary && prm.stages > 3) { prm.stages -= step; prm.w_stages = prm.stages; }
        else if (prm.a_stages > 2) prm.a_stages -= step;
        else if (!prm.w_stationary && prm.stages > 2) { prm.stages -= step; prm.w_stages = prm.stages; }
        else if (prm.nbuf > 1) prm.nbuf /= 2;
        else break;
    }
    prm.a_stages = std::max(prm.a_stages, 2);
    prm.stages = std::max(prm.stages, 2);
    if (!prm.w_stationary) prm.w_stages = prm.stages;
    const int smem_bytes = need();
    ensure(smem_bytes <= Cfg::MAX_SMEM, "tensor-core kernel: shared memory budget exceeded");
    if (CELL) ensure(cell != nullptr && prm.tma_epi != 0 && e.residual != nullptr && N % 64 == 0 && g.Ho == 1 && g.Wo == 1 && nb == 7,
                     "internal: the LSTM step kernel needs the TMA epilogue form");
    launch_pdl(gemm_tc_kernel<BN, CELL>, dim3((unsigned)grid), dim3(TC_THREADS), (size_t)smem_bytes, s, mA, mWb, mWs, mC, mR, prm);
}

}  // namespace

bool conv_tc_supported(const ConvTcGeom& g, int N, int64_t ldw, const void* in, const void* W) {
    if (g.B <= 0 || N <= 0 || g.C <= 0 || g.Ho <= 0 || g.Wo <= 0) return false;
    if ((g.C & 3) || (g.pix & 3) || (ldw & 3)) return false;
    if (g.win_stride > 0 && ((g.win_stride & 3) || g.kw * g.C > TC_BK)) return false;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return false;
    if (g.sx < 1 || g.sx > 8 || g.sy < 1 || g.sy > 8) return false;
    if (g.D < 1 || g.Do < 1 || g.kd < 1 || g.sz < 1) return false;
    if (g.B * g.D > 0x7fffffffLL || g.B * g.Do * g.Ho * g.Wo > 0x7fffffffLL) return false;
    return tc_get_encode() != nullptr;
}

void launch_conv_tc(const float* in, const ConvTcGeom& g, const float* Wbig, const float* Wsmall, int64_t ldw, float* C, int64_t ldc,
                    int N, const Epilogue& e, cudaStream_t s) {
    // 64 columns per tile also when 128-column tiles would leave more than half of the SMs without one (few rows: a
    // small batch in the late layers).  The tile width does not touch a result: every output value is the same chain
    // of k blocks whatever tile it sits in, so this choice may depend on the batch.
    bool narrow = N <= 64;
    if (!narrow) {
        int wb, hb, nb;
        choose_box(g, wb, hb, nb, (g.D > 1 || g.Do > 1 || g.kd > 1) ? 0 : 7);
        const int64_t row_tiles = (int64_t)((g.Wo + (1 << wb) - 1) >> wb) * ((g.Ho + (1 << hb) - 1) >> hb) * ((g.B * g.Do + (1 << nb) - 1) >> nb);
        narrow = row_tiles * ((N + 127) / 128) * 2 <= tc_sm_count();
    }
    if (narrow) launch_tc<64>(in, g, Wbig, Wsmall, ldw, C, ldc, N, e, s);
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

bool lstm_step_tc_supported(int64_t B, int U, const void* h, const void* W, int64_t ldw, const void* x, int64_t ldx, const void* c,
                            const void* h_next, const void* out, int64_t out_stride) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (U <= 0 || U % 16 != 0 || B <= 0 || (ldx & 3) || !al16(x) || !al16(c) || !al16(h_next)) return false;
    if (out != nullptr && (!al16(out) || (out_stride & 3))) return false;
    return gemm_tc_supported(B, 4 * U, U, U, ldw, h, W);
}

void launch_lstm_step_tc(const float* h, const float* Wbig, const float* Wsmall, int64_t ldw, const float* x, int64_t ldx, float* c,
                         float* h_next, float* out, int64_t out_stride, float* z_unused, int64_t B, int U, cudaStream_t s) {
    Epilogue e;
    e.residual = x;
    e.ldr = ldx;
    CellState cell;
    cell.c = c; cell.h = h_next; cell.out = out; cell.out_stride = out_stride; cell.U = U;
    launch_tc<128, true>(h, gemm_geom(B, U, U), Wbig, Wsmall, ldw, z_unused, (int64_t)4 * U, 4 * U, e, s, &cell);
}

const int* gemm_tc_status_address() {
    int* p = nullptr;
    FDK_CUDA(cudaGetSymbolAddress((void**)&p, g_tc_status));
    return p;
}

int gemm_tc_take_status(cudaStream_t s) {
    const int rows = gemm_rows_take_status(s);   // the row-product kernel keeps its own status word
    const int dw = dwconv_tiles_take_status(s);  // so does the tiled depthwise kernel
    int v = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (v != 0) {
        int d[16] = {};
        if (cudaMemcpyFromSymbol(d, g_tc_diag, sizeof(d)) == cudaSuccess)
            fprintf(stderr, "gemm_tc: wait gave up: code %d block %d/%d thread %d barrier offset %d parity %d | BN %d N %d k_blocks %d stages %d nbuf %d M %d residual %d\n",
                    d[8], d[9], d[13], d[10], d[11] - d[7], d[12], d[0], d[1], d[2], d[3], d[4], d[5], d[6]);
        else cudaGetLastError();
        const int zero = 0;
        cudaMemcpyToSymbolAsync(g_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return v != 0 ? v : (rows != 0 ? 100 + rows : (dw != 0 ? 200 + dw : 0));
}

void launch_split_tf32(const float* w, float* big, float* small, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    int64_t g = (n + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    split_tf32_kernel<<<(unsigned)g, 256, 0, s>>>(w, big, small, (long long)n);
    FDK_CUDA(cudaGetLastError());
}

}  // namespace fdk
