// Micro-benchmark: how fast one thread per SM can pull the contraction kernel's operand tiles into shared memory on
// sm_100a, from an L2-resident matrix:
//   * tiled TMA loads of a box of 32 floats x ROWS rows (128-byte rows, 128-byte swizzle) out of a row-major matrix
//     whose rows are K floats apart: what the kernel issues for W (two boxes of BN rows) and, in 4-D form, for A;
//   * plain bulk copies (cp.async.bulk) of the same number of bytes from a contiguous block: what a W tile costs when
//     the weights are stored tile by tile.
// All 148 CTAs run the same loop: 1, 2 or 4 issuing warps per CTA, each with DEPTH copies in flight (its own ring of
// buffers, one mbarrier each); prints cycles per copy as seen by CTA 0's first warp and the aggregate rate.  Every
// wait is bounded.
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o tma_load_rate tma_load_rate.cu
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// poll != 0: test_wait in a loop (never suspends) instead of the suspending try_wait
__device__ int g_poll = 0;
__device__ int g_lanes = 1;   // issuing lanes per warp (each with its own ring): are copies of one WARP serialised, or of one thread?
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    if (g_poll) {
        for (long long spin = 0; spin < 400000000ll && !ok; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        return ok != 0;
    }
    for (int spin = 0; spin < 20000 && !ok; ++spin)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(100000u) : "memory");
    return ok != 0;
}
// mode 0: tiled 2-D box loads, mode 1: bulk copies of contiguous blocks.  bytes = size of one copy.
// Every warp of the CTA is an independent issuer (lane 0) with its own ring of buffers and barriers.
__global__ void __launch_bounds__(128, 1) load_kernel(const __grid_constant__ CUtensorMap map, const float* flat, int mode, int rows, int K, int n_row_tiles,
                                                      int iters, int depth, long long* cycles, int* status) {
    extern __shared__ uint8_t raw[];
    const uint32_t bytes = (uint32_t)rows * 128u;
    const int lanes = g_lanes;
    const int warp = (threadIdx.x >> 5) * lanes + (int)(threadIdx.x & 31);   // issuer index
    const uint32_t base = ((smem_u32(raw) + 1023u) & ~1023u) + (uint32_t)warp * (uint32_t)depth * bytes;
    __shared__ uint64_t all_bars[64];
    uint64_t* bars = all_bars + warp * 8;
    if ((int)(threadIdx.x & 31) < lanes) {
        for (int i = 0; i < depth; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if ((int)(threadIdx.x & 31) >= lanes) return;
    const int k_tiles = K / 32;
    auto issue = [&](int it) {
        const int slot = it % depth;
        const uint32_t bar = smem_u32(&bars[slot]), dst = base + (uint32_t)slot * bytes;
        // walk the matrix like the kernel does: k blocks of one row tile, then the next row tile (offset per CTA)
        const int kt = it % k_tiles, rt = (it / k_tiles + (int)blockIdx.x + warp * 3) % n_row_tiles;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        if (mode == 0)
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst), "l"(reinterpret_cast<uint64_t>(&map)), "r"(kt * 32), "r"(rt * rows), "r"(bar) : "memory");
        else
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst), "l"(flat + ((size_t)rt * k_tiles + kt) * (bytes / 4)), "r"(bytes), "r"(bar) : "memory");
    };
    bool ok = true;
    const long long t0 = clock64();
    for (int it = 0; it < depth && it < iters; ++it) issue(it);
    for (int it = 0; it < iters && ok; ++it) {
        ok = wait_bar(smem_u32(&bars[it % depth]), (uint32_t)((it / depth) & 1));
        if (it + depth < iters) issue(it + depth);
    }
    if (warp == 0) cycles[blockIdx.x] = clock64() - t0;
    if (!ok) atomicExch(status, 1);
}
int main() {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    EncodeFn enc = (EncodeFn)p;
    const int K = 2304, N = 1024;  // a 9.4 MB matrix: stays in L2
    float* w; CK(cudaMalloc(&w, (size_t)N * K * sizeof(float))); CK(cudaMemset(w, 0, (size_t)N * K * sizeof(float)));
    long long* d_cycles; int* d_status;
    CK(cudaMalloc(&d_cycles, 148 * sizeof(long long))); CK(cudaMalloc(&d_status, sizeof(int))); CK(cudaMemset(d_status, 0, sizeof(int)));
    const int iters = 20000;
    for (int poll = 0; poll < 3; ++poll)
    for (int rows : {64, 128, 256}) {
        const int lanes = poll == 2 ? 2 : 1, pl = poll == 1 ? 1 : 0;
        CK(cudaMemcpyToSymbol(g_poll, &pl, sizeof(int)));
        CK(cudaMemcpyToSymbol(g_lanes, &lanes, sizeof(int)));
        if (poll && rows != 128) continue;
        CUtensorMap m;
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 4};
        const cuuint32_t box[2] = {32, (cuuint32_t)rows};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
        for (int mode = 0; mode < 2; ++mode)
            for (int depth : {1, 2, 4}) for (int warps : {1, 2, 4}) {
                if (depth == 1 && warps > 1) continue;
                if (lanes * warps > 4) continue;
                const int smem = lanes * warps * depth * rows * 128 + 1024;
                if (smem > 227 * 1024) continue;
                CK(cudaFuncSetAttribute(load_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
                float ms = 0.f; long long h[148];
                for (int rep = 0; rep < 2; ++rep) {
                    CK(cudaEventRecord(e0));
                    load_kernel<<<148, 32 * warps, smem>>>(m, w, mode, rows, K, N / rows, iters, depth, d_cycles, d_status);
                    CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1)); CK(cudaGetLastError());
                    CK(cudaEventElapsedTime(&ms, e0, e1));
                    CK(cudaMemcpy(h, d_cycles, sizeof(h), cudaMemcpyDeviceToHost));
                }
                int st; CK(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
                const double bytes = (double)rows * 128;
                printf("%s%-22s %3d rows (%5.0f KB) depth %d, %d issuing warps: %7.1f clk per copy and warp, %6.1f clk per 16 KB of the SM, %6.2f TB/s all SMs  status %d\n",
                       poll == 1 ? "[polling wait] " : poll == 2 ? "[2 issuing lanes per warp] " : "", mode == 0 ? "tiled box 32 x rows" : "bulk copy, contiguous", rows, bytes / 1024, depth, warps, (double)h[0] / iters,
                       (double)h[0] / iters / (warps * lanes) * 16384.0 / bytes, bytes * iters * warps * lanes * 148 / (ms * 1e-3) / 1e12, st);
            }
    }
    return 0;
}
