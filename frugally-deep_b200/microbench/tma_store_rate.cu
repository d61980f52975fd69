// Micro-benchmark: the output-stream rate of an epilogue on sm_100a, for a [802816 x N] fp32 matrix (N = 256, 64):
//   * one output row per lane written as float4 (how a register-resident accumulator tile is laid out),
//   * rows written by whole warps (coalesced),
//   * 32-column boxes staged in shared memory and stored with cp.async.bulk.tensor (what gemm_tc.cu does).
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o tma_store_rate tma_store_rate.cu
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// each warp w of the CTA stores boxes [cols 32][rows R] ; tile = 128 rows x N cols ; tiles strided over CTAs
template <int ROWS>
__global__ void __launch_bounds__(256, 1) store_kernel(const __grid_constant__ CUtensorMap map, int N, long long m_tiles, int nbuf) {
    extern __shared__ uint8_t raw[];
    const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int boxes_per_tile = (128 / ROWS) * (N / 32);   // per 128-row tile
    int ring = 0;
    for (long long t = blockIdx.x; t < m_tiles; t += gridDim.x) {
        for (int b = warp; b < boxes_per_tile; b += 8) {
            const int rb = b % (128 / ROWS), cb = b / (128 / ROWS);
            const uint32_t buf = base + (uint32_t)((warp * nbuf + ring) * ROWS * 128);
            if (lane == 0) {
                if (nbuf == 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                else if (nbuf == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                else asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
            }
            __syncwarp();
            // touch the buffer like an epilogue would (one row per lane, ROWS/32 passes)
            for (int r = lane; r < ROWS; r += 32)
                for (int c = 0; c < 8; ++c) asm volatile("st.shared.v4.f32 [%0], {%1, %1, %1, %1};" ::"r"(buf + r * 128 + ((c ^ (r & 7)) << 4)), "f"((float)t));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"(reinterpret_cast<uint64_t>(&map)), "r"(buf), "r"(cb * 32), "r"((int)(t * 128 + rb * ROWS)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            ring = (ring + 1) % nbuf;
        }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// reference: each lane stores its row as float4s (row-per-lane, like a register epilogue)
__global__ void __launch_bounds__(256, 1) direct_kernel(float* out, int N, long long m_tiles) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (long long t = blockIdx.x; t < m_tiles; t += gridDim.x) {
        const int q = warp & 3, half = warp >> 2;
        float* row = out + (t * 128 + q * 32 + lane) * (long long)N + half * (N / 2);
        for (int c = 0; c < N / 2; c += 4) *reinterpret_cast<float4*>(row + c) = make_float4((float)t, 1.f, 2.f, 3.f);
    }
}
// coalesced: each warp writes whole rows (lanes across columns)
__global__ void __launch_bounds__(256, 1) coalesced_kernel(float* out, int N, long long m_tiles) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (long long t = blockIdx.x; t < m_tiles; t += gridDim.x)
        for (int r = warp; r < 128; r += 8) {
            float* row = out + (t * 128 + r) * (long long)N;
            for (int c = lane * 4; c < N; c += 128) *reinterpret_cast<float4*>(row + c) = make_float4((float)t, 1.f, 2.f, 3.f);
        }
}
int main() {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    EncodeFn enc = (EncodeFn)p;
    const long long M = 802816;
    for (int N : {256, 64}) {
        float* out; CK(cudaMalloc(&out, M * N * sizeof(float)));
        const long long m_tiles = M / 128;
        const double gb = (double)M * N * 4 / 1e9;
        cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
        auto timeit = [&](auto launch, const char* name) {
            float best = 1e30f;
            for (int rep = 0; rep < 4; ++rep) {
                cudaEventRecord(e0); launch(); cudaEventRecord(e1); cudaEventSynchronize(e1);
                float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
            }
            cudaError_t e = cudaGetLastError();
            printf("N=%3d %-34s %7.3f ms %7.0f GB/s %s\n", N, name, best, gb / best * 1e3, e == cudaSuccess ? "" : cudaGetErrorString(e));
        };
        timeit([&] { direct_kernel<<<148, 256>>>(out, N, m_tiles); }, "direct row-per-lane float4");
        timeit([&] { coalesced_kernel<<<148, 256>>>(out, N, m_tiles); }, "coalesced float4");
        for (int rows : {32, 128}) for (int nbuf : {1, 2, 4}) {
            CUtensorMap m;
            const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
            const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
            const cuuint32_t box[2] = {32, (cuuint32_t)rows};
            const cuuint32_t estr[2] = {1, 1};
            CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
            const int smem = 8 * nbuf * rows * 128 + 1024;
            if (smem > 227 * 1024) continue;
            char name[64]; snprintf(name, sizeof(name), "TMA box 32x%d nbuf %d", rows, nbuf);
            if (rows == 32) { CK(cudaFuncSetAttribute(store_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); timeit([&] { store_kernel<32><<<148, 256, smem>>>(m, N, m_tiles, nbuf); }, name); }
            else { CK(cudaFuncSetAttribute(store_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); timeit([&] { store_kernel<128><<<148, 256, smem>>>(m, N, m_tiles, nbuf); }, name); }
        }
        cudaFree(out);
    }
    return 0;
}
