// Micro-benchmark: how fast four warps can turn a 128 x 32 fp32 tile in shared memory into its two TF32 halves in
// tensor memory (the contraction kernel's converter stage), and what each part of that costs on sm_100a.
// One CTA per SM, 128 converter threads (thread = tile row, 128-byte swizzled rows) plus, optionally, a fifth warp
// whose first thread issues 128 x 128 x 8 TF32 MMAs (A from tensor memory, B from shared memory) back to back for
// the same number of k blocks (12 MMAs each), to see how the two streams slow each other down.
// Variants: full (loads + rounded split + 4 stores of 16 columns + wait), trunc (masked split), no_st (no
// tensor-memory stores), st_only (stores of constants), x32 (2 stores of 32 columns per half pair), wait2 (one
// store wait per two k blocks).  Prints cycles per k block as seen by warp 0.
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o tmem_convert_rate tmem_convert_rate.cu
// Every wait is bounded.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t a) {
    uint64_t d = 0; d |= (uint64_t)((a >> 4) & 0x3FFF); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d;
}
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) { return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24); }
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void st16(uint32_t t, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(t), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void st32(uint32_t t, const uint32_t (&a)[16], const uint32_t (&b)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(t), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
                   "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]),
                   "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(b[8]), "r"(b[9]), "r"(b[10]), "r"(b[11]), "r"(b[12]), "r"(b[13]), "r"(b[14]), "r"(b[15]) : "memory");
}
enum { V_FULL = 0, V_TRUNC, V_NO_ST, V_ST_ONLY, V_X32, V_WAIT2 };

template <int V, bool WITH_MMA>
__global__ void __launch_bounds__(160, 1) convert_kernel(int iters, long long* cycles, int* status, uint32_t* sink) {
    extern __shared__ uint8_t raw[];
    const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
    uint8_t* tile = raw + (base - smem_u32(raw));           // A tile 16 KB, then B 16 KB
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    for (uint32_t i = threadIdx.x; i < 32768 / 4; i += blockDim.x) reinterpret_cast<float*>(tile)[i] = 1.0f + 1e-3f * (float)(i & 1023);
    if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < 4) {
        const int r = threadIdx.x;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16) + 256u;  // A slots start at column 256
        const uint8_t* row0 = tile + r * 128;
        uint32_t keep = 0;
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
            const uint32_t dst = lane_addr + (uint32_t)((it & 3) * 64);
            const uint8_t* row = row0 + (it & 1) * 16384;  // alternate between two tiles: the loads stay in the loop
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t hi[16], lo[16];
                if (V == V_ST_ONLY) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) { hi[i] = (uint32_t)(it + i); lo[i] = (uint32_t)(it - i); }
                } else {
                    float finite = 0.0f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float x[4];
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3])
                                     : "r"(smem_u32(row + (((4 * h + c) ^ (r & 7)) << 4))) : "memory");
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            finite = fmaf(x[t], 0.0f, finite);
                            if (V == V_TRUNC) {
                                const uint32_t b = __float_as_uint(x[t]) & 0xFFFFE000u;
                                hi[4 * c + t] = b;
                                lo[4 * c + t] = __float_as_uint(x[t] - __uint_as_float(b));
                            } else {
                                const uint32_t b = (__float_as_uint(x[t]) + 0x1000u) & 0xFFFFE000u;
                                hi[4 * c + t] = b;
                                lo[4 * c + t] = (__float_as_uint(x[t] - __uint_as_float(b)) + 0x1000u) & 0xFFFFE000u;
                            }
                        }
                    }
                    if (finite != finite) keep ^= 1u;
                }
                if (V == V_NO_ST) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) keep ^= hi[i] + lo[i];
                } else if (V == V_X32) {
                    st32(dst + (uint32_t)(32 * h), hi, lo);  // layout differs from the kernel's: timing only
                } else {
                    st16(dst + (uint32_t)(16 * h), hi);
                    st16(dst + (uint32_t)(32 + 16 * h), lo);
                }
            }
            if (V != V_NO_ST && (V != V_WAIT2 || (it & 1))) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        const long long t1 = clock64();
        if (threadIdx.x == 0) cycles[blockIdx.x * 2] = t1 - t0;
        if (keep == 0x12345678u) sink[0] = keep;
    } else if (WITH_MMA && lane == 0) {
        constexpr uint32_t idesc = make_idesc(128, 128);
        const uint64_t db = make_smem_desc(base + 16384);
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
            const uint32_t a_t = tmem + 256u + (uint32_t)((it & 3) * 64);
#pragma unroll
            for (int m = 0; m < 12; ++m) mma_ts(tmem + (uint32_t)((m & 1) * 128), a_t + (uint32_t)((m & 3) * 8), db + (uint64_t)((m & 3) * 2), idesc, 1u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
        uint32_t ok = 0;
        for (long long spin = 0; spin < 20000ll && !ok; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(&bar)), "r"(0u), "r"(100000u) : "memory");
        cycles[blockIdx.x * 2 + 1] = clock64() - t0;
        if (!ok) atomicExch(status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory"); }
}
template <int V, bool WITH_MMA>
int run(const char* name, int iters) {
    long long* d_cycles; int* d_status; uint32_t* d_sink;
    CK(cudaMalloc(&d_cycles, 148 * 2 * sizeof(long long))); CK(cudaMalloc(&d_status, sizeof(int))); CK(cudaMalloc(&d_sink, 4));
    CK(cudaMemset(d_status, 0, sizeof(int))); CK(cudaMemset(d_cycles, 0, 148 * 2 * sizeof(long long)));
    const int smem = 32768 + 2048;
    CK(cudaFuncSetAttribute(convert_kernel<V, WITH_MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    long long h[296];
    float ms = 0.f;
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int rep = 0; rep < 2; ++rep) {
        CK(cudaEventRecord(e0));
        convert_kernel<V, WITH_MMA><<<148, 160, smem>>>(iters, d_cycles, d_status, d_sink);
        CK(cudaEventRecord(e1));
        CK(cudaDeviceSynchronize()); CK(cudaGetLastError());
        CK(cudaEventElapsedTime(&ms, e0, e1));
        CK(cudaMemcpy(h, d_cycles, sizeof(h), cudaMemcpyDeviceToHost));
    }
    int st; CK(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
    printf("%-34s %8.1f clk per k block (converter)  %8.1f clk per k block (12 MMAs)  kernel %7.3f ms  status %d\n", name, (double)h[0] / iters, (double)h[1] / iters, ms, st);
    cudaFree(d_cycles); cudaFree(d_status); cudaFree(d_sink);
    return 0;
}
int main() {
    const int iters = 20000;
    run<V_FULL, false>("full", iters);
    run<V_TRUNC, false>("trunc split", iters);
    run<V_NO_ST, false>("no tensor-memory stores", iters);
    run<V_ST_ONLY, false>("stores only", iters);
    run<V_X32, false>("32-column stores", iters);
    run<V_WAIT2, false>("store wait every 2 k blocks", iters);
    run<V_FULL, true>("full + MMA stream", iters);
    run<V_TRUNC, true>("trunc split + MMA stream", iters);
    run<V_ST_ONLY, true>("stores only + MMA stream", iters);
    run<V_NO_ST, true>("no stores + MMA stream", iters);
    return 0;
}
