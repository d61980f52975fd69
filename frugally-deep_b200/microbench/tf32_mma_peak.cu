// Micro-benchmark: the issue and execution rate of tcgen05.mma.kind::tf32 on sm_100a.
// One CTA per SM; one thread issues 128 x N x 8 MMAs back to back (operands all zero, A from shared memory or
// from tensor memory, 1 to 4 accumulators in rotation) and commits once at the end.  Prints cycles per MMA and
// the aggregate rate.  This is the denominator behind the contraction kernel's "issued" roofline fraction, and
// the source of its design rule that one thread cannot issue more than one MMA per ~45 cycles.
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o tf32_mma_peak tf32_mma_peak.cu
// Every wait is bounded (2 s).
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t a) {
    uint64_t d = 0; d |= (uint64_t)((a >> 4) & 0x3FFF); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d;
}
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) { return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24); }
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
template <int N, bool A_TMEM, int NACC>
__global__ void __launch_bounds__(128, 1) peak_kernel(int iters, long long* cycles, int* status) {
    extern __shared__ uint8_t raw[];
    const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    // zero the operand tiles: A 16 KB at base, B N*128 bytes after it
    for (uint32_t i = threadIdx.x; i < (16384 + N * 128) / 4; i += blockDim.x) asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + i * 4), "r"(0u));
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
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = make_idesc(128, N);
        const uint64_t da = make_smem_desc(base), db = make_smem_desc(base + 16384);
        const uint32_t a_t = tmem + (uint32_t)(NACC * N);  // A in TMEM (garbage values: timing only)
        const long long t0 = clock64();
        for (int i = 0; i < iters; ++i) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t d = tmem + (uint32_t)(((i * 4 + kk) % NACC) * N);
                if (A_TMEM) mma_ts(d, a_t + kk * 8, db + (uint64_t)(kk * 2), idesc, 1u);
                else mma_ss(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, 1u);
            }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
        uint32_t ok = 0;
        for (long long spin = 0; spin < 20000ll && !ok; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(&bar)), "r"(0u), "r"(100000u) : "memory");
        const long long t1 = clock64();
        cycles[blockIdx.x] = t1 - t0;
        if (!ok) atomicExch(status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory"); }
}
template <int N, bool A_TMEM, int NACC>
int run(const char* name, int iters) {
    long long* d_cycles; int* d_status;
    CK(cudaMalloc(&d_cycles, 148 * sizeof(long long))); CK(cudaMalloc(&d_status, sizeof(int))); CK(cudaMemset(d_status, 0, sizeof(int)));
    const int smem = 16384 + N * 128 + 2048;
    CK(cudaFuncSetAttribute(peak_kernel<N, A_TMEM, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    float best = 1e30f; long long cyc = 0;
    for (int rep = 0; rep < 3; ++rep) {
        CK(cudaEventRecord(e0));
        peak_kernel<N, A_TMEM, NACC><<<148, 128, smem>>>(iters, d_cycles, d_status);
        CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1)); CK(cudaGetLastError());
        float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); if (ms < best) best = ms;
        long long h[148]; CK(cudaMemcpy(h, d_cycles, sizeof(h), cudaMemcpyDeviceToHost)); cyc = h[0];
    }
    int st; CK(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
    const double mmas = (double)iters * 4;
    const double flops = mmas * 2.0 * 128 * N * 8 * 148;
    printf("%-28s %8.3f ms  %7.1f clk/mma  %7.1f TF/s issued  status %d\n", name, best, (double)cyc / mmas, flops / best / 1e9, st);
    cudaFree(d_cycles); cudaFree(d_status);
    return 0;
}
int main() {
    const int iters = 20000;
    run<128, false, 1>("N=128 A=smem 1 acc", iters);
    run<128, false, 2>("N=128 A=smem 2 acc", iters);
    run<128, true, 1>("N=128 A=tmem 1 acc", iters);
    run<128, true, 2>("N=128 A=tmem 2 acc", iters);
    run<256, false, 1>("N=256 A=smem 1 acc", iters);
    run<256, true, 1>("N=256 A=tmem 1 acc", iters);
    run<64, false, 1>("N=64 A=smem 1 acc", iters);
    run<64, true, 1>("N=64 A=tmem 1 acc", iters);
    run<64, true, 4>("N=64 A=tmem 4 acc", iters);
    return 0;
}
