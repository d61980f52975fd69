// Inline-PTX wrappers for the sm_100a features the contraction kernels are built from: mbarriers, TMA tensor copies,
// tensor memory (tcgen05.alloc / ld / st), tcgen05.mma descriptors and commits.  Shared by gemm_tc.cu and gemm_rows.cu.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace fdk {

// try_wait suspends the warp in hardware until the phase completes or a time limit passes (hint: 20 us),
// so waiting roles do not compete for issue slots with the working ones.
constexpr uint32_t TC_WAIT_HINT_NS = 20000;

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
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(TC_WAIT_HINT_NS)
        : "memory");
    return ok != 0;
}
// Non-blocking test of up to five barrier phases in one round trip (all tests are in flight together).
__device__ __forceinline__ bool mbar_test5(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1, uint32_t b2, uint32_t p2, uint32_t b3,
                                           uint32_t p3, uint32_t b4, uint32_t p4) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred q0, q1, q2, q3, q4;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q0, [%1], %2;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q1, [%3], %4;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q2, [%5], %6;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q3, [%7], %8;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q4, [%9], %10;\n\t"
        "and.pred q0, q0, q1;\n\t"
        "and.pred q2, q2, q3;\n\t"
        "and.pred q0, q0, q2;\n\t"
        "and.pred q0, q0, q4;\n\t"
        "selp.b32 %0, 1, 0, q0;\n\t}"
        : "=r"(ok)
        : "r"(b0), "r"(p0), "r"(b1), "r"(p1), "r"(b2), "r"(p2), "r"(b3), "r"(p3), "r"(b4), "r"(p4)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test3(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1, uint32_t b2, uint32_t p2) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred q0, q1, q2;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q0, [%1], %2;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q1, [%3], %4;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q2, [%5], %6;\n\t"
        "and.pred q0, q0, q1;\n\t"
        "and.pred q0, q0, q2;\n\t"
        "selp.b32 %0, 1, 0, q0;\n\t}"
        : "=r"(ok)
        : "r"(b0), "r"(p0), "r"(b1), "r"(p1), "r"(b2), "r"(p2)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test2(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred q0, q1;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q0, [%1], %2;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q1, [%3], %4;\n\t"
        "and.pred q0, q0, q1;\n\t"
        "selp.b32 %0, 1, 0, q0;\n\t}"
        : "=r"(ok)
        : "r"(b0), "r"(p0), "r"(b1), "r"(p1)
        : "memory");
    return ok != 0;
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

// Tiled 4-D load into this CTA only.  c0 is a multiple of 32 floats, so the innermost coordinate is 16-byte
// aligned; the spatial coordinates may be negative or beyond the image: those elements read as zero.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int x, int y, int b, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(x), "r"(y), "r"(b), "r"(bar)
        : "memory");
}

// Tiled 4-D store of a shared-memory box (bulk async group of the issuing thread).  Elements outside the
// tensor are not written; the start coordinates are never negative and c0 is a multiple of 32 floats.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int x, int y, int b) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(x), "r"(y), "r"(b)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most PENDING of this thread's bulk groups still read their shared-memory source.
template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <int REGS>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS)); }
template <int REGS>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS)); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
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
// Each lane reads 16 consecutive columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Each lane writes 16 consecutive columns of its own TMEM lane (the warp's lane quadrant).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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

}  // namespace fdk
