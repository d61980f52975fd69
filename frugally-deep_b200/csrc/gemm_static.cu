// The tensor-core contraction for callers that must not allocate device memory.
//
// Who needs this.  fdk_gemm's tensor-core path asks the CUDA allocator for a temporary buffer on every
// call, to hold the two TF32 halves of the weight matrix.  Some callers cannot afford that, or are not
// allowed to:
//   * a serving loop with a latency budget: cudaMalloc and cudaFree take a device-wide lock and cudaFree
//     waits for the whole device to go idle, so one call stalls every other stream of the process;
//   * a host application that has already handed (nearly) all of the GPU's memory to its own pool (a tensor
//     framework's caching allocator, a database buffer manager): the runtime allocator then simply fails;
//   * code that runs between the bookkeeping points of such a pool and must leave the amount of free device
//     memory unchanged.
// For them the halves live in a fixed array that is part of the loaded library image on every device.  Its
// size is fixed when the library is built, so matrices beyond that size are refused; nothing is ever
// allocated or freed here, neither through the CUDA runtime nor through any library.
//
// Consequences of one shared array (per device):
//   * all calls on a device use the same floats.  Calls queued on ONE stream run in order and are safe.  Calls
//     that can overlap on the GPU (different streams, several host threads with their own streams) race on
//     the array and produce garbage; the caller has to serialise them.
//   * the array keeps whatever the previous call left in it.  Nothing needs to start at zero: every float that
//     the contraction reads (the first K floats of N rows, ldw apart, in each half) is rewritten by the same
//     call's split kernel, queued on the same stream in front of the contraction.  Only those floats of W are
//     read: the ldw - K floats between rows (and after the last row) may lie outside the caller's allocation.
//   * the first call on each device looks the array's device address up and may load the kernels; make that
//     first call before starting any stream capture.
#include "kernels.cuh"

#include <mutex>

namespace fdk {

// Largest weight matrix, in floats including row padding (N * ldw).  Two halves of this size: 8 MiB per device.
constexpr int64_t STATIC_WEIGHT_FLOATS = 1 << 20;

// Only device code and cudaGetSymbolAddress may refer to this name; the host never uses it as an address.
static __device__ __align__(256) float g_weight_halves[2 * STATIC_WEIGHT_FLOATS];

constexpr int MAX_DEVICES = 64;
static std::mutex g_lookup_mutex;
static float* g_halves_addr[MAX_DEVICES] = {};

// Device address of the array on the CURRENT device (each device holds its own copy of the image).
static float* halves_on_current_device() {
    int dev = -1;
    FDK_CUDA(cudaGetDevice(&dev));
    ensure(dev >= 0 && dev < MAX_DEVICES, "fdk_gemm_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_lookup_mutex);
    if (g_halves_addr[dev] == nullptr) {
        float* p = nullptr;
        FDK_CUDA(cudaGetSymbolAddress((void**)&p, g_weight_halves));
        ensure(p != nullptr, "fdk_gemm_static: the scratch array has no device address");
        g_halves_addr[dev] = p;
    }
    return g_halves_addr[dev];
}

// big = rna_tf32(w), small = rna_tf32(w - big) for the first K floats of each of the N rows (ldw apart), written at
// the same offsets of the two halves (half_stride floats apart).  The padding between rows is neither read nor written.
__global__ void split_into_static_kernel(const float* __restrict__ w, float* __restrict__ halves, long long half_stride, long long ldw,
                                         int K, long long n_values) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_values; i += (long long)gridDim.x * blockDim.x) {
        const long long at = (i / K) * ldw + (i % K);
        const float x = w[at];
        uint32_t hi, lo;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
        halves[at] = __uint_as_float(hi);
        halves[half_stride + at] = __uint_as_float(lo);
    }
}

int64_t gemm_static_max_weight_floats() { return STATIC_WEIGHT_FLOATS; }

void launch_gemm_tc_static(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc, int64_t M, int N, int K,
                           const Epilogue& e, cudaStream_t s) {
    ensure(A && W && C && N > 0 && ldw > 0, "fdk_gemm_static: invalid argument");
    ensure(K > 0 && K <= ldw && K <= lda, "fdk_gemm_static: K must not exceed the row strides lda and ldw");
    const int64_t n = (int64_t)N * ldw;
    if (n > STATIC_WEIGHT_FLOATS)
        raise("fdk_gemm_static: the weight matrix has " + std::to_string(n) + " floats (N * ldw); the built-in scratch holds at most " +
              std::to_string(STATIC_WEIGHT_FLOATS) + ".  Use fdk_gemm_presplit with buffers of your own for larger matrices.");
    ensure(gemm_tc_supported(M, N, K, lda, ldw, A, W), "fdk_gemm_static: shape not supported by the tensor-core path");
    float* halves = halves_on_current_device();
    const int64_t n_values = (int64_t)N * K;
    int64_t grid = (n_values + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    split_into_static_kernel<<<(unsigned)grid, 256, 0, s>>>(W, halves, (long long)STATIC_WEIGHT_FLOATS, (long long)ldw, K, (long long)n_values);
    FDK_CUDA(cudaGetLastError());
    launch_gemm_tc(A, lda, halves, halves + STATIC_WEIGHT_FLOATS, ldw, C, ldc, M, N, K, e, s);
}

}  // namespace fdk
