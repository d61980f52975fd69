// Programmatic dependent launch (sm_90+): a kernel launched with the attribute below may be scheduled while its
// predecessor in the stream still runs; it must execute pdl_wait() before it reads or writes anything that kernels
// before it in the stream touch (weights and other constants may be read earlier), and pdl_launch_dependents() lets
// its own successor be scheduled.  In an ordinary launch both instructions do nothing, so a kernel prepared this way
// can be launched either way.  A chain of short dependent kernels (one decode position) saves the launch latency
// between every two of them this way.
#pragma once

#include "common.hpp"

namespace fdk {

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// kernel<<<grid, block, smem, s>>>(args...) with programmatic stream serialisation allowed.
template <typename... KArgs, typename... Args>
void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FDK_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}
#endif

}  // namespace fdk
