// Programmatic dependent launch: a kernel launched with launch_pdl may become resident while the previous kernel of
// the stream is still running (its blocks are scheduled as soon as every block of that kernel has called pdl_go or
// exited), and must call pdl_wait before it touches anything the previous kernel wrote.  Every kernel launched this
// way calls pdl_wait in all of its threads before any of them can exit, so that "the previous kernel has completed"
// carries through a chain of such launches.
#pragma once
#include <cuda_runtime.h>

namespace infr {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_go() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace infr
