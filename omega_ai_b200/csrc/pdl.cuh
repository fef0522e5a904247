// Programmatic dependent launch: a kernel launched with the attribute below may be scheduled as soon as every
// CTA of the kernel before it in the stream has executed pdl_trigger() (or exited), so its launch latency and its
// prologue (barrier set-up, tensor-memory allocation) overlap the tail of its predecessor.  It must execute
// pdl_wait() before it touches anything the predecessor reads or writes: that returns once the predecessor has
// completed and its memory operations are visible.  In a kernel launched without the attribute both
// instructions do nothing, so every kernel of the forward chain carries them and the launch site decides.
#pragma once

#include <cuda_runtime.h>

#include <utility>

namespace omoe {

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with (pdl) or without the programmatic-serialization attribute; arguments are converted to the
// kernel's parameter types.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                             Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

}  // namespace omoe
