// Kernel launch with programmatic dependent launch (PDL).
//
// The kernels of one ABI call form a chain in the caller's stream.  With the attribute set, a
// kernel may begin (block scheduling, shared-memory set-up, loads of tensors the call received as
// INPUTS) while the blocks of its predecessor in the chain are still draining; it calls
// pdl_wait() before it touches anything the predecessor wrote.  Rules kept by every user:
//   * the first kernel of an ABI call is launched WITHOUT the attribute (what precedes it in the
//     stream is not ours and may still be writing our inputs);
//   * every kernel of a chain executes pdl_wait() at some point, so that "my predecessor has
//     completed" implies "everything before it has completed" all along the chain;
//   * nothing is written to global memory before pdl_wait().
// pdl_trigger() at the top of a kernel lets its successor be scheduled as soon as every block of
// this kernel is resident; in a kernel launched without the attribute both calls are no-ops.
#pragma once

#include <cuda_runtime.h>

namespace mhc {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                         bool dependent, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace mhc
