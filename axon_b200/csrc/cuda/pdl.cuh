// Programmatic dependent launch: a kernel may start while the kernel before it on the
// stream is still running, do whatever does not depend on that kernel (set-up, loading
// weights), and wait for it only before it touches data the earlier kernel produces or
// still reads.  The reference chains its decode kernels the same way
// (src/cuda/decode.cu:23-43).
//
// Rules kept by every kernel launched through launch_pdl:
//  * pdl_launch_dependents() at the top lets the next kernel begin its independent part;
//  * pdl_wait() comes before the first read of anything an earlier kernel writes and
//    before the first global write of any kind (an earlier kernel may still be reading
//    the target).  After it, all memory operations of all earlier kernels are visible.
//  * Before pdl_wait() a kernel only reads data that no kernel of the step writes
//    (weights, tensor maps) and touches its own shared and tensor memory.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace axon {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with the programmatic-serialization attribute (works inside stream capture too).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // AXON_PDL=0 in the environment launches everything fully serialised (for measurements)
    static const int allowed = [] { const char* e = getenv("AXON_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = allowed;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace axon
