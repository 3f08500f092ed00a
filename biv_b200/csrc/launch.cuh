// Kernel launches with programmatic dependent launch: the kernel may be scheduled while
// the previous kernel of the stream is still draining, so that its launch latency and its
// prologue (barrier set-up, shared-memory carving) overlap the predecessor's tail.  Every
// kernel launched this way calls pdl_wait() before it touches anything an earlier kernel
// of the stream wrote - in every thread, before any early return - which is what keeps
// the chain of dependencies intact: a kernel that has passed its wait knows that its
// predecessor, and through the predecessor's own wait everything before it, is complete.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>

namespace bivmoe {

__device__ __forceinline__ void pdl_wait() {
    // without the launch attribute this is a no-op
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets the next kernel of the stream be scheduled once every block of this one has got
// here (or exited): placed at the top of a kernel, the successor's blocks fill in as this
// kernel's last wave drains, and then sit in their own pdl_wait().
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// both, for kernels with nothing to do before their inputs are ready
__device__ __forceinline__ void pdl_enter() {
    pdl_launch_dependents();
    pdl_wait();
}

template <class... KArgs, class... Args>
inline cudaError_t launch_after(cudaStream_t stream, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                size_t smem, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // Off unless BIVMOE_PDL=1 (read once; a tuning aid): measured on a B200 at the decode
    // shape the overlapped chain was 4-5 us per pass SLOWER than plain launches replayed
    // from a CUDA graph (100.7 against 95.2 us), so plain launches are the default.
    static const bool overlap = [] { const char* e = getenv("BIVMOE_PDL"); return e && atoi(e) != 0; }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace bivmoe
