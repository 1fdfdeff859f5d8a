// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may start
// while the kernel before it in the stream is still running; pdl_wait() blocks the calling thread until that kernel
// has completed and its writes are visible (a no-op for a normally launched kernel).  pdl_launch_dependents() tells the
// device that, as far as this CTA is concerned, the next kernel of the stream may begin to start: its CTAs become
// resident where there is room and run up to their own pdl_wait().  Only kernels that call pdl_wait() before they touch
// global memory are ever launched with the attribute; every kernel may call pdl_launch_dependents().
#pragma once
#include <cuda_runtime.h>

namespace ob200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace ob200
