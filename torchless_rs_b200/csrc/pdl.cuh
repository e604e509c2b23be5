// Launch helper and device calls for programmatic dependent launch, shared by all kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this package is launched with the
// programmatic-serialisation attribute: it may start while the kernel before it in the
// stream is still draining, so its launch latency and set-up overlap that tail.  In
// return every kernel calls pdl_wait() before it reads or writes anything an earlier
// kernel may have touched; the call returns once all earlier kernels have completed and
// their writes are visible.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline int tl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  static const int pdl_on = getenv("TL_NO_PDL") ? 0 : 1;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_on;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
