// Launch helper and device calls for programmatic dependent launch, shared by all kernels.
#pragma once
#include <cuda_runtime.h>

// Tokens per cache page.  The build gives the number (build.py: PAGE_TOKENS), so that the host's
// page arithmetic and every kernel's agree by construction.
#ifndef TL_PAGE
#error "TL_PAGE (tokens per cache page) must be given by the build: -DTL_PAGE=<n>"
#endif

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
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
