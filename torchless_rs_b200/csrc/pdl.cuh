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

// ---------------------------------------------------------------------------
// Timeline of a step (diagnostic build only, -DTL_TRACE; `measure timeline` builds with it).
// A traced kernel notes the GPU's global nanosecond timer when its first block starts and when
// its last block ends, so that overlaps and gaps between the kernels of a CUDA graph with
// programmatic dependent launch can be seen, which no per-kernel profiler shows.  Every
// translation unit keeps its own records; TL_TRACE_EXPORT(name) gives the host a reader.
// ---------------------------------------------------------------------------
#ifdef TL_TRACE
#define TL_TRACE_MAX 8192
#define TL_TRACE_KEYS 64
static __device__ unsigned long long tl_trace_buf[TL_TRACE_MAX * 4];   // kind + 256 extra, start, released, end
static __device__ unsigned int tl_trace_n;
static __device__ unsigned int tl_trace_cur[TL_TRACE_KEYS];    // record of the launch in flight, per key
static __device__ unsigned int tl_trace_done[TL_TRACE_KEYS];
__device__ __forceinline__ unsigned long long tl_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// `key` tells launches apart that may be in flight at the same time (neighbours in the stream
// overlap under programmatic dependent launch); launches with the same key must not overlap.
struct TlTraceScope {
  int key;
  __device__ __forceinline__ TlTraceScope(int kind, long long extra, int key_) : key(key_ % TL_TRACE_KEYS) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
      const unsigned int s = atomicAdd(&tl_trace_n, 1u);
      if (s < TL_TRACE_MAX) {
        tl_trace_buf[4 * s] = (unsigned long long)kind + 256ull * (unsigned long long)extra;
        tl_trace_buf[4 * s + 1] = tl_globaltimer();
        tl_trace_buf[4 * s + 2] = 0;
      }
      tl_trace_cur[key] = s;
      __threadfence();
    }
  }
  // after the wait for the kernels before: block 0 notes when it was let go
  __device__ __forceinline__ void released() {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
      const unsigned int s = tl_trace_cur[key];
      if (s < TL_TRACE_MAX && tl_trace_buf[4 * s + 2] == 0) tl_trace_buf[4 * s + 2] = tl_globaltimer();
    }
  }
  __device__ __forceinline__ ~TlTraceScope() {
    if (threadIdx.x == 0) {
      const unsigned int nb = gridDim.x * gridDim.y * gridDim.z;
      if (atomicAdd(&tl_trace_done[key], 1u) == nb - 1) {
        tl_trace_done[key] = 0;
        const unsigned int s = tl_trace_cur[key];
        if (s < TL_TRACE_MAX) tl_trace_buf[4 * s + 3] = tl_globaltimer();
      }
    }
  }
};
#define TL_TRACE_SCOPE(kind, extra, key) TlTraceScope tl_trace_scope_((kind), (long long)(extra), (key))
#define TL_TRACE_RELEASED() tl_trace_scope_.released()
// Copies the records to `host` (room for `max` records of four 64-bit words), clears them and
// returns their number.  Synchronises the device.
#define TL_TRACE_EXPORT(name)                                                               \
  extern "C" int tl_trace_take_##name(unsigned long long* host, int max) {                  \
    unsigned int n = 0, zero = 0;                                                           \
    if (cudaMemcpyFromSymbol(&n, tl_trace_n, sizeof(n)) != cudaSuccess) return -1;          \
    if (n > TL_TRACE_MAX) n = TL_TRACE_MAX;                                                 \
    if ((int)n > max) n = (unsigned int)max;                                                \
    if (n && cudaMemcpyFromSymbol(host, tl_trace_buf, (size_t)n * 32) != cudaSuccess) return -1; \
    cudaMemcpyToSymbol(tl_trace_n, &zero, sizeof(zero));                                    \
    return (int)n;                                                                          \
  }
#else
#define TL_TRACE_SCOPE(kind, extra, key)
#define TL_TRACE_RELEASED()
#define TL_TRACE_EXPORT(name)
#endif
