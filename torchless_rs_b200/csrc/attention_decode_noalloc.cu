// Implementation of attention_decode_noalloc.h: the split-KV decode attention with its
// scratch in a fixed device array of this library instead of a buffer from the caller.
// The kernels are those of attention_decode_bf16.cu, compiled into this translation
// unit so that they can be launched from here; the ordinary library is not touched.
#include "attention_decode_bf16.cu"
#include "attention_decode_noalloc.h"

#include <mutex>

// Partial results of the key splits.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) float tl_noalloc_scratch[TL_NOALLOC_SCRATCH_FLOATS];

#define TL_MAX_DEVICES 64
static float* g_scratch_ptr[TL_MAX_DEVICES];   // device address of the array, per device
static std::mutex g_setup_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= TL_MAX_DEVICES) return TL_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, tl_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return TL_NOALLOC_SETUP_FAILED;
    g_scratch_ptr[dev] = p;
  }
  *ptr = g_scratch_ptr[dev];
  return 0;
}

extern "C" int FN(tl_attn_decode_noalloc)(const void* q, const void* k_pages, const void* v_pages,
                                          void* out, const int* seq_len, const int* seq_slot,
                                          const int* page_table, int table_stride, int B, int nh,
                                          int nkv, int window, float scale, int n_splits,
                                          cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nh <= 0 || n_splits < 1) return -2;
  const long long need = FN(tl_attn_decode_scratch_floats)(B, nh, n_splits);
  if (need > (long long)TL_NOALLOC_SCRATCH_FLOATS) return TL_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int st = scratch_for_current_device(&scratch);
  if (st != 0) return st;
  return FN(tl_attn_decode)(q, k_pages, v_pages, out, scratch, seq_len, seq_slot, page_table,
                            table_stride, B, nh, nkv, window, scale, n_splits, stream);
}

extern "C" const char* tl_attn_decode_noalloc_error(int code) {
  switch (code) {
    case 0: return "ok";
    case -2: return "these sizes are not supported by the decode attention kernel";
    case TL_NOALLOC_TOO_LARGE:
      return "sequences * heads * splits * (head_dim + 2) exceeds the fixed scratch of "
             "2 Mi floats; lower the number of splits or the batch";
    case TL_NOALLOC_SETUP_FAILED:
      return "the device address of the fixed scratch array could not be obtained";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error code";
  }
}
