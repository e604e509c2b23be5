// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in rglonek/torchless-rs; it exists for users of
// this library only.
//
// Who needs it: code that runs where cudaMalloc is not allowed or not safe.  Examples
// are a plugin inside a host application that owns the whole device heap and hands
// out fixed buffers, a real-time loop that may not take the allocator's lock or its
// implicit device synchronisation, and a process that has already given all free
// device memory to its own pool.  The ordinary entry point, tl_attn_decode_hd<N>,
// needs a scratch buffer for the partial results of its key splits, and someone has
// to allocate that buffer (this package's Python side does, through torch).  The
// entry point below needs none: its scratch is a fixed array inside the library.
//
// What it costs: TL_NOALLOC_SCRATCH_FLOATS 32-bit floats (8 MiB) of device memory on
// every GPU on which the library is used, from the moment the library's module is
// loaded there until the process exits.
//
// Limit: sequences * heads * splits * (HEAD_DIM + 2) must not exceed
// TL_NOALLOC_SCRATCH_FLOATS; a larger request is refused with TL_NOALLOC_TOO_LARGE
// and nothing is launched.  Lower `n_splits` (or the batch) to fit.
//
// First call on each device: looks up the device address of the scratch array
// (cudaGetSymbolAddress) for the device that is current at that moment and keeps it.
// Make that first call outside any stream capture.
//
// Sharing: every call on a device uses the same array.  Calls that may overlap on the
// GPU (different streams without an ordering between them) race on it; put them on
// one stream or order them with events.  The array keeps what the last call wrote;
// nothing in it has to be cleared between calls, because each call writes every
// element that it later reads.
//
// It calls no cudaMalloc, cudaFree or other allocating routine.  Inputs and outputs
// are the caller's, exactly as for tl_attn_decode_hd<N>.
#pragma once
#include <cuda_runtime.h>

#define TL_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TL_NOALLOC_TOO_LARGE (-3)
#define TL_NOALLOC_SETUP_FAILED (-4)

#ifdef __cplusplus
extern "C" {
#endif

// One per compiled head size: tl_attn_decode_noalloc_hd32, _hd64, _hd128.
// Returns 0, a positive cudaError_t of the set-up or a launch, -2 for sizes the kernel
// does not take, TL_NOALLOC_TOO_LARGE, or TL_NOALLOC_SETUP_FAILED.
#define TL_NOALLOC_DECLARE(hd)                                                                  \
  int tl_attn_decode_noalloc_hd##hd(const void* q, const void* k_pages, const void* v_pages,    \
                                    void* out, const int* seq_len, const int* seq_slot,         \
                                    const int* page_table, int table_stride, int B, int nh,     \
                                    int nkv, int window, float scale, int n_splits,             \
                                    cudaStream_t stream);
TL_NOALLOC_DECLARE(32)
TL_NOALLOC_DECLARE(64)
TL_NOALLOC_DECLARE(128)

// A sentence for a return code of the functions above.
const char* tl_attn_decode_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
