// Waiting on an mbarrier with a limit.
//
// A kernel of this package never waits for ever: a wait polls at most TL_WAIT_LIMIT times.
// When the limit is hit the waiting thread writes `code` into the block's `abort_flag` (other
// roles of the block see it at their next look and stop waiting too) and into the library's
// error word in global memory (the first code stays), and the wait returns false.  The caller
// then skips its work, frees what it holds (tensor memory) and returns, so the context stays
// usable and the host can read the word.
#pragma once
#include <stdint.h>

#ifndef TL_WAIT_LIMIT
#define TL_WAIT_LIMIT (1u << 22)
#endif

__device__ __forceinline__ uint32_t tl_smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void tl_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tl_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool tl_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(tl_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false when the limit is hit or another role of the block has given up.
__device__ __forceinline__ bool tl_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                             int code, int* error_word) {
  for (uint32_t i = 0; i < TL_WAIT_LIMIT; ++i) {
    if (tl_mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = code;
  atomicCAS(error_word, 0, code);
  return false;
}
