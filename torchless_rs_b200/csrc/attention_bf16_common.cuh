// Shared pieces of the tensor-core attention kernels of the bfloat16 path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bounded_wait.cuh"
#include "pdl.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#define PAGE TL_PAGE
static_assert(PAGE == 64, "the tensor-core attention kernels lay out their shared-memory slabs, TMA "
                          "boxes and tensor-memory columns for pages of 64 tokens");
#define GROUP 32            // keys per warp iteration
#define NCHUNK (HEAD_DIM / 32)  // 16-byte chunks of a K row per thread
#define NDT (HEAD_DIM / 8)      // 8-wide tiles of the head dimension

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(base) CAT(CAT(base, _hd), HEAD_DIM)

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
