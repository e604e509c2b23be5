// Shared device helpers for the sm_100a kernels of this package.
//
// Every translation unit is compiled once per activation type: -DTL_DTYPE=0 gives
// float (the true 32-bit path), -DTL_DTYPE=1 gives __nv_bfloat16.  Exported
// launchers are plain C functions that take raw device pointers and a stream, so
// the libraries build in seconds and load through ctypes without any binding layer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef TL_DTYPE
#define TL_DTYPE 1
#endif

#if TL_DTYPE == 0
typedef float act_t;
#define TL_NAME(base) base##_f32
#else
typedef __nv_bfloat16 act_t;
#define TL_NAME(base) base##_bf16
#endif

#include "pdl.cuh"   // TL_PAGE, tokens per cache page, comes from the build

// Launch status: 0 = ok, otherwise the cudaError_t of the launch, or a negative
// code for arguments that a kernel refuses.
#define TL_ERR_BAD_ARG (-1)
#define TL_ERR_UNSUPPORTED (-2)

#define TL_LAUNCH_STATUS() ((int)cudaGetLastError())

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions for blocks of up to 1024 threads; `scratch` holds 33 floats.
// All threads receive the result.  Two calls in a row may share the scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

#include "pdl.cuh"
