// Matrix products on CUDA cores with 32-bit accumulation, for every size.
//
//   C[M, N] (op)= A[M, K] * W[N, K]^T        A, W of act_t, K contiguous in both
//
// These kernels are the whole of the true 32-bit path (no tensor-core mode of
// reduced precision is ever used there) and the fallback of the bfloat16 path for
// shapes that the tensor-core kernels refuse.  The reference computes each output as
// one sequential 32-bit dot product (src/loader/parameters.rs:551-594).
//
// Output modes:
//   0  C (float)  = product
//   1  C (float) += product                     (residual sum kept in 32-bit)
//   2  C (act_t)  = silu(g) * u, where W holds N gate rows followed by N up rows
//   3  C (act_t)  = product
#include "common.cuh"

#define MODE_STORE_F32 0
#define MODE_ACCUM_F32 1
#define MODE_SWIGLU 2
#define MODE_STORE_ACT 3

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

template <int MODE>
__device__ __forceinline__ void store_out(void* C, int ldc, int m, int n, float v, float u) {
  if (MODE == MODE_STORE_F32) {
    ((float*)C)[(size_t)m * ldc + n] = v;
  } else if (MODE == MODE_ACCUM_F32) {
    ((float*)C)[(size_t)m * ldc + n] += v;
  } else if (MODE == MODE_SWIGLU) {
    ((act_t*)C)[(size_t)m * ldc + n] = from_f32<act_t>(silu_f(v) * u);
  } else {
    ((act_t*)C)[(size_t)m * ldc + n] = from_f32<act_t>(v);
  }
}

// ---------------------------------------------------------------------------
// Tiled kernel: 64x64 output tile, 16-wide K steps, 256 threads with 4x4 outputs each.
// ---------------------------------------------------------------------------
#define BM 64
#define BN 64
#define BK 16

template <int MODE>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const act_t* __restrict__ A, int lda, const act_t* __restrict__ W, int ldw,
                  void* __restrict__ C, int ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[MODE == MODE_SWIGLU ? BK : 1][BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {}, acu[4][4] = {};
  // loader mapping: 64 rows x 16 k; each thread takes 4 consecutive k of one row
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + j][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.0f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.0f;
      if (MODE == MODE_SWIGLU)
        Us[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)(N + wn) * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
      if (MODE == MODE_SWIGLU) {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = Us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (MODE == MODE_SWIGLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) store_out<MODE>(C, ldc, m, n, acc[i][j], acu[i][j]);
    }
  }
}

// ---------------------------------------------------------------------------
// Skinny kernel for up to 8 rows of A: one warp per output column streams one row
// of W (two in SwiGLU mode) once, with 16-byte loads when the row stride allows it.
// ---------------------------------------------------------------------------
#if TL_DTYPE == 0
#define VEC 4
#else
#define VEC 8
#endif

__device__ __forceinline__ void load_vec(const act_t* p, float* out) {
#if TL_DTYPE == 0
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
#else
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
#endif
}

template <int MODE, int MB, bool VECTOR>
__global__ void __launch_bounds__(256)
gemm_skinny_kernel(const act_t* __restrict__ A, int lda, const act_t* __restrict__ W, int ldw,
                   void* __restrict__ C, int ldc, int M, int N, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const act_t* wrow = W + (size_t)n * ldw;
  const act_t* urow = W + (size_t)(N + n) * ldw;
  float acc[MB], acu[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = acu[m] = 0.0f;
  if (VECTOR) {
    for (int k = lane * VEC; k < K; k += 32 * VEC) {
      float w[VEC], u[VEC], a[VEC];
      load_vec(wrow + k, w);
      if (MODE == MODE_SWIGLU) load_vec(urow + k, u);
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < M) {
          load_vec(A + (size_t)m * lda + k, a);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            acc[m] = fmaf(a[i], w[i], acc[m]);
            if (MODE == MODE_SWIGLU) acu[m] = fmaf(a[i], u[i], acu[m]);
          }
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float w = to_f32(wrow[k]);
      const float u = MODE == MODE_SWIGLU ? to_f32(urow[k]) : 0.0f;
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < M) {
          const float a = to_f32(A[(size_t)m * lda + k]);
          acc[m] = fmaf(a, w, acc[m]);
          if (MODE == MODE_SWIGLU) acu[m] = fmaf(a, u, acu[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    acc[m] = warp_sum(acc[m]);
    if (MODE == MODE_SWIGLU) acu[m] = warp_sum(acu[m]);
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MB; ++m)
      if (m < M) store_out<MODE>(C, ldc, m, n, acc[m], acu[m]);
  }
}

template <int MODE>
static int launch_mode(const act_t* A, int lda, const act_t* W, int ldw, void* C, int ldc, int M,
                       int N, int K, cudaStream_t stream) {
  if (M <= 8) {
    const bool vec = (K % VEC == 0) && (lda % VEC == 0) && (ldw % VEC == 0) &&
                     ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    const int warps = 8;
    dim3 grid((N + warps - 1) / warps), block(warps * 32);
#define SKINNY(MB)                                                                               \
  return vec ? tl_launch(gemm_skinny_kernel<MODE, MB, true>, grid, block, 0, stream, A, lda, W,  \
                         ldw, C, ldc, M, N, K)                                                   \
             : tl_launch(gemm_skinny_kernel<MODE, MB, false>, grid, block, 0, stream, A, lda, W, \
                         ldw, C, ldc, M, N, K)
    if (M == 1) SKINNY(1);
    else if (M == 2) SKINNY(2);
    else if (M <= 4) SKINNY(4);
    else SKINNY(8);
#undef SKINNY
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  return tl_launch(gemm_tiled_kernel<MODE>, grid, dim3(256), 0, stream, A, lda, W, ldw, C, ldc, M, N, K);
}

// N counts output columns; in SwiGLU mode W has 2*N rows.
extern "C" int TL_NAME(tl_gemm_generic)(const void* A, int lda, const void* W, int ldw, void* C,
                                        int ldc, int M, int N, int K, int mode,
                                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return TL_ERR_BAD_ARG;
  const act_t* a = (const act_t*)A;
  const act_t* w = (const act_t*)W;
  switch (mode) {
    case MODE_STORE_F32: return launch_mode<MODE_STORE_F32>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    case MODE_ACCUM_F32: return launch_mode<MODE_ACCUM_F32>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    case MODE_SWIGLU: return launch_mode<MODE_SWIGLU>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    case MODE_STORE_ACT: return launch_mode<MODE_STORE_ACT>(a, lda, w, ldw, C, ldc, M, N, K, stream);
  }
  return TL_ERR_BAD_ARG;
}
