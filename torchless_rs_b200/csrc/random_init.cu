// Random weights drawn on the device, bit for bit the values that weights/random_init.py
// draws on the host for the same (seed, tensor name, element index).
//
// The reference has no seeded generator (its test fixture is drawn with numpy's unseeded
// normal, tests/generate_test_model.py:89-110).  Here element i of a tensor is a function of
// the tensor's 64-bit key and i alone: a counter-based generator, so any part of any tensor can
// be drawn anywhere, in any order.  Normal numbers come from the Box-Muller transform with its
// logarithm, sine and cosine written out as fixed sequences of correctly rounded double
// operations (__dadd_rn, __dmul_rn, __ddiv_rn, __dsqrt_rn: never fused), with the same
// constants as the host passes in, so that a CPU that follows the same sequence gets the same bits.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct RandomConsts {
  double ln2, half_pi, sqrt_half;
  double ln_c[12];    // 1/1, 1/3, ..., 1/23
  double sin_c[11];   // 1/1!, -1/3!, ..., +1/21!
  double cos_c[12];   // 1/0!, -1/2!, ..., -1/22!
};

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// One standard normal number for element `i`: elements 2c and 2c + 1 share the counter c and
// take the cosine and the sine branch.
__device__ double normal_of(uint64_t key, uint64_t i, const RandomConsts& k) {
  const uint64_t bits = mix64(key + ((i >> 1) + 1) * 0x9E3779B97F4A7C15ull);
  const uint32_t k1 = (uint32_t)(bits >> 32), k2 = (uint32_t)bits;
  // u1 in (0, 1]; ln(u1) = e ln 2 + ln(m), m in [sqrt(1/2), sqrt(2)), ln(m) = 2 atanh((m-1)/(m+1))
  const double u1 = __dmul_rn((double)k1 + 1.0, 1.0 / 4294967296.0);
  int e;
  double m = frexp(u1, &e);          // exact: u1 = m 2^e, m in [1/2, 1)
  if (m < k.sqrt_half) { m = __dmul_rn(m, 2.0); e -= 1; }
  const double s = __ddiv_rn(__dadd_rn(m, -1.0), __dadd_rn(m, 1.0));
  const double s2 = __dmul_rn(s, s);
  double p = k.ln_c[11];
#pragma unroll
  for (int j = 10; j >= 0; --j) p = __dadd_rn(__dmul_rn(p, s2), k.ln_c[j]);
  const double ln_u = __dadd_rn(__dmul_rn((double)e, k.ln2), __dmul_rn(__dmul_rn(2.0, s), p));
  const double r = __dsqrt_rn(__dmul_rn(-2.0, ln_u));
  // angle 2 pi u2 = (q + f) pi / 2 with q the quadrant and f in [0, 1)
  const double t4 = __dmul_rn((double)k2, 1.0 / 1073741824.0);
  const int q = (int)t4;
  const double x = __dmul_rn(__dadd_rn(t4, -(double)q), k.half_pi);
  const double x2 = __dmul_rn(x, x);
  double sp = k.sin_c[10], cp = k.cos_c[11];
#pragma unroll
  for (int j = 9; j >= 0; --j) sp = __dadd_rn(__dmul_rn(sp, x2), k.sin_c[j]);
#pragma unroll
  for (int j = 10; j >= 0; --j) cp = __dadd_rn(__dmul_rn(cp, x2), k.cos_c[j]);
  const double sn = __dmul_rn(x, sp), cs = cp;
  double c, sgn;
  if ((i & 1) == 0) {   // cosine of the whole angle
    c = (q & 1) ? sn : cs;
    sgn = (q == 1 || q == 2) ? -1.0 : 1.0;
  } else {              // sine of the whole angle
    c = (q & 1) ? cs : sn;
    sgn = (q >= 2) ? -1.0 : 1.0;
  }
  return __dmul_rn(r, __dmul_rn(sgn, c));
}

template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// out[i] = T(float(z_i) * scale + shift), product and sum rounded to 32-bit one after the other
template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, uint64_t key, float scale, float shift,
                                     const RandomConsts k) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float z = __double2float_rn(normal_of(key, (uint64_t)i, k));
    out[i] = cast_out<T>(__fadd_rn(__fmul_rn(z, scale), shift));
  }
}

__global__ void random_int_kernel(int* __restrict__ out, long long n, uint64_t key, int modulus) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = (int)((mix64(key + ((uint64_t)i + 1) * 0x9E3779B97F4A7C15ull) >> 32) % (uint32_t)modulus);
}

// kind: 0 = 32-bit floats, 1 = bfloat16, 2 = int32 in [0, modulus).  Returns 0 or a CUDA error.
extern "C" int tl_random_fill(void* out, long long n, unsigned long long key, int kind, float scale, float shift,
                              int modulus, const RandomConsts* consts, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (kind < 0 || kind > 2 || (kind < 2 && consts == nullptr) || (kind == 2 && modulus <= 0)) return -1;
  const long long want = (n + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (kind == 0)
    random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, key, scale, shift, *consts);
  else if (kind == 1)
    random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, scale, shift, *consts);
  else
    random_int_kernel<<<blocks, 256, 0, stream>>>((int*)out, n, key, modulus);
  return (int)cudaGetLastError();
}
