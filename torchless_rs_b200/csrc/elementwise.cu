// Memory-bound parts of the step: embedding gather, RMSNorm, rotation + cache
// write, SiLU-gate.  The residual stream is always 32-bit; `act_t` is the type
// of what feeds the matrix products and of the cache.
#include "common.cuh"

#include <cuda_fp16.h>

// ---------------------------------------------------------------------------
// Embedding: x[t, :] = table[tokens[t], :]; the reference's Mistral does no more
// (src/model/modules/embedding.rs:15-21).  Two things other arrangements put between the
// table and the first layer are taken here, since this kernel writes the stream anyway:
// a multiplier (`scale`, 1 = none) and a learned row per position (`pos_table`
// [max_pos, H] with `token_pos`, null = none): x[t, :] = scale * table[tok, :] +
// pos_table[token_pos[t], :], in 32-bit.
// ---------------------------------------------------------------------------
// A token may also be taken from a device buffer (the tokens that the previous step selected):
// with `token_src` given, token t is token_src[token_from[t]] wherever token_from[t] >= 0.
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ token_from,
                             const int* __restrict__ token_src, const act_t* __restrict__ table,
                             float* __restrict__ x, int H, int vocab, float scale,
                             const act_t* __restrict__ pos_table, const int* __restrict__ token_pos,
                             int max_pos) {
  TL_TRACE_SCOPE(1, H, 1);
  pdl_wait();
  TL_TRACE_RELEASED();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (token_src != nullptr && token_from[t] >= 0) tok = token_src[token_from[t]];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // the host has checked the range already
  const act_t* src = table + (size_t)tok * H;
  float* dst = x + (size_t)t * H;
  if (pos_table == nullptr) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = scale * to_f32(src[i]);
  } else {
    int p = token_pos[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);   // the host refuses longer sequences
    const act_t* pr = pos_table + (size_t)p * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = fmaf(scale, to_f32(src[i]), to_f32(pr[i]));
  }
}

extern "C" int TL_NAME(tl_embed)(const int* tokens, const int* token_from, const int* token_src,
                                 const void* table, float* x, int T, int H, int vocab, float scale,
                                 const void* pos_table, const int* token_pos, int max_pos,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (pos_table != nullptr && (token_pos == nullptr || max_pos <= 0)) return TL_ERR_BAD_ARG;
  return tl_launch(embed_kernel, dim3(T), dim3(256), 0, stream, tokens, token_from, token_src,
                   (const act_t*)table, x, H, vocab, scale, (const act_t*)pos_table, token_pos, max_pos);
}

// ---------------------------------------------------------------------------
// Soft cap of the logits, in place: v <- cap * tanh(v / cap).  The reference's Mistral has
// none (src/model/mod.rs:439-446); the head of another arrangement may ask for it.
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ v, long long n, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  const float inv = 1.0f / cap;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}

extern "C" int TL_NAME(tl_softcap)(float* v, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.0f)) return TL_ERR_BAD_ARG;
  const long long blocks = (n + 255) / 256;
  return tl_launch(softcap_kernel, dim3((unsigned)(blocks < 2368 ? blocks : 2368)), dim3(256), 0, stream, v,
                   n, cap);
}

// ---------------------------------------------------------------------------
// RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, all in 32-bit, output rounded to
// act_t (reference: src/kernels/mod.rs:558-568).  `rows` (optional) picks the
// input rows, so the final norm runs on the wanted rows only.
// ---------------------------------------------------------------------------
#define NORM_MAX_PER_THREAD 16
template <typename W>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const W* __restrict__ w, act_t* __restrict__ y, int H, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
  act_t* yr = y + (size_t)r * H;
  // the row is read once and kept in registers if it fits, else read a second time
  const bool fits = H <= (int)blockDim.x * NORM_MAX_PER_THREAD;
  float keep[NORM_MAX_PER_THREAD];
  float ss = 0.0f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < NORM_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      keep[j] = i < H ? xr[i] : 0.0f;
      ss = fmaf(keep[j], keep[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = xr[i];
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  if (fits) {
#pragma unroll
    for (int j = 0; j < NORM_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < H) yr[i] = from_f32<act_t>((keep[j] / rms) * to_f32(w[i]));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      yr[i] = from_f32<act_t>((xr[i] / rms) * to_f32(w[i]));
  }
}

// Four values at a time: 16-byte loads of the row, 8- or 16-byte stores of the result.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// The same norm for rows of H = 4n values that fit the block's registers (H <= 16 per thread).
template <typename W>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   const W* __restrict__ w, act_t* __restrict__ y, int H, float eps) {
  TL_TRACE_SCOPE(2, H, 2);
  __shared__ float scratch[33];
  pdl_wait();
  TL_TRACE_RELEASED();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
  act_t* yr = y + (size_t)r * H;
  float keep[4][4];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    if (i < H) load4(xr + i, keep[j]);
    else keep[j][0] = keep[j][1] = keep[j][2] = keep[j][3] = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) ss = fmaf(keep[j][e], keep[j][e], ss);
  }
  // the weights do not depend on the sum: fetched before the block waits for it
  float wv[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    if (i < H) load4(w + i, wv[j]);
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#if TL_DTYPE == 0
  // the 32-bit path keeps the reference's order: divide, then multiply (src/kernels/mod.rs:558-568)
#define NORM_SCALE(v) ((v) / rms)
#else
  // rounded to bfloat16 afterwards: one division per row and a multiplication per value
  const float rinv = 1.0f / rms;
#define NORM_SCALE(v) ((v) * rinv)
#endif
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    if (i < H) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = NORM_SCALE(keep[j][e]) * wv[j][e];
      store4(yr + i, o);
    }
  }
#undef NORM_SCALE
}

extern "C" int TL_NAME(tl_rmsnorm)(const float* x, const int* rows, const void* w, int w_is_f32,
                                   void* y, int n_rows, int H, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H % 4 == 0 && H <= 16384 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0) {
    const int vthreads = H <= 2048 ? 128 : H <= 4096 ? 256 : H <= 8192 ? 512 : 1024;
    if (w_is_f32)
      return tl_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(vthreads), 0, stream, x, rows,
                       (const float*)w, (act_t*)y, H, eps);
    return tl_launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vthreads), 0, stream, x,
                     rows, (const __nv_bfloat16*)w, (act_t*)y, H, eps);
  }
  const int threads = H >= 2048 ? 512 : 256;
  if (w_is_f32)
    return tl_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows,
                     (const float*)w, (act_t*)y, H, eps);
  return tl_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, rows,
                   (const __nv_bfloat16*)w, (act_t*)y, H, eps);
}

// ---------------------------------------------------------------------------
// Rotation of q and k at each token's own position and the write of k and v into
// the token's cache page (reference: rotation src/kernels/mod.rs:572-608, cache
// write src/model/kv_cache.rs:87-104; v is not rotated).
//   qkv      [T, ld] 32-bit: nh*hd columns of q, then nkv*hd of k, then nkv*hd of v
//   q_out    [T, nh*hd]
//   k_pages  [n_pages, nkv, TL_PAGE, hd]; v_pages  [n_pages, nkv, hd, TL_PAGE] (values are
//            kept transposed, so that the attention kernels read runs of positions of
//            one dimension); both null when the layer keeps no cache
//   inv_freq [hd/2] 32-bit, null for no rotation
//   style 0: dimension i pairs with i + hd/2;  style 1: 2i pairs with 2i+1
// The angle pos * inv_freq and its sine and cosine are computed in 32-bit.
// ---------------------------------------------------------------------------
__global__ void rope_cache_write_kernel(const float* __restrict__ qkv, int ld,
                                        act_t* __restrict__ q_out, act_t* __restrict__ k_pages,
                                        act_t* __restrict__ v_pages,
                                        const int* __restrict__ token_pos,
                                        const int* __restrict__ token_seq,
                                        const int* __restrict__ seq_slot,
                                        const int* __restrict__ page_table, int table_stride,
                                        const float* __restrict__ inv_freq, int style, int nh,
                                        int nkv, int hd, int heads_per_block) {
  // grid (tokens, groups of heads); heads count query heads, then key heads, then value heads.
  // A warp takes every fourth head of its group, so that sine and cosine of a (position, i)
  // are computed once per warp and used for all its heads.
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const int half = hd >> 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int total_heads = nh + (k_pages ? 2 * nkv : 0);
  const int h_begin = blockIdx.y * heads_per_block;
  const int h_end = min(h_begin + heads_per_block, total_heads);
  int page = -1;
  if (k_pages) page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
  const float fpos = (float)pos;
  // up to 256 / 2 / 32 = 4 rotation pairs per lane
  float cs[4], sn[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    cs[j] = 1.0f; sn[j] = 0.0f;
    if (inv_freq && i < half) sincosf(fpos * inv_freq[i], &sn[j], &cs[j]);
  }
  for (int h = h_begin + warp; h < h_end; h += n_warps) {
    const float* row = qkv + (size_t)t * ld + (size_t)h * hd;
    if (h >= nh && page < 0) continue;
    const int kvh = h < nh ? 0 : (h - nh < nkv ? h - nh : h - nh - nkv);
    const size_t page_base = ((size_t)(page < 0 ? 0 : page) * nkv + kvh) * (size_t)(TL_PAGE * hd);
    if (h < nh + nkv) {
      act_t* dst = h < nh ? q_out + (size_t)t * nh * hd + (size_t)h * hd
                          : k_pages + page_base + (size_t)(pos % TL_PAGE) * hd;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        if (i >= half) break;
        const int d0 = style == 0 ? i : 2 * i;
        const int d1 = style == 0 ? i + half : 2 * i + 1;
        const float a = row[d0], b = row[d1];
        dst[d0] = from_f32<act_t>(a * cs[j] - b * sn[j]);
        dst[d1] = from_f32<act_t>(a * sn[j] + b * cs[j]);
      }
    } else {
      // values lie transposed in a page: [hd][TL_PAGE]
      act_t* dst = v_pages + page_base + (pos % TL_PAGE);
      for (int d = lane; d < hd; d += 32) dst[(size_t)d * TL_PAGE] = from_f32<act_t>(row[d]);
    }
  }
}

// The same for steps of many tokens, half-split pairs (style 0) and head sizes of 32, 64,
// 128 or 256.  Two kinds of block in one launch:
//  - blockIdx.y < rot_groups: one token; its query and key heads are rotated four pairs per
//    lane with 16-byte loads, hd/8 lanes per head and 256/hd heads per warp at a time;
//  - blockIdx.y == rot_groups: 32 consecutive tokens of one value head; the tile is turned
//    in shared memory, so that the transposed value pages are written in runs of positions.
__global__ void __launch_bounds__(128)
rope_cache_write_vec_kernel(const float* __restrict__ qkv, int ld, act_t* __restrict__ q_out,
                            act_t* __restrict__ k_pages, act_t* __restrict__ v_pages,
                            const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                            const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                            int table_stride, const float* __restrict__ inv_freq, int T, int nh,
                            int nkv, int hd, int rot_groups) {
  extern __shared__ float vt[];   // [32 tokens][hd + 1]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((int)blockIdx.y == rot_groups) {
    const int tiles_t = (T + 31) / 32;
    for (int tile = blockIdx.x; tile < tiles_t * nkv; tile += gridDim.x) {
      const int t0 = (tile / nkv) * 32, kvh = tile % nkv;
      const int nt = min(32, T - t0);
      const int vec_per_row = hd >> 2;
      for (int idx = threadIdx.x; idx < nt * vec_per_row; idx += blockDim.x) {
        const int tt = idx / vec_per_row, d = (idx % vec_per_row) * 4;
        float v[4];
        load4(qkv + (size_t)(t0 + tt) * ld + (size_t)(nh + nkv + kvh) * hd + d, v);
        float* dst = vt + tt * (hd + 1) + d;
        dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; dst[3] = v[3];
      }
      __syncthreads();
      if (lane < nt) {
        const int t = t0 + lane;
        const int pos = token_pos[t];
        const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
        act_t* dst = v_pages + ((size_t)page * nkv + kvh) * (size_t)(TL_PAGE * hd) + (pos % TL_PAGE);
        for (int d = warp; d < hd; d += 4) dst[(size_t)d * TL_PAGE] = from_f32<act_t>(vt[lane * (hd + 1) + d]);
      }
      __syncthreads();
    }
    return;
  }
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const int half = hd >> 1;
  const int lph = hd >> 3;            // lanes per head
  const int hpp = 32 / lph;           // heads per warp pass
  const int sub = lane / lph, i0 = (lane % lph) * 4;
  const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
  // cosine and sine of the token's angles: each once per block (a thread per pair of dimensions),
  // then read by every lane that turns that pair; the full-precision sine is most of this
  // kernel's arithmetic otherwise
  float2* cs_s = reinterpret_cast<float2*>(vt);   // [hd / 2]; the value blocks use `vt` otherwise
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s_ = 0.0f, c_ = 1.0f;
    if (inv_freq) sincosf((float)pos * inv_freq[i], &s_, &c_);
    cs_s[i] = make_float2(c_, s_);
  }
  __syncthreads();
  float cs[4], sn[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) { cs[j] = cs_s[i0 + j].x; sn[j] = cs_s[i0 + j].y; }
  const int rot_heads = nh + nkv;
  const int passes = (rot_heads + hpp - 1) / hpp;
  const int per_group = (passes + rot_groups - 1) / rot_groups;
  const int p_end = min(((int)blockIdx.y + 1) * per_group, passes);
#pragma unroll 2
  for (int p = (int)blockIdx.y * per_group + warp; p < p_end; p += 4) {
    const int h = p * hpp + sub;
    if (h >= rot_heads) continue;
    const float* row = qkv + (size_t)t * ld + (size_t)h * hd;
    act_t* dst = h < nh ? q_out + ((size_t)t * nh + h) * hd
                        : k_pages + ((size_t)page * nkv + (h - nh)) * (size_t)(TL_PAGE * hd) +
                              (size_t)(pos % TL_PAGE) * hd;
    float a[4], b[4], lo[4], hi[4];
    load4(row + i0, a);
    load4(row + half + i0, b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo[j] = a[j] * cs[j] - b[j] * sn[j];
      hi[j] = a[j] * sn[j] + b[j] * cs[j];
    }
    store4(dst + i0, lo);
    store4(dst + half + i0, hi);
  }
}

extern "C" int TL_NAME(tl_rope_cache_write)(const float* qkv, int ld, void* q_out, void* k_pages,
                                            void* v_pages, const int* token_pos,
                                            const int* token_seq, const int* seq_slot,
                                            const int* page_table, int table_stride,
                                            const float* inv_freq, int style, int T, int nh,
                                            int nkv, int hd, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hd & 1) || hd > 256) return TL_ERR_BAD_ARG;
  const int heads = nh + (k_pages ? 2 * nkv : 0);
  if (T >= 256 && style == 0 && k_pages && v_pages && (hd == 32 || hd == 64 || hd == 128 || hd == 256) &&
      ld % 4 == 0 && ((uintptr_t)qkv & 15) == 0 && nkv <= 65535) {
    const int passes = (nh + nkv + 256 / hd - 1) / (256 / hd);
    int rot_groups = (passes + 7) / 8;   // at most two passes for each of a block's four warps
    if (rot_groups > 65534) return TL_ERR_UNSUPPORTED;
    dim3 grid(T, rot_groups + 1);
    return tl_launch(rope_cache_write_vec_kernel, grid, dim3(128), (size_t)32 * (hd + 1) * sizeof(float),
                     stream, qkv, ld, (act_t*)q_out, (act_t*)k_pages, (act_t*)v_pages, token_pos,
                     token_seq, seq_slot, page_table, table_stride, inv_freq, T, nh, nkv, hd, rot_groups);
  }
  // few tokens: one warp per (token, head), for parallelism; many tokens: one block per token
  const int per_block = T >= 256 ? heads : 1;
  const int groups = (heads + per_block - 1) / per_block;
  if (groups > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid(T, groups);
  return tl_launch(rope_cache_write_kernel, grid, dim3(T >= 256 ? 128 : 32), 0, stream, qkv, ld, (act_t*)q_out,
                   (act_t*)k_pages, (act_t*)v_pages, token_pos, token_seq, seq_slot, page_table,
                   table_stride, inv_freq, style, nh, nkv, hd, per_block);
}

// ---------------------------------------------------------------------------
// SiLU-gate on an unfused gate/up product: out[t, j] = silu(gu[t, j]) * gu[t, I + j]
// with silu(z) = z / (1 + exp(-z)) (reference: src/kernels/mod.rs:546-548,
// src/model/modules/mlp.rs:34-40).
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const float* __restrict__ gu, act_t* __restrict__ out, int I,
                                size_t total) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int j = (int)(idx - t * I);
    const float g = gu[t * 2 * I + j], u = gu[t * 2 * I + I + j];
    out[idx] = from_f32<act_t>((g / (1.0f + expf(-g))) * u);
  }
}

extern "C" int TL_NAME(tl_silu_mul)(const float* gu, void* out, int T, int I, cudaStream_t stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(silu_mul_kernel, dim3(blocks), dim3(256), 0, stream, gu, (act_t*)out, I, total);
}

// ---------------------------------------------------------------------------
// Weights on their way in: a stored tensor (32-bit, float16 or bfloat16, already on the device as
// stored) becomes the activation type at its place in a matrix of the model, so that stacked
// matrices (q/k/v; gate and up) are filled row block by row block without a joined copy.
// bfloat16 to 32-bit and float16 to 32-bit are exact (the reference widens the same way,
// src/loader/formats/safetensors.rs:367-390); to bfloat16 rounds to nearest even.
// ---------------------------------------------------------------------------
template <typename S> __device__ __forceinline__ float widen(S v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }

template <typename S>
__global__ void convert_kernel(const S* __restrict__ src, act_t* __restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<act_t>(widen<S>(src[i]));
}

// src_kind: 0 = 32-bit floats, 1 = bfloat16, 2 = float16.  Returns 0, a CUDA error or TL_ERR_BAD_ARG.
extern "C" int TL_NAME(tl_convert)(const void* src, int src_kind, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 32 ? want : 148 * 32);
  if (src_kind == 0) convert_kernel<float><<<blocks, 256, 0, stream>>>((const float*)src, (act_t*)dst, (size_t)n);
  else if (src_kind == 1) convert_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (act_t*)dst, (size_t)n);
  else if (src_kind == 2) convert_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)src, (act_t*)dst, (size_t)n);
  else return TL_ERR_BAD_ARG;
  return TL_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// The per-sequence state of a running batch on the device: each row's position and length go up
// by one.  When a decode step has the same sequences in the same rows as the step before and its
// tokens come from the device (the tokens the sampler selected), nothing that the kernels read
// has changed but these two arrays, so the engine advances them here instead of laying the step
// out on the host and copying it over.  (The reference's state is one counter that its caller
// increments after each forward pass, src/model/mod.rs:93, src/main.rs:562.)
// ---------------------------------------------------------------------------
__global__ void advance_step_kernel(int* __restrict__ token_pos, int* __restrict__ seq_len, int n) {
  pdl_wait();   // the step before still reads both arrays
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { token_pos[i] += 1; seq_len[i] += 1; }
}

extern "C" int TL_NAME(tl_advance_step)(int* token_pos, int* seq_len, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  return tl_launch(advance_step_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, token_pos, seq_len, n);
}

// ---------------------------------------------------------------------------
// A decode step of some of the rows of the decode step before, in any order (sequences have ended,
// or the rows take their tokens from other places of the sampler's output): the new step's arrays
// are made here from the old ones, each kept row's position and length one higher.  `base` is the
// buffer that holds both layouts (they overlap), so one block reads all it needs before any thread
// writes.  off[]: where the eight arrays of the new layout start in `base`, in the order tokens,
// token_seq, token_pos, seq_slot, seq_start, seq_len, want_rows, token_from.
// ---------------------------------------------------------------------------
#define REGROUP_MAX_ROWS 256
struct RegroupRows { unsigned short keep[REGROUP_MAX_ROWS]; unsigned short from[REGROUP_MAX_ROWS]; };
struct RegroupOffsets { int off[8]; };

__global__ void __launch_bounds__(REGROUP_MAX_ROWS)
regroup_step_kernel(const int* old_pos, const int* old_len, const int* old_slot, int* base,
                    const RegroupOffsets o, int n, const __grid_constant__ RegroupRows rows) {
  pdl_wait();   // the step before still reads the old arrays
  pdl_launch_dependents();
  const int j = threadIdx.x;
  int pos = 0, len = 0, slot = 0;
  if (j < n) {
    const int r = rows.keep[j];
    pos = old_pos[r];
    len = old_len[r];
    slot = old_slot[r];
  }
  __syncthreads();
  if (j < n) {
    base[o.off[0] + j] = 0;
    base[o.off[1] + j] = j;
    base[o.off[2] + j] = pos + 1;
    base[o.off[3] + j] = slot;
    base[o.off[4] + j] = j;
    base[o.off[5] + j] = len + 1;
    base[o.off[6] + j] = j;
    base[o.off[7] + j] = rows.from[j];
  }
  if (j == 0) base[o.off[4] + n] = n;
}

extern "C" int TL_NAME(tl_regroup_step)(const int* old_pos, const int* old_len, const int* old_slot, int* base,
                                        const int* offsets, int n, const unsigned short* keep,
                                        const unsigned short* from, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > REGROUP_MAX_ROWS) return -2;
  RegroupRows rows;
  RegroupOffsets o;
  for (int i = 0; i < n; ++i) { rows.keep[i] = keep[i]; rows.from[i] = from[i]; }
  for (int i = n; i < REGROUP_MAX_ROWS; ++i) rows.keep[i] = rows.from[i] = 0;
  for (int i = 0; i < 8; ++i) o.off[i] = offsets[i];
  return tl_launch(regroup_step_kernel, dim3(1), dim3(REGROUP_MAX_ROWS), 0, stream, old_pos, old_len, old_slot,
                   base, o, n, rows);
}

TL_TRACE_EXPORT(elementwise)
