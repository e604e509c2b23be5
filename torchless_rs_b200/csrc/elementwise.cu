// Memory-bound parts of the step: embedding gather, RMSNorm, rotation + cache
// write, SiLU-gate.  The residual stream is always 32-bit; `act_t` is the type
// of what feeds the matrix products and of the cache.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[t, :] = table[tokens[t], :], no scaling
// (reference: src/model/modules/embedding.rs:15-21).
// ---------------------------------------------------------------------------
// A token may also be taken from a device buffer (the tokens that the previous step selected):
// with `token_src` given, token t is token_src[token_from[t]] wherever token_from[t] >= 0.
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ token_from,
                             const int* __restrict__ token_src, const act_t* __restrict__ table,
                             float* __restrict__ x, int H, int vocab) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (token_src != nullptr && token_from[t] >= 0) tok = token_src[token_from[t]];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // the host has checked the range already
  const act_t* src = table + (size_t)tok * H;
  float* dst = x + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32(src[i]);
}

extern "C" int TL_NAME(tl_embed)(const int* tokens, const int* token_from, const int* token_src,
                                 const void* table, float* x, int T, int H, int vocab,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  return tl_launch(embed_kernel, dim3(T), dim3(256), 0, stream, tokens, token_from, token_src,
                   (const act_t*)table, x, H, vocab);
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

extern "C" int TL_NAME(tl_rmsnorm)(const float* x, const int* rows, const void* w, int w_is_f32,
                                   void* y, int n_rows, int H, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
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

extern "C" int TL_NAME(tl_rope_cache_write)(const float* qkv, int ld, void* q_out, void* k_pages,
                                            void* v_pages, const int* token_pos,
                                            const int* token_seq, const int* seq_slot,
                                            const int* page_table, int table_stride,
                                            const float* inv_freq, int style, int T, int nh,
                                            int nkv, int hd, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hd & 1) || hd > 256) return TL_ERR_BAD_ARG;
  const int heads = nh + (k_pages ? 2 * nkv : 0);
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
