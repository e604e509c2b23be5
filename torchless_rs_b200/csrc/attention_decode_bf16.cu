// Decode attention of the bfloat16 path: one new token per sequence against the
// paged cache, split over the keys so that a single long sequence fills the GPU.
//
// Compiled once per head size (-DHEAD_DIM=32|64|128).  Grid (splits, kv heads,
// sequences), four warps per block.  A warp takes 32 keys at a time and needs no
// shared memory in its loop: fragments of K and of the transposed V pages are loaded
// from global memory with 16-byte loads straight into the register layout of
// mma.m16n8k16.  That works because a dot product does not care about the order of
// its terms: the 16 contraction slots of an instruction are mapped to whatever 16
// dimensions (for q.k) or keys (for p.v) the 16-byte loads happen to deliver, the same
// way for both operands.  The query heads of one key/value head (up to 16) are the
// rows of the instruction.  Scores, maxima and sums are 32-bit; p is rounded to
// bfloat16 for the second product.
//
// Each block writes an unnormalised partial result with its maximum and sum; a second
// kernel merges the splits.  Math as in the reference (src/model/modules/attention.rs:
// 88-121) with the window of src/model/models/gpt_oss.rs:168-176.
#include "attention_bf16_common.cuh"

#define WARPS 4

// partial results: [seq][head][split][HEAD_DIM + 2] floats (values, then max and sum)
#define PART_STRIDE (HEAD_DIM + 2)

template <bool HI>  // HI: more than 8 query heads per kv head, rows 8..15 are in use
__global__ void __launch_bounds__(WARPS * 32, 2)
FN(attn_decode_kernel)(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                       const __nv_bfloat16* __restrict__ v_pages, float* __restrict__ part,
                       const int* __restrict__ seq_len, const int* __restrict__ seq_slot,
                       const int* __restrict__ page_table, int table_stride, int nh, int nkv,
                       int window, float scale_log2, int n_splits) {
  __shared__ float sm_o[WARPS][HI ? 16 : 8][HEAD_DIM];
  __shared__ float sm_m[WARPS][16], sm_l[WARPS][16];
  pdl_wait();
  pdl_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = nh / nkv;
  const int len = seq_len[b];
  const int lo = (window > 0 && len - window > 0) ? len - window : 0;
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;
  const int g0 = lo / GROUP, g1 = (len - 1) / GROUP;
  const int per = (g1 - g0 + 1 + n_splits - 1) / n_splits;
  const int gs = g0 + split * per;
  const int ge = min(gs + per, g1 + 1);

  // query fragments: rows are the query heads of this kv head
  uint32_t qa[NCHUNK][4], qb[NCHUNK][4];  // rows g and g + 8
  {
    const __nv_bfloat16* qrow = q + (size_t)b * nh * HEAD_DIM + (size_t)(kvh * G) * HEAD_DIM;
#pragma unroll
    for (int j = 0; j < NCHUNK; ++j) {
      uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
      if (g < G) va = ldg16(qrow + (size_t)g * HEAD_DIM + (4 * j + t) * 8);
      if (HI && g + 8 < G) vb = ldg16(qrow + (size_t)(g + 8) * HEAD_DIM + (4 * j + t) * 8);
      qa[j][0] = va.x; qa[j][1] = va.y; qa[j][2] = va.z; qa[j][3] = va.w;
      qb[j][0] = vb.x; qb[j][1] = vb.y; qb[j][2] = vb.z; qb[j][3] = vb.w;
    }
  }

  float o[NDT][4];
#pragma unroll
  for (int i = 0; i < NDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // rows g and g + 8

  for (int grp = gs + warp; grp < ge; grp += WARPS) {
    const int base = grp * GROUP;
    const int page = table[base / PAGE];
    const size_t pbase = ((size_t)page * nkv + kvh) * (size_t)(PAGE * HEAD_DIM);
    const int in_page = base % PAGE;
    // ---- scores: 4 tiles of 8 keys; column g of tile jt is key 8*(g>>1) + 2*jt + (g&1)
    float s[4][4];
#pragma unroll
    for (int jt = 0; jt < 4; ++jt) {
      s[jt][0] = s[jt][1] = s[jt][2] = s[jt][3] = 0.0f;
      const int kl = 8 * (g >> 1) + 2 * jt + (g & 1);
      const __nv_bfloat16* krow = k_pages + pbase + (size_t)(in_page + kl) * HEAD_DIM;
#pragma unroll
      for (int j = 0; j < NCHUNK; ++j) {
        const uint4 kv = ldg16(krow + (4 * j + t) * 8);
        uint32_t a[4];
        a[0] = qa[j][0]; a[1] = qb[j][0]; a[2] = qa[j][1]; a[3] = qb[j][1];
        mma_bf16(s[jt], a, kv.x, kv.y);
        a[0] = qa[j][2]; a[1] = qb[j][2]; a[2] = qa[j][3]; a[3] = qb[j][3];
        mma_bf16(s[jt], a, kv.z, kv.w);
      }
    }
    // ---- mask, running maximum, probabilities.  Column 2t+e of tile jt is key 8t + 2jt + e.
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int jt = 0; jt < 4; ++jt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = base + 8 * t + 2 * jt + e;
        const bool ok = idx >= lo && idx < len;
        s[jt][e] = ok ? s[jt][e] * scale_log2 : -INFINITY;
        s[jt][2 + e] = ok ? s[jt][2 + e] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[jt][e]);
        mx1 = fmaxf(mx1, s[jt][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    // a group always holds a visible key, so n0 is finite; rows 8..15 may be padding
    const float al0 = exp2f(m0 - n0);
    const float al1 = HI ? exp2f(m1 - n1) : 0.0f;
    m0 = n0; m1 = n1;
    uint32_t pa[2][4];  // A fragments of p for the two 16-key halves
    float r0 = 0.0f, r1 = 0.0f;
#pragma unroll
    for (int jt = 0; jt < 4; ++jt) {
      const float p0 = exp2f(s[jt][0] - n0), p1 = exp2f(s[jt][1] - n0);
      const float p2 = HI ? exp2f(s[jt][2] - n1) : 0.0f, p3 = HI ? exp2f(s[jt][3] - n1) : 0.0f;
      r0 += p0 + p1;
      r1 += p2 + p3;
      pa[jt >> 1][(jt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[jt >> 1][(jt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l0 = l0 * al0 + r0;
    l1 = l1 * al1 + r1;
    // ---- o = o * alpha + p . v; thread (g, t) loads v^T[dim 8i + g][keys 8t .. 8t+7]
    const __nv_bfloat16* vbase = v_pages + pbase + in_page + 8 * t;
#pragma unroll
    for (int i = 0; i < NDT; ++i) {
      const uint4 vv = ldg16(vbase + (size_t)(8 * i + g) * PAGE);
      o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1;
      mma_bf16(o[i], pa[0], vv.x, vv.y);
      mma_bf16(o[i], pa[1], vv.z, vv.w);
    }
  }

  // ---- merge the four warps of the block
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (t == 0) {
    sm_m[warp][g] = m0; sm_l[warp][g] = l0;
    sm_m[warp][g + 8] = m1; sm_l[warp][g + 8] = l1;
  }
#pragma unroll
  for (int i = 0; i < NDT; ++i) {
    sm_o[warp][g][8 * i + 2 * t] = o[i][0];
    sm_o[warp][g][8 * i + 2 * t + 1] = o[i][1];
    if (HI) {
      sm_o[warp][g + 8][8 * i + 2 * t] = o[i][2];
      sm_o[warp][g + 8][8 * i + 2 * t + 1] = o[i][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HEAD_DIM; idx += WARPS * 32) {
    const int r = idx / HEAD_DIM, d = idx - r * HEAD_DIM;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_m[w][r]);
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float wm = sm_m[w][r];
      const float f = wm == -INFINITY ? 0.0f : exp2f(wm - m);
      acc += f * sm_o[w][r][d];
      l += f * sm_l[w][r];
    }
    float* dst = part + (((size_t)b * nh + kvh * G + r) * n_splits + split) * PART_STRIDE;
    dst[d] = acc;
    if (d == 0) { dst[HEAD_DIM] = m; dst[HEAD_DIM + 1] = l; }
  }
}

// Merges the splits of one (sequence, head) and writes the normalised result.
__global__ void __launch_bounds__(HEAD_DIM)
FN(attn_decode_combine_kernel)(const float* __restrict__ part, __nv_bfloat16* __restrict__ out,
                               int nh, int n_splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* src = part + ((size_t)b * nh + h) * n_splits * PART_STRIDE;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[s * PART_STRIDE + HEAD_DIM]);
  float acc = 0.0f, l = 0.0f;
  for (int s = 0; s < n_splits; ++s) {
    const float sm = src[s * PART_STRIDE + HEAD_DIM];
    const float f = sm == -INFINITY ? 0.0f : exp2f(sm - m);
    acc += f * src[s * PART_STRIDE + d];
    l += f * src[s * PART_STRIDE + HEAD_DIM + 1];
  }
  out[((size_t)b * nh + h) * HEAD_DIM + d] = __float2bfloat16_rn(acc / l);
}

// Floats of scratch that `part` must hold.
extern "C" long long FN(tl_attn_decode_scratch_floats)(int B, int nh, int n_splits) {
  return (long long)B * nh * n_splits * PART_STRIDE;
}

// q [B, nh*HEAD_DIM] (row b is the new token of sequence b), out likewise;
// seq_len[b] counts the new token.  Returns -2 for sizes this kernel does not take.
extern "C" int FN(tl_attn_decode)(const void* q, const void* k_pages, const void* v_pages,
                                  void* out, float* part, const int* seq_len,
                                  const int* seq_slot, const int* page_table, int table_stride,
                                  int B, int nh, int nkv, int window, float scale, int n_splits,
                                  cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || n_splits < 1 || n_splits > 65535 ||
      nkv > 65535 || B > 65535)
    return -2;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_splits, nkv, B);
  int st;
  if (nh / nkv > 8)
    st = tl_launch(FN(attn_decode_kernel)<true>, grid, dim3(WARPS * 32), 0, stream,
                   (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                   part, seq_len, seq_slot, page_table, table_stride, nh, nkv, window, scale_log2, n_splits);
  else
    st = tl_launch(FN(attn_decode_kernel)<false>, grid, dim3(WARPS * 32), 0, stream,
                   (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                   part, seq_len, seq_slot, page_table, table_stride, nh, nkv, window, scale_log2, n_splits);
  if (st) return st;
  return tl_launch(FN(attn_decode_combine_kernel), dim3(nh, B), dim3(HEAD_DIM), 0, stream,
                   (const float*)part, (__nv_bfloat16*)out, nh, n_splits);
}
