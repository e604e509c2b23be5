// Prefill attention of the bfloat16 path: the new tokens of every sequence of a step
// against the paged cache (which already holds their own keys and values), causal,
// with an optional window, grouped-query.
//
// Compiled once per head size.  Grid (query tiles of 64, heads, sequences); each of the
// four warps of a block owns 16 consecutive queries and walks its own range of keys, 32
// at a time, with a running maximum and sum in 32-bit (the recurrence of the reference's
// tiled attention helper, src/model/modules/flash_attention.rs:101-136; scores and mask
// as src/model/modules/attention.rs:88-121 and src/model/models/gpt_oss.rs:168-176).
// As in the decode kernel, fragments of K and of the transposed V pages go from global
// memory straight into the register layout of mma.m16n8k16; warps of a block and the
// heads of a group meet the same keys at nearly the same time, so these loads are
// served by L1 and L2.
#include "attention_bf16_common.cuh"

#define PF_WARPS 4
#define PF_TILE (PF_WARPS * 16)

__global__ void __launch_bounds__(PF_WARPS * 32, 2)
FN(attn_prefill_kernel)(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_len,
                        const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                        int table_stride, int nh, int nkv, int window, float scale_log2) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tok0 = seq_start[b];
  const int n_new = seq_start[b + 1] - tok0;
  const int r0 = blockIdx.x * PF_TILE + warp * 16;   // first query of this warp within the new tokens
  if (r0 >= n_new) return;
  const int len = seq_len[b];
  const int past = len - n_new;
  const int kvh = h / (nh / nkv);
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;

  // rows g and g + 8 of the warp's 16 queries; rows past the end repeat the last one
  const int ra = min(r0 + g, n_new - 1), rb = min(r0 + g + 8, n_new - 1);
  const int pa_pos = past + ra, pb_pos = past + rb;     // positions of the two rows
  uint32_t qa[NCHUNK][4], qb[NCHUNK][4];
  {
    const __nv_bfloat16* qra = q + ((size_t)(tok0 + ra) * nh + h) * HEAD_DIM;
    const __nv_bfloat16* qrb = q + ((size_t)(tok0 + rb) * nh + h) * HEAD_DIM;
#pragma unroll
    for (int j = 0; j < NCHUNK; ++j) {
      const uint4 va = ldg16(qra + (4 * j + t) * 8), vb = ldg16(qrb + (4 * j + t) * 8);
      qa[j][0] = va.x; qa[j][1] = va.y; qa[j][2] = va.z; qa[j][3] = va.w;
      qb[j][0] = vb.x; qb[j][1] = vb.y; qb[j][2] = vb.z; qb[j][3] = vb.w;
    }
  }
  const int lo_a = (window > 0 && pa_pos - window + 1 > 0) ? pa_pos - window + 1 : 0;
  const int lo_b = (window > 0 && pb_pos - window + 1 > 0) ? pb_pos - window + 1 : 0;
  // keys this warp can see: from the first row's window start to the last row's position
  const int first_pos = past + r0, last_pos = past + min(r0 + 15, n_new - 1);
  const int lo_w = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
  const int g0 = lo_w / GROUP, g1 = last_pos / GROUP;

  float o[NDT][4];
#pragma unroll
  for (int i = 0; i < NDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

  for (int grp = g0; grp <= g1; ++grp) {
    const int base = grp * GROUP;
    const int page = table[base / PAGE];
    const size_t pbase = ((size_t)page * nkv + kvh) * (size_t)(PAGE * HEAD_DIM);
    const int in_page = base % PAGE;
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
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int jt = 0; jt < 4; ++jt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = base + 8 * t + 2 * jt + e;
        s[jt][e] = (idx >= lo_a && idx <= pa_pos) ? s[jt][e] * scale_log2 : -INFINITY;
        s[jt][2 + e] = (idx >= lo_b && idx <= pb_pos) ? s[jt][2 + e] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[jt][e]);
        mx1 = fmaxf(mx1, s[jt][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    // a row may see no key of this group (window or causal edge): keep its state unchanged
    const float ref0 = n0 == -INFINITY ? 0.0f : n0, ref1 = n1 == -INFINITY ? 0.0f : n1;
    const float al0 = exp2f(m0 - ref0), al1 = exp2f(m1 - ref1);
    m0 = n0; m1 = n1;
    uint32_t pa[2][4];
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int jt = 0; jt < 4; ++jt) {
      const float p0 = exp2f(s[jt][0] - ref0), p1 = exp2f(s[jt][1] - ref0);
      const float p2 = exp2f(s[jt][2] - ref1), p3 = exp2f(s[jt][3] - ref1);
      sum0 += p0 + p1;
      sum1 += p2 + p3;
      pa[jt >> 1][(jt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[jt >> 1][(jt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l0 = l0 * al0 + sum0;
    l1 = l1 * al1 + sum1;
    const __nv_bfloat16* vbase = v_pages + pbase + in_page + 8 * t;
#pragma unroll
    for (int i = 0; i < NDT; ++i) {
      const uint4 vv = ldg16(vbase + (size_t)(8 * i + g) * PAGE);
      o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1;
      mma_bf16(o[i], pa[0], vv.x, vv.y);
      mma_bf16(o[i], pa[1], vv.z, vv.w);
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
  const bool wa = r0 + g < n_new, wb = r0 + g + 8 < n_new;
  __nv_bfloat16* oa = out + ((size_t)(tok0 + ra) * nh + h) * HEAD_DIM;
  __nv_bfloat16* ob = out + ((size_t)(tok0 + rb) * nh + h) * HEAD_DIM;
#pragma unroll
  for (int i = 0; i < NDT; ++i) {
    if (wa) *reinterpret_cast<uint32_t*>(oa + 8 * i + 2 * t) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    if (wb) *reinterpret_cast<uint32_t*>(ob + 8 * i + 2 * t) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// q, out [T, nh*HEAD_DIM]; max_new = the most new tokens any sequence of the step has.
extern "C" int FN(tl_attn_prefill)(const void* q, const void* k_pages, const void* v_pages,
                                   void* out, const int* seq_start, const int* seq_len,
                                   const int* seq_slot, const int* page_table, int table_stride,
                                   int B, int max_new, int nh, int nkv, int window, float scale,
                                   cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh > 65535 || B > 65535) return -2;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((max_new + PF_TILE - 1) / PF_TILE, nh, B);
  return tl_launch(FN(attn_prefill_kernel), grid, dim3(PF_WARPS * 32), 0, stream,
                   (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                   (__nv_bfloat16*)out, seq_start, seq_len, seq_slot, page_table, table_stride, nh, nkv,
                   window, scale_log2);
}
