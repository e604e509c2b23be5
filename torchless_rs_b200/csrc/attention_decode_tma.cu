// Decode attention of the bfloat16 path with the cache pages brought in by TMA.
// (Reference: per head, scores of the cached keys times 1/sqrt(head_dim), softmax with the
// maximum subtracted, weighted sum of the cached values: src/model/modules/attention.rs:186-226.)
//
// Same arithmetic and the same partial results as attention_decode_bf16.cu (and the same
// second kernel merges the splits), but keys and values do not pass through registers on
// their way from HBM: a block walks over the pages of its share of a sequence, one
// thread requests each page's K slab [64 keys x HEAD_DIM] and transposed V slab
// [HEAD_DIM x 64 keys] of this kv head as 128-byte-swizzled tiles, three pages ahead of
// the four warps that consume them.  Each warp takes 16 keys of a page.  The fragments of
// mma.m16n8k16 are read from shared memory with the same freedom as before: contraction
// slots are mapped to whatever dimensions or keys a 16-byte (K) or 8-byte (V) read
// delivers, identically for both operands.  Head sizes 64 and 128.
//
// Every wait on an mbarrier is bounded; when a bound is hit the block records a code in
// tl_attn_tma_error and stops.
#include <cuda.h>
#include <stdlib.h>

#include "attention_bf16_common.cuh"

#include <map>
#include <mutex>
#include <tuple>

#define TD_WARPS 4
#define TD_STAGES 3
#define K_SUB (HEAD_DIM / 64)                       // 64-column boxes of a K slab
#define K_BYTES (PAGE * HEAD_DIM * 2)
#define V_BYTES (HEAD_DIM * PAGE * 2)
#define TD_STAGE_BYTES (K_BYTES + V_BYTES)
#define PART_STRIDE (HEAD_DIM + 2)

__device__ int tl_attn_tma_error = 0;

__device__ __forceinline__ uint32_t td_smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void td_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(td_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void td_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(td_smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void td_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(td_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool td_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                             int code) {
  return tl_mbar_wait(bar, parity, abort_flag, code, &tl_attn_tma_error);   // bounded_wait.cuh
}
__device__ __forceinline__ void td_tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                               int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      :
      : "r"(td_smem_u32(dst)), "l"(map), "r"(td_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

template <bool HI>
__global__ void __launch_bounds__(TD_WARPS * 32, 2)
FN(attn_decode_tma_kernel)(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                           const __nv_bfloat16* __restrict__ q, float* __restrict__ part,
                           __nv_bfloat16* __restrict__ out,
                           const int* __restrict__ seq_len, const int* __restrict__ seq_slot,
                           const int* __restrict__ page_table, int table_stride, int nh, int nkv,
                           int window, float scale_log2, int n_splits, int quantum) {
  TL_TRACE_SCOPE(4, n_splits, 4);
  extern __shared__ uint8_t td_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)td_smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + TD_STAGES * TD_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + TD_STAGES;
  volatile int* abort_flag = (volatile int*)(empty_bar + TD_STAGES);
  // the merge of the four warps reuses the first stage after the loop
  float* sm_o = (float*)smem;                                   // [warps][16][HEAD_DIM]
  float* sm_m = sm_o + TD_WARPS * 16 * HEAD_DIM;                // [warps][16]
  float* sm_l = sm_m + TD_WARPS * 16;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = nh / nkv;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TD_STAGES; ++s) { td_mbar_init(&full_bar[s], 1); td_mbar_init(&empty_bar[s], TD_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Lengths and page tables were copied to the device before the step's first kernel, and every
  // page but a sequence's last was filled by earlier steps: only the last page (it holds the
  // newest token's keys and values) and the queries come from the kernels just before this one.
  const int len = seq_len[b];
  const int lo = (window > 0 && len - window > 0) ? len - window : 0;
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;
  const int first_page = lo / PAGE, last_page = (len - 1) / PAGE;
  // quantum 0: every sequence is cut into n_splits equal shares.  quantum > 0: a block takes that many
  // pages whatever the sequence's length (sequences of unequal lengths: the long ones get more blocks
  // that work, the short ones' later blocks find nothing and write an empty partial result); the
  // last block takes what is left, should the host have counted short.
  const int per = quantum > 0 ? quantum : (last_page - first_page + 1 + n_splits - 1) / n_splits;
  const int ps = first_page + split * per;
  const int n_pg = max(0, (split == n_splits - 1 ? last_page + 1 : min(ps + per, last_page + 1)) - ps);

  if (n_pg == 0 && n_splits > 1) {
    // nothing of this sequence lies in this block's share (a short sequence beside long ones): an
    // empty partial result, marked by a sum of zero, and no more
    pdl_wait();   // the merge kernel of the step before may still read the partial results
    pdl_launch_dependents();
    if (threadIdx.x < G) {
      float* dst = part + (((size_t)b * nh + kvh * G + threadIdx.x) * n_splits + split) * PART_STRIDE;
      dst[HEAD_DIM] = -INFINITY;
      dst[HEAD_DIM + 1] = 0.0f;
    }
    return;
  }

  // one thread requests pages; `issue(i)` brings page ps + i into stage i % TD_STAGES
  auto issue = [&](int i) -> bool {
    const int s = i % TD_STAGES;
    if (!td_mbar_wait(&empty_bar[s], ((uint32_t)(i / TD_STAGES) & 1u) ^ 1u, abort_flag, 1)) return false;
    const int slab = table[ps + i] * nkv + kvh;
    uint8_t* st = smem + (size_t)s * TD_STAGE_BYTES;
    td_mbar_expect_tx(&full_bar[s], TD_STAGE_BYTES);
#pragma unroll
    for (int sub = 0; sub < K_SUB; ++sub)
      td_tma_load_2d(st + sub * (PAGE * 128), &tm_k, &full_bar[s], sub * 64, slab * PAGE);
    td_tma_load_2d(st + K_BYTES, &tm_v, &full_bar[s], 0, slab * HEAD_DIM);
    return true;
  };
  int ahead = 0;   // pages requested before the wait for the earlier kernels
  if (threadIdx.x == 0)
    for (; ahead < TD_STAGES - 1 && ahead < n_pg && ps + ahead < last_page; ++ahead) issue(ahead);
  pdl_wait();
  TL_TRACE_RELEASED();
  pdl_launch_dependents();
  if (threadIdx.x == 0)
    for (int i = ahead; i < TD_STAGES - 1 && i < n_pg; ++i) issue(i);

  // query fragments: rows are the query heads of this kv head
  uint32_t qa[NCHUNK][4], qb[NCHUNK][4];
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
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

  for (int i = 0; i < n_pg; ++i) {
    if (threadIdx.x == 0 && i + TD_STAGES - 1 < n_pg) issue(i + TD_STAGES - 1);
    __syncwarp();
    const int s = i % TD_STAGES;
    if (!td_mbar_wait(&full_bar[s], (uint32_t)(i / TD_STAGES) & 1u, abort_flag, 2)) break;
    const uint32_t kb = td_smem_u32(smem + (size_t)s * TD_STAGE_BYTES);
    const uint32_t vb_ = kb + K_BYTES;
    const int key0 = (ps + i) * PAGE + 16 * warp;   // first of this warp's 16 keys
    // ---- scores: 2 tiles of 8 keys; column c of tile jt is key 4*(c>>1) + 2*jt + (c&1)
    float sc[2][4];
#pragma unroll
    for (int jt = 0; jt < 2; ++jt) {
      sc[jt][0] = sc[jt][1] = sc[jt][2] = sc[jt][3] = 0.0f;
      const int r = 16 * warp + 4 * (g >> 1) + 2 * jt + (g & 1);   // row of the K slab
#pragma unroll
      for (int j = 0; j < NCHUNK; ++j) {
        const int chunk = 4 * j + t;
        const uint32_t addr = kb + (uint32_t)(chunk >> 3) * (PAGE * 128) + (uint32_t)r * 128 +
                              (uint32_t)(((chunk & 7) ^ (r & 7)) << 4);
        const uint4 kv = lds128(addr);
        uint32_t a[4];
        a[0] = qa[j][0]; a[1] = qb[j][0]; a[2] = qa[j][1]; a[3] = qb[j][1];
        mma_bf16(sc[jt], a, kv.x, kv.y);
        a[0] = qa[j][2]; a[1] = qb[j][2]; a[2] = qa[j][3]; a[3] = qb[j][3];
        mma_bf16(sc[jt], a, kv.z, kv.w);
      }
    }
    // ---- mask and running maximum; column 2t+e of tile jt is key 4t + 2jt + e
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int jt = 0; jt < 2; ++jt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = key0 + 4 * t + 2 * jt + e;
        const bool ok = idx >= lo && idx < len;
        sc[jt][e] = ok ? sc[jt][e] * scale_log2 : -INFINITY;
        sc[jt][2 + e] = ok ? sc[jt][2 + e] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, sc[jt][e]);
        mx1 = fmaxf(mx1, sc[jt][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    // the 16 keys of a warp may all lie outside the sequence or the window
    const float ref0 = n0 == -INFINITY ? 0.0f : n0, ref1 = n1 == -INFINITY ? 0.0f : n1;
    const float al0 = exp2f(m0 - ref0), al1 = HI ? exp2f(m1 - ref1) : 0.0f;
    m0 = n0; m1 = n1;
    uint32_t pa[4];
    float r0 = 0.0f, r1 = 0.0f;
#pragma unroll
    for (int jt = 0; jt < 2; ++jt) {
      const float p0 = exp2f(sc[jt][0] - ref0), p1 = exp2f(sc[jt][1] - ref0);
      const float p2 = HI ? exp2f(sc[jt][2] - ref1) : 0.0f, p3 = HI ? exp2f(sc[jt][3] - ref1) : 0.0f;
      r0 += p0 + p1;
      r1 += p2 + p3;
      pa[2 * jt] = pack_bf16(p0, p1);
      pa[2 * jt + 1] = pack_bf16(p2, p3);
    }
    l0 = l0 * al0 + r0;
    l1 = l1 * al1 + r1;
    // ---- o = o * alpha + p . v; thread (g, t) reads v^T[dim 8i + g][keys 16*warp + 4t .. +3]
#pragma unroll
    for (int i2 = 0; i2 < NDT; ++i2) {
      const int row = 8 * i2 + g;
      const uint32_t addr = vb_ + (uint32_t)row * 128 +
                            (uint32_t)(((2 * warp + (t >> 1)) ^ (row & 7)) << 4) + (uint32_t)(t & 1) * 8;
      const uint2 vv = lds64(addr);
      o[i2][0] *= al0; o[i2][1] *= al0; o[i2][2] *= al1; o[i2][3] *= al1;
      mma_bf16(o[i2], pa, vv.x, vv.y);
    }
    __syncwarp();
    if (lane == 0) td_mbar_arrive(&empty_bar[s]);
  }

  // ---- merge the four warps of the block (their keys are disjoint)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();   // every warp is done with the stages; the first one now holds the merge
  if (t == 0) {
    sm_m[warp * 16 + g] = m0; sm_l[warp * 16 + g] = l0;
    sm_m[warp * 16 + g + 8] = m1; sm_l[warp * 16 + g + 8] = l1;
  }
#pragma unroll
  for (int i = 0; i < NDT; ++i) {
    float* ro = sm_o + (size_t)(warp * 16 + g) * HEAD_DIM + 8 * i + 2 * t;
    ro[0] = o[i][0]; ro[1] = o[i][1];
    if (HI) { ro[8 * HEAD_DIM] = o[i][2]; ro[8 * HEAD_DIM + 1] = o[i][3]; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HEAD_DIM; idx += TD_WARPS * 32) {
    const int r = idx / HEAD_DIM, d = idx - r * HEAD_DIM;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < TD_WARPS; ++w) m = fmaxf(m, sm_m[w * 16 + r]);
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < TD_WARPS; ++w) {
      const float wm = sm_m[w * 16 + r];
      const float f = wm == -INFINITY ? 0.0f : exp2f(wm - m);
      acc += f * sm_o[(size_t)(w * 16 + r) * HEAD_DIM + d];
      l += f * sm_l[w * 16 + r];
    }
    if (n_splits == 1) {   // nothing to merge: this is the result
      out[((size_t)b * nh + kvh * G + r) * HEAD_DIM + d] = __float2bfloat16_rn(acc / l);
    } else {
      float* dst = part + (((size_t)b * nh + kvh * G + r) * n_splits + split) * PART_STRIDE;
      dst[d] = acc;
      if (d == 0) { dst[HEAD_DIM] = m; dst[HEAD_DIM + 1] = l; }
    }
  }
}

// ---------------------------------------------------------------------------
// Prefill with the same page pipeline: a block owns 64 consecutive queries of one head
// (16 per warp) and walks over the pages that any of them can see; every warp reads the
// fragments of the page it needs from shared memory.  Arithmetic as in
// attention_prefill_bf16.cu.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TD_WARPS * 32, 2)
FN(attn_prefill_tma_kernel)(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                            const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_len,
                            const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                            int table_stride, int nh, int nkv, int window, float scale_log2) {
  extern __shared__ uint8_t td_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)td_smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + TD_STAGES * TD_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + TD_STAGES;
  volatile int* abort_flag = (volatile int*)(empty_bar + TD_STAGES);
  const int b = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TD_STAGES; ++s) { td_mbar_init(&full_bar[s], 1); td_mbar_init(&empty_bar[s], TD_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();
  const int tok0 = seq_start[b];
  const int n_new = seq_start[b + 1] - tok0;
  const int blk0 = blockIdx.x * (TD_WARPS * 16);       // first query of the block
  if (blk0 >= n_new) return;
  const int len = seq_len[b];
  const int past = len - n_new;
  const int kvh = h / (nh / nkv);
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;
  // pages the block walks over: from the window start of its first query to its last query
  const int blk_first = past + blk0, blk_last = past + min(blk0 + TD_WARPS * 16, n_new) - 1;
  const int blk_lo = (window > 0 && blk_first - window + 1 > 0) ? blk_first - window + 1 : 0;
  const int ps = blk_lo / PAGE;
  const int n_pg = blk_last / PAGE - ps + 1;

  auto issue = [&](int i) -> bool {
    const int s = i % TD_STAGES;
    if (!td_mbar_wait(&empty_bar[s], ((uint32_t)(i / TD_STAGES) & 1u) ^ 1u, abort_flag, 1)) return false;
    const int slab = table[ps + i] * nkv + kvh;
    uint8_t* st = smem + (size_t)s * TD_STAGE_BYTES;
    td_mbar_expect_tx(&full_bar[s], TD_STAGE_BYTES);
#pragma unroll
    for (int sub = 0; sub < K_SUB; ++sub)
      td_tma_load_2d(st + sub * (PAGE * 128), &tm_k, &full_bar[s], sub * 64, slab * PAGE);
    td_tma_load_2d(st + K_BYTES, &tm_v, &full_bar[s], 0, slab * HEAD_DIM);
    return true;
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < TD_STAGES - 1 && i < n_pg; ++i) issue(i);

  // this warp's 16 queries; a warp past the end of the sequence only keeps the pipeline going
  const int r0 = blk0 + warp * 16;
  const bool active = r0 < n_new;
  const int ra = min(r0 + g, n_new - 1), rb = min(r0 + g + 8, n_new - 1);
  const int pa_pos = past + ra, pb_pos = past + rb;
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
  const int first_pos = past + min(r0, n_new - 1), last_pos = past + min(r0 + 15, n_new - 1);
  const int lo_w = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;

  float o[NDT][4];
#pragma unroll
  for (int i = 0; i < NDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

  for (int i = 0; i < n_pg; ++i) {
    if (threadIdx.x == 0 && i + TD_STAGES - 1 < n_pg) issue(i + TD_STAGES - 1);
    __syncwarp();
    const int s = i % TD_STAGES;
    if (!td_mbar_wait(&full_bar[s], (uint32_t)(i / TD_STAGES) & 1u, abort_flag, 2)) break;
    const uint32_t kb = td_smem_u32(smem + (size_t)s * TD_STAGE_BYTES);
    const uint32_t vb_ = kb + K_BYTES;
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      const int base = (ps + i) * PAGE + GROUP * grp;    // first key of this group of 32
      if (!active || base > last_pos || base + GROUP <= lo_w) continue;   // nothing of it is visible
      float sc[4][4];
#pragma unroll
      for (int jt = 0; jt < 4; ++jt) {
        sc[jt][0] = sc[jt][1] = sc[jt][2] = sc[jt][3] = 0.0f;
        const int r = GROUP * grp + 8 * (g >> 1) + 2 * jt + (g & 1);
#pragma unroll
        for (int j = 0; j < NCHUNK; ++j) {
          const int chunk = 4 * j + t;
          const uint4 kv = lds128(kb + (uint32_t)(chunk >> 3) * (PAGE * 128) + (uint32_t)r * 128 +
                                  (uint32_t)(((chunk & 7) ^ (r & 7)) << 4));
          uint32_t a[4];
          a[0] = qa[j][0]; a[1] = qb[j][0]; a[2] = qa[j][1]; a[3] = qb[j][1];
          mma_bf16(sc[jt], a, kv.x, kv.y);
          a[0] = qa[j][2]; a[1] = qb[j][2]; a[2] = qa[j][3]; a[3] = qb[j][3];
          mma_bf16(sc[jt], a, kv.z, kv.w);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int jt = 0; jt < 4; ++jt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int idx = base + 8 * t + 2 * jt + e;
          sc[jt][e] = (idx >= lo_a && idx <= pa_pos) ? sc[jt][e] * scale_log2 : -INFINITY;
          sc[jt][2 + e] = (idx >= lo_b && idx <= pb_pos) ? sc[jt][2 + e] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, sc[jt][e]);
          mx1 = fmaxf(mx1, sc[jt][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float ref0 = n0 == -INFINITY ? 0.0f : n0, ref1 = n1 == -INFINITY ? 0.0f : n1;
      const float al0 = exp2f(m0 - ref0), al1 = exp2f(m1 - ref1);
      m0 = n0; m1 = n1;
      uint32_t pa[2][4];
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int jt = 0; jt < 4; ++jt) {
        const float p0 = exp2f(sc[jt][0] - ref0), p1 = exp2f(sc[jt][1] - ref0);
        const float p2 = exp2f(sc[jt][2] - ref1), p3 = exp2f(sc[jt][3] - ref1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pa[jt >> 1][(jt & 1) * 2 + 0] = pack_bf16(p0, p1);
        pa[jt >> 1][(jt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      l0 = l0 * al0 + sum0;
      l1 = l1 * al1 + sum1;
#pragma unroll
      for (int i2 = 0; i2 < NDT; ++i2) {
        const int row = 8 * i2 + g;
        const uint4 vv = lds128(vb_ + (uint32_t)row * 128 + (uint32_t)(((4 * grp + t) ^ (row & 7)) << 4));
        o[i2][0] *= al0; o[i2][1] *= al0; o[i2][2] *= al1; o[i2][3] *= al1;
        mma_bf16(o[i2], pa[0], vv.x, vv.y);
        mma_bf16(o[i2], pa[1], vv.z, vv.w);
      }
    }
    __syncwarp();
    if (lane == 0) td_mbar_arrive(&empty_bar[s]);
  }
  if (!active) return;
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

// Merges the splits of one (sequence, head) and writes the normalised result.  A thread per
// dimension; the splits' maxima and sums are fetched by one thread each, so that no thread
// walks through the splits one dependent load after the other (with 33 splits that chain was
// 10 us of a 100 us layer), and the sum over the splits runs eight loads at a time.
#define COMBINE_MAX_SPLITS 256
__global__ void __launch_bounds__(HEAD_DIM)
FN(attn_decode_tma_combine_kernel)(const float* __restrict__ part, __nv_bfloat16* __restrict__ out,
                                   int nh, int n_splits) {
  TL_TRACE_SCOPE(5, n_splits, 5);
  __shared__ float f_s[COMBINE_MAX_SPLITS];
  __shared__ float red_s[2 * (HEAD_DIM / 32)];
  pdl_wait();
  TL_TRACE_RELEASED();
  pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int warp = d >> 5, lane = d & 31;
  const float* src = part + ((size_t)b * nh + h) * n_splits * PART_STRIDE;
  if (n_splits <= COMBINE_MAX_SPLITS) {
    // this thread's dimension of the first 32 splits: all loads at once, before anything waits for
    // them (they do not depend on the factors)
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = j < n_splits ? src[j * PART_STRIDE + d] : 0.0f;
    // each split's maximum and sum, one thread per split (several rounds if there are more splits)
    float m = -INFINITY, lsum[(COMBINE_MAX_SPLITS + HEAD_DIM - 1) / HEAD_DIM], msp[(COMBINE_MAX_SPLITS + HEAD_DIM - 1) / HEAD_DIM];
    int cnt = 0;
    for (int s = d; s < n_splits; s += HEAD_DIM, ++cnt) {
      msp[cnt] = src[s * PART_STRIDE + HEAD_DIM];
      lsum[cnt] = src[s * PART_STRIDE + HEAD_DIM + 1];
      m = fmaxf(m, msp[cnt]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red_s[warp] = m;
    __syncthreads();
    m = red_s[0];
#pragma unroll
    for (int w = 1; w < HEAD_DIM / 32; ++w) m = fmaxf(m, red_s[w]);
    float l = 0.0f;
    cnt = 0;
    for (int s = d; s < n_splits; s += HEAD_DIM, ++cnt) {
      const float f = msp[cnt] == -INFINITY ? 0.0f : exp2f(msp[cnt] - m);
      f_s[s] = f;
      l += f * lsum[cnt];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) red_s[HEAD_DIM / 32 + warp] = l;
    __syncthreads();
    l = red_s[HEAD_DIM / 32];
#pragma unroll
    for (int w = 1; w < HEAD_DIM / 32; ++w) l += red_s[HEAD_DIM / 32 + w];
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j)   // an empty split's values were never written: its factor is 0, its values are not touched
      if (j < n_splits && f_s[j] != 0.0f) acc += f_s[j] * v[j];
    for (int s = 32; s < n_splits; ++s)
      if (f_s[s] != 0.0f) acc += f_s[s] * src[s * PART_STRIDE + d];
    out[((size_t)b * nh + h) * HEAD_DIM + d] = __float2bfloat16_rn(acc / l);
    return;
  }
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[s * PART_STRIDE + HEAD_DIM]);
  float acc = 0.0f, l = 0.0f;
  for (int s = 0; s < n_splits; ++s) {
    const float sm = src[s * PART_STRIDE + HEAD_DIM];
    const float f = sm == -INFINITY ? 0.0f : exp2f(sm - m);
    if (f != 0.0f) acc += f * src[s * PART_STRIDE + d];
    l += f * src[s * PART_STRIDE + HEAD_DIM + 1];
  }
  out[((size_t)b * nh + h) * HEAD_DIM + d] = __float2bfloat16_rn(acc / l);
}

// ---------------------------------------------------------------------------
// Host side: tensor maps over the page storage (cached by address), launch.
// ---------------------------------------------------------------------------
typedef CUresult (*TdEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

static TdEncodeFn td_encode_fn() {
  static TdEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TdEncodeFn)p;
  });
  return fn;
}

// rows x cols bfloat16, contiguous rows; boxes of 64 columns (128 bytes) x box_rows, 128-byte swizzle
static bool td_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
  typedef std::tuple<const void*, long long, long long, int> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key(ptr, rows, cols, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  TdEncodeFn fn = td_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = m;
  *map = m;
  return true;
}

// As tl_attn_decode_hd<N>, plus the number of pages of the storage (for the tensor maps) and `quantum`:
// 0, or the pages a block takes (see the kernel).
// Returns -2 for sizes this kernel does not take.
extern "C" int FN(tl_attn_decode_tma)(const void* q, const void* k_pages, const void* v_pages,
                                      long long n_pages, void* out, float* part, const int* seq_len,
                                      const int* seq_slot, const int* page_table, int table_stride,
                                      int B, int nh, int nkv, int window, float scale, int n_splits,
                                      int quantum, cudaStream_t stream) {
#if HEAD_DIM % 64 != 0
  return -2;
#else
  if (B <= 0) return 0;
  if (quantum < 0) return -1;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || n_splits < 1 || n_splits > 65535 ||
      nkv > 65535 || B > 65535 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    return -2;
  CUtensorMap tk, tv;
  if (!td_make_map(&tk, k_pages, n_pages * nkv * PAGE, HEAD_DIM, PAGE)) return -2;
  if (!td_make_map(&tv, v_pages, n_pages * nkv * HEAD_DIM, PAGE, HEAD_DIM)) return -2;
  const size_t smem = 1024 + (size_t)TD_STAGES * TD_STAGE_BYTES + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(FN(attn_decode_tma_kernel)<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(FN(attn_decode_tma_kernel)<false>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_splits, nkv, B);
  int st;
  if (nh / nkv > 8)
    st = tl_launch(FN(attn_decode_tma_kernel)<true>, grid, dim3(TD_WARPS * 32), smem, stream, tk, tv,
                   (const __nv_bfloat16*)q, part, (__nv_bfloat16*)out, seq_len, seq_slot, page_table,
                   table_stride, nh, nkv, window, scale_log2, n_splits, quantum);
  else
    st = tl_launch(FN(attn_decode_tma_kernel)<false>, grid, dim3(TD_WARPS * 32), smem, stream, tk, tv,
                   (const __nv_bfloat16*)q, part, (__nv_bfloat16*)out, seq_len, seq_slot, page_table,
                   table_stride, nh, nkv, window, scale_log2, n_splits, quantum);
  if (st || n_splits == 1) return st;   // a single split has written the result itself
  return tl_launch(FN(attn_decode_tma_combine_kernel), dim3(nh, B), dim3(HEAD_DIM), 0, stream,
                   (const float*)part, (__nv_bfloat16*)out, nh, n_splits);
#endif
}

// As tl_attn_prefill_hd<N>, plus the number of pages of the storage.
extern "C" int FN(tl_attn_prefill_tma)(const void* q, const void* k_pages, const void* v_pages,
                                       long long n_pages, void* out, const int* seq_start,
                                       const int* seq_len, const int* seq_slot, const int* page_table,
                                       int table_stride, int B, int max_new, int nh, int nkv,
                                       int window, float scale, cudaStream_t stream) {
#if HEAD_DIM % 64 != 0
  return -2;
#else
  if (B <= 0 || max_new <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh > 65535 || B > 65535 || ((uintptr_t)k_pages & 15) ||
      ((uintptr_t)v_pages & 15))
    return -2;
  CUtensorMap tk, tv;
  if (!td_make_map(&tk, k_pages, n_pages * nkv * PAGE, HEAD_DIM, PAGE)) return -2;
  if (!td_make_map(&tv, v_pages, n_pages * nkv * HEAD_DIM, PAGE, HEAD_DIM)) return -2;
  const size_t smem = 1024 + (size_t)TD_STAGES * TD_STAGE_BYTES + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(FN(attn_prefill_tma_kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_new + TD_WARPS * 16 - 1) / (TD_WARPS * 16), nh, B);
  return tl_launch(FN(attn_prefill_tma_kernel), grid, dim3(TD_WARPS * 32), smem, stream, tk, tv,
                   (const __nv_bfloat16*)q, (__nv_bfloat16*)out, seq_start, seq_len, seq_slot,
                   page_table, table_stride, nh, nkv, window, scale * 1.4426950408889634f);
#endif
}

extern "C" int FN(tl_attn_tma_take_error)() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, tl_attn_tma_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(tl_attn_tma_error, &zero, sizeof(int));
  return v;
}

TL_TRACE_EXPORT(attn_tma)
