// Prefill attention of the bfloat16 path on the fifth-generation tensor cores.
//
// A block owns 128 consecutive queries of one head (the M of tcgen05.mma) and walks over
// the cache pages that any of them can see.  Per page of 64 keys:
//   S[128, 64]  = Q . K^T        tcgen05.mma, Q and the page's K slab in shared memory,
//                                S in tensor memory
//   softmax     four warps, one thread per query row: tcgen05.ld of the row, mask, running
//               maximum and sum in 32-bit (no shuffles: a row lives in one thread), P
//               rounded to bfloat16 back into tensor memory (tcgen05.st, over the S buffer);
//               O is rescaled in tensor memory only when some row's maximum moved
//   O[128, hd] += P . V          tcgen05.mma with P as the A operand in tensor memory and
//                                the page's transposed V slab as the K-major B operand
// S has two buffers in tensor memory: Q . K^T of page i + 1 is issued (by a thread of its
// own) before the softmax of page i has ended, and P . V of page i (issued by another thread)
// runs under the softmax of page i + 1, so the softmax warps rarely wait for a product.  Pages
// come by TMA, K slabs one page ahead of V slabs.  What was measured with clock64() stamps in
// one block while P still went through shared memory: per page the softmax takes about 1100
// cycles of arithmetic (bound by the 16 exponentials a cycle of an SM when two blocks share
// it), 450 for the P stores and the proxy fence that the tensor core's reads of shared memory
// need (what moving P to tensor memory saves), 200 for the barrier; issuing one tcgen05.mma
// costs its thread about 80 cycles.
// Arithmetic as in attention_prefill_bf16.cu (reference: src/model/modules/attention.rs:88-121,
// src/model/modules/flash_attention.rs:101-136, window of src/model/models/gpt_oss.rs:168-176).
// Head sizes 64 and 128.
//
// Every wait on an mbarrier is bounded; when a bound is hit the block records a code in
// tl_attn_tc_error, stops, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>

#include "attention_bf16_common.cuh"

#include <map>
#include <mutex>
#include <tuple>

#define TC_Q 128                         // queries per block
// Two blocks per SM (one block's products overlap the other's softmax) leave each block room
// for five page slabs beside its queries: three of K, whose page i + 1 is wanted one softmax
// earlier than its V and which Q . K^T alone reads, and two of V, free again after P . V.
#define TC_KSLOTS 3
#define TC_VSLOTS 2
#define TC_THREADS 224                   // warps 0-3 softmax, warp 4 TMA, warp 5 issues Q.K^T, warp 6 issues P.V
#define TC_KSUB (HEAD_DIM / 64)
#define TC_Q_BYTES (TC_Q * HEAD_DIM * 2)
#define TC_K_BYTES (PAGE * HEAD_DIM * 2)
#define TC_V_BYTES (HEAD_DIM * PAGE * 2)
// P goes back into tensor memory, over the first 32 columns of the S buffer it was computed
// from (two bfloat16 per column), and P . V takes its A operand from there: no shared memory
// for P and no proxy fence between the softmax's stores and the tensor core's reads.
#define TC_SMEM_BYTES (TC_Q_BYTES + TC_KSLOTS * TC_K_BYTES + TC_VSLOTS * TC_V_BYTES + 256)
#define TC_TMEM_COLS 256   // S twice (64 columns each), then O (HEAD_DIM columns)

__device__ int tl_attn_tc_error = 0;


__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  return tl_mbar_wait(bar, parity, abort_flag, code, &tl_attn_tc_error);   // bounded_wait.cuh
}
__device__ __forceinline__ void tc_tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(tc_smem_u32(dst)), "l"(map), "r"(tc_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
      : "memory");
}
// The same with the A operand in tensor memory (row = lane, two bfloat16 per column).
__device__ __forceinline__ void tc_umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc)
      : "memory");
}
// A wait that lets the hardware park the thread (up to about a microsecond per try) instead of
// spinning: the spinning threads would take issue slots from the softmax warps.
__device__ __forceinline__ bool tc_mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  for (uint32_t i = 0; i < (TL_WAIT_LIMIT >> 2); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc_smem_u32(bar)), "r"(parity), "r"(1000u)
        : "memory");
    if (ok) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = code;
  atomicCAS(&tl_attn_tc_error, 0, code);
  return false;
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tc_ex2(float x) {   // 2^x, one instruction; tiny results flush to zero
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two 32-bit floats in one 64-bit register, and the packed arithmetic of sm_100 on them.
__device__ __forceinline__ uint64_t tc_pack2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void tc_unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t tc_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t tc_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float tc_max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// K-major tile with 128-byte rows and the 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t tc_idesc(int n) {   // bf16 x bf16 -> f32, M = 128, both K-major
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__global__ void __launch_bounds__(TC_THREADS)
FN(attn_prefill_tc_kernel)(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, __nv_bfloat16* __restrict__ out,
                           const int* __restrict__ seq_start, const int* __restrict__ seq_len,
                           const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                           int table_stride, int nh, int nkv, int window, float scale_log2) {
  // The tiles need 1024-byte alignment (128-byte swizzle) and two blocks per SM leave no room
  // for padding, so the dynamic shared memory itself must start on such a boundary (it does
  // when the kernel has no static shared memory; checked below).
  extern __shared__ __align__(1024) uint8_t tc_smem_raw[];
  uint8_t* smem = tc_smem_raw;
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + TC_Q_BYTES;
  uint8_t* v_s = k_s + TC_KSLOTS * TC_K_BYTES;
  uint64_t* q_full = (uint64_t*)(v_s + TC_VSLOTS * TC_V_BYTES);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + TC_KSLOTS;
  uint64_t* v_full = k_empty + TC_KSLOTS;
  uint64_t* v_empty = v_full + TC_VSLOTS;
  uint64_t* s_full = v_empty + TC_VSLOTS;   // [2], one per S buffer
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* o_done = p_full + 2;
  uint64_t* pv_done = o_done + 1;            // [2]: P . V of the page whose P lies in S buffer u is done
  uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int b = blockIdx.z, h = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  pdl_launch_dependents();
  const int tok0 = seq_start[b];
  const int n_new = seq_start[b + 1] - tok0;
  // the last queries of a sequence see the most keys: their blocks come first in the grid, for all
  // heads (the fastest index) before any shorter block, so that the launch ends with the short ones
  const int blk0 = (int)(gridDim.y - 1 - blockIdx.y) * TC_Q;
  if (blk0 >= n_new) return;   // before any tensor memory is taken
  if (tc_smem_u32(tc_smem_raw) & 1023u) {   // see above; nothing has been allocated yet
    if (threadIdx.x == 0) atomicCAS(&tl_attn_tc_error, 0, 9);
    return;
  }

  if (threadIdx.x == 0) {
    tc_mbar_init(q_full, 1);
    for (int s = 0; s < TC_KSLOTS; ++s) { tc_mbar_init(&k_full[s], 1); tc_mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < TC_VSLOTS; ++s) { tc_mbar_init(&v_full[s], 1); tc_mbar_init(&v_empty[s], 1); }
    for (int u = 0; u < 2; ++u) { tc_mbar_init(&s_full[u], 1); tc_mbar_init(&p_full[u], 128); }
    tc_mbar_init(o_done, 1);
    tc_mbar_init(&pv_done[0], 1);
    tc_mbar_init(&pv_done[1], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)),
                 "r"((uint32_t)TC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * PAGE;   // the two S buffers take the first 128 columns

  const int len = seq_len[b];
  const int past = len - n_new;
  const int kvh = h / (nh / nkv);
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;
  const int rows = min(TC_Q, n_new - blk0);
  const int blk_first = past + blk0, blk_last = past + blk0 + rows - 1;
  const int blk_lo = (window > 0 && blk_first - window + 1 > 0) ? blk_first - window + 1 : 0;
  const int ps = blk_lo / PAGE;
  const int n_pg = blk_last / PAGE - ps + 1;

  if (warp == 4 && lane == 0) {
    // ---- TMA producer: the block's queries once, then the pages
    tc_mbar_expect_tx(q_full, TC_Q_BYTES);
#pragma unroll
    for (int sub = 0; sub < TC_KSUB; ++sub)
      tc_tma_load_2d(q_s + sub * (TC_Q * 128), &tm_q, q_full, h * HEAD_DIM + sub * 64, tok0 + blk0);
    for (int i = 0; i <= n_pg; ++i) {
      if (i < n_pg) {
        const int s = i % TC_KSLOTS;
        if (!tc_mbar_wait_parked(&k_empty[s], ((uint32_t)(i / TC_KSLOTS) & 1u) ^ 1u, abort_flag, 1)) break;
        const int slab = table[ps + i] * nkv + kvh;
        tc_mbar_expect_tx(&k_full[s], TC_K_BYTES);
#pragma unroll
        for (int sub = 0; sub < TC_KSUB; ++sub)
          tc_tma_load_2d(k_s + (size_t)s * TC_K_BYTES + sub * (PAGE * 128), &tm_k, &k_full[s], sub * 64, slab * PAGE);
      }
      if (i > 0) {
        const int j = i - 1, s = j % TC_VSLOTS;
        if (!tc_mbar_wait_parked(&v_empty[s], ((uint32_t)(j / TC_VSLOTS) & 1u) ^ 1u, abort_flag, 1)) break;
        const int slab = table[ps + j] * nkv + kvh;
        tc_mbar_expect_tx(&v_full[s], TC_V_BYTES);
        tc_tma_load_2d(v_s + (size_t)s * TC_V_BYTES, &tm_v, &v_full[s], 0, slab * HEAD_DIM);
      }
    }
  } else if ((warp == 5 || warp == 6) && lane == 0) {
    // ---- two MMA issuers.  Issuing costs some 80 cycles an instruction, twelve instructions a
    // page, so one thread (warp 5) issues Q . K^T and another (warp 6) P . V.  A descriptor is a
    // constant high word and a low word = (address >> 4) | 1 << 16.
    const uint32_t idesc_s = tc_idesc(PAGE), idesc_o = tc_idesc(HEAD_DIM);
    const uint32_t desc_hi = (uint32_t)(tc_desc(0) >> 32);
    auto lo_of = [](uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); };
    auto desc_of = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | lo; };
    const uint32_t q_lo = lo_of(tc_smem_u32(q_s));
    const uint32_t k_lo = lo_of(tc_smem_u32(k_s)), v_lo = lo_of(tc_smem_u32(v_s));
    bool ok = true;
    if (warp == 5) {
      // S(j) = Q . K(j)^T into buffer j & 1, up to two pages ahead of the softmax
      ok = tc_mbar_wait_parked(q_full, 0, abort_flag, 2);
      for (int j = 0; j < n_pg && ok; ++j) {
        if (j >= 2) {
          // the buffer holds P(j - 2) until P(j - 2) . V(j - 2) has read it
          ok = tc_mbar_wait_parked(&pv_done[j & 1], (uint32_t)((j - 2) >> 1) & 1u, abort_flag, 4);
          if (!ok) break;
        }
        ok = tc_mbar_wait_parked(&k_full[j % TC_KSLOTS], (uint32_t)(j / TC_KSLOTS) & 1u, abort_flag, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ka = k_lo + (uint32_t)(j % TC_KSLOTS) * (TC_K_BYTES >> 4);
        const uint32_t acc = tmem_base + (uint32_t)(j & 1) * PAGE;
#pragma unroll
        for (int kk = 0; kk < HEAD_DIM / 16; ++kk) {
          // 32 bytes per step inside a 64-column box; the boxes of Q and of K lie one after another
          const uint32_t q_off = (uint32_t)(kk >> 2) * ((TC_Q * 128) >> 4) + (kk & 3) * 2;
          const uint32_t k_off = (uint32_t)(kk >> 2) * ((PAGE * 128) >> 4) + (kk & 3) * 2;
          tc_umma(acc, desc_of(q_lo + q_off), desc_of(ka + k_off), idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[j % TC_KSLOTS]);   // nothing else reads the K slab
      }
    } else {
      // O (+)= P(j) . V(j)
      for (int j = 0; j < n_pg && ok; ++j) {
        ok = tc_mbar_wait_parked(&v_full[j % TC_VSLOTS], (uint32_t)(j / TC_VSLOTS) & 1u, abort_flag, 3) &&
             tc_mbar_wait_parked(&p_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = v_lo + (uint32_t)(j % TC_VSLOTS) * (TC_V_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < PAGE / 16; ++k)   // 16 keys = 8 columns of P
          tc_umma_ts(tmem_o, tmem_base + (uint32_t)(j & 1) * PAGE + k * 8, desc_of(va + k * 2), idesc_o,
                     (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(o_done);
        tc_commit(&pv_done[j & 1]);
        tc_commit(&v_empty[j % TC_VSLOTS]);
      }
    }
  } else if (warp < 4) {
    // ---- softmax: one thread per query row
    const int r = threadIdx.x;
    const bool valid_row = r < rows;
    const int pos = past + blk0 + min(r, rows - 1);
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const uint32_t t_s = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t t_o = tmem_o + ((uint32_t)(warp * 32) << 16);
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int i = 0; i < n_pg; ++i) {
      ok = tc_mbar_wait(&s_full[i & 1], (uint32_t)(i >> 1) & 1u, abort_flag, 5);
      if (!ok) break;
      tc_fence_after();
      uint32_t sa[32], sb[32];
      tc_ld32(t_s + (uint32_t)(i & 1) * PAGE, sa);
      tc_ld32(t_s + (uint32_t)(i & 1) * PAGE + 32, sb);
      tc_wait_ld();
      const int key0 = (ps + i) * PAGE;
      // a page that every row of this warp sees whole needs no mask (all but the pages on the
      // diagonal and at a window's edge)
      const bool whole = __all_sync(0xffffffffu, valid_row && key0 >= lo && key0 + PAGE - 1 <= pos);
      float mx = -INFINITY;
      if (whole) {
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = tc_max3(mx, __uint_as_float(sa[j]), __uint_as_float(sb[j]));
        mx *= scale_log2;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int ka_ = key0 + j, kb_ = key0 + 32 + j;
          const float va = (valid_row && ka_ >= lo && ka_ <= pos) ? __uint_as_float(sa[j]) : -INFINITY;
          const float vb = (valid_row && kb_ >= lo && kb_ <= pos) ? __uint_as_float(sb[j]) : -INFINITY;
          sa[j] = __float_as_uint(va);
          sb[j] = __float_as_uint(vb);
          mx = tc_max3(mx, va, vb);
        }
        mx *= scale_log2;   // the scale is positive; -inf stays -inf
      }
      // `m` is the reference of the exponentials, not the exact running maximum: it moves only
      // when a score exceeds it by more than 2^8, so that O in tensor memory is rarely rescaled;
      // until then p may be as large as 256, which bfloat16 and the 32-bit sums hold with ease
      const float m_new = (mx > m + 8.0f || m == -INFINITY) ? fmaxf(m, mx) : m;
      const float ref = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = exp2f(m - ref);
      m = m_new;
      // two scores at a time: one packed multiply-add for the exponents, one packed add for
      // the sums (fma.rn.f32x2, add.rn.f32x2); the exponentials themselves are single
      uint32_t pk[32];   // the row of P as bfloat16 pairs: 64 keys = 128 bytes
      const uint64_t scale2 = tc_pack2(scale_log2, scale_log2), nref2 = tc_pack2(-ref, -ref);
      uint64_t sum_a = tc_pack2(0.0f, 0.0f), sum_b = sum_a;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1, x2, x3;
        tc_unpack2(tc_fma2(tc_pack2(__uint_as_float(sa[2 * j]), __uint_as_float(sa[2 * j + 1])), scale2, nref2), x0, x1);
        tc_unpack2(tc_fma2(tc_pack2(__uint_as_float(sb[2 * j]), __uint_as_float(sb[2 * j + 1])), scale2, nref2), x2, x3);
        const float p0 = tc_ex2(x0), p1 = tc_ex2(x1), p2 = tc_ex2(x2), p3 = tc_ex2(x3);
        sum_a = tc_add2(sum_a, tc_pack2(p0, p1));
        sum_b = tc_add2(sum_b, tc_pack2(p2, p3));
        pk[j] = pack_bf16(p0, p1);
        pk[16 + j] = pack_bf16(p2, p3);
      }
      float sum, sum_hi;
      tc_unpack2(tc_add2(sum_a, sum_b), sum, sum_hi);
      sum += sum_hi;
      l = l * alpha + sum;
      // O is touched only when some row's reference moved.  Every warp waits for P(i-1) . V(i-1)
      // on every page all the same (by now it has nearly always ended): a warp that looked at
      // this barrier only now and then could take the phase of P(i-3) . V(i-3) for this one,
      // because nothing orders the arrival of page i - 2 on it before this warp gets here.
      if (i > 0) {
        ok = tc_mbar_wait(o_done, (uint32_t)(i - 1) & 1u, abort_flag, 6);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
          for (int c = 0; c < HEAD_DIM; c += 32) {
            uint32_t ov[32];
            tc_ld32(t_o + c, ov);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
            tc_st32(t_o + c, ov);
          }
          tc_wait_st();
        }
      }
      tc_st32(t_s + (uint32_t)(i & 1) * PAGE, pk);   // this lane's row of P, keys 2c and 2c + 1 in column c
      tc_wait_st();
      tc_fence_before();
      tc_mbar_arrive(&p_full[i & 1]);
    }
    if (ok) ok = tc_mbar_wait(o_done, (uint32_t)(n_pg - 1) & 1u, abort_flag, 7);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = out + ((size_t)(tok0 + blk0 + r) * nh + h) * HEAD_DIM;
#pragma unroll
      for (int c = 0; c < HEAD_DIM; c += 32) {
        uint32_t ov[32];
        tc_ld32(t_o + c, ov);
        tc_wait_ld();
        if (valid_row) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(ov[j]) * inv, __uint_as_float(ov[j + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(ov[j + 2]) * inv, __uint_as_float(ov[j + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(ov[j + 4]) * inv, __uint_as_float(ov[j + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(ov[j + 6]) * inv, __uint_as_float(ov[j + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + j) = w;
          }
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TC_TMEM_COLS)
                 : "memory");
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

static TcEncodeFn tc_encode_fn() {
  static TcEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TcEncodeFn)p;
  });
  return fn;
}

// rows x cols bfloat16, contiguous rows; boxes of 64 columns (128 bytes) x box_rows, 128-byte swizzle
static bool tc_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
  typedef std::tuple<const void*, long long, long long, int> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key(ptr, rows, cols, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  TcEncodeFn fn = tc_encode_fn();
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

// q, out [T, nh*HEAD_DIM]; max_new = the most new tokens any sequence of the step has.
// Returns -2 for sizes this kernel does not take.
extern "C" int FN(tl_attn_prefill_tc)(const void* q, long long T, const void* k_pages, const void* v_pages,
                                      long long n_pages, void* out, const int* seq_start,
                                      const int* seq_len, const int* seq_slot, const int* page_table,
                                      int table_stride, int B, int max_new, int nh, int nkv, int window,
                                      float scale, cudaStream_t stream) {
#if HEAD_DIM % 64 != 0
  return -2;
#else
  if (B <= 0 || max_new <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh > 65535 || B > 65535 || ((uintptr_t)q & 15) ||
      ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    return -2;
  CUtensorMap tq, tk, tv;
  if (!tc_make_map(&tq, q, T, (long long)nh * HEAD_DIM, TC_Q)) return -2;
  if (!tc_make_map(&tk, k_pages, n_pages * nkv * PAGE, HEAD_DIM, PAGE)) return -2;
  if (!tc_make_map(&tv, v_pages, n_pages * nkv * HEAD_DIM, PAGE, HEAD_DIM)) return -2;
  const size_t smem = TC_SMEM_BYTES;   // the last 256 bytes hold the barriers
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(FN(attn_prefill_tc_kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int q_tiles = (max_new + TC_Q - 1) / TC_Q;
  if (q_tiles > 65535) return -2;
  dim3 grid(nh, q_tiles, B);
  return tl_launch(FN(attn_prefill_tc_kernel), grid, dim3(TC_THREADS), smem, stream, tq, tk, tv,
                   (__nv_bfloat16*)out, seq_start, seq_len, seq_slot, page_table, table_stride, nh, nkv,
                   window, scale * 1.4426950408889634f);
#endif
}

extern "C" int FN(tl_attn_tc_take_error)() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, tl_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(tl_attn_tc_error, &zero, sizeof(int));
  return v;
}

