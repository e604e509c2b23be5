// Matrix products of the bfloat16 path on the fifth-generation tensor cores.
//
//   C[M, N] (op)= X[M, K] * W[N, K]^T      X, W bfloat16 with K contiguous, 32-bit sums
//
// (The reference computes one output at a time as a sequential 32-bit dot product of a weight row
// with one token's activations, widening bfloat16 on the fly: src/loader/weight_matrix.rs:82-91,
// src/loader/parameters.rs:551-594.)
//
// The product is computed transposed: 128 rows of W are the M operand of tcgen05.mma,
// a tile of BN rows of X (tokens) is its N operand, and the accumulator lies in tensor
// memory as [128 weight rows][BN tokens].  So the same kernel serves one decoded token
// per sequence (BN = 16: the weights stream through TMA at full width and the padding
// costs nothing that matters) and more tokens (up to BN = 256; from 129 tokens on the
// kernel on pairs of SMs further down takes over).  Operands come by TMA into
// 128-byte-swizzled shared memory tiles of 64 K-elements, one or two of them per operand
// and stage; one thread issues the instructions (each costs it some 70 cycles, a stage's
// barrier wait, commit and loop some 400, which is why a stage holds eight instructions);
// four warps read the accumulator back with tcgen05.ld and write C, each warp-store
// covering 32 consecutive columns of one row of C.
//
// When a product has too few tiles to fill the GPU (decode), K is split over
// blockIdx.z and the blocks of one tile form a thread-block cluster.  Each block puts
// its partial tile into its own shared memory; after a cluster barrier the blocks share
// the columns of the tile among them, and each adds the partials of its columns in split
// order through distributed shared memory and writes C.  No scratch in global memory,
// no atomics, the same bits every run.
//
// Output modes as in gemm_generic.cu: 0 store 32-bit, 1 add into 32-bit C, 2 SiLU-gate
// (W holds N gate rows then N up rows; two accumulators), 3 store bfloat16.
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel records a code
// in tl_gemm_tc_error, stops waiting everywhere, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "bounded_wait.cuh"
#include "pdl.cuh"

#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

#define TILE_N 128        // weight rows per tile (M of the instruction)
#define TILE_K 64         // K elements per shared memory tile (128 bytes)
#define UMMA_K 16
#define NUM_THREADS 192   // warps 0-3 epilogue, warp 4 TMA, warp 5 MMA

#define MODE_STORE_F32 0
#define MODE_ACCUM_F32 1
#define MODE_SWIGLU 2
#define MODE_STORE_ACT 3

__device__ int tl_gemm_tc_error = 0;

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return tl_smem_u32(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) { tl_mbar_init(bar, count); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded wait (bounded_wait.cuh).  Returns false when the bound is hit or another role has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int code) {
  return tl_mbar_wait(bar, parity, abort_flag, code, &tl_gemm_tc_error);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when all tcgen05.mma issued so far by this thread are done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,"
      "%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared memory matrix descriptor of a K-major tile whose rows are 128 bytes with the
// 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                     // leading byte offset (unused with a swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                     // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_remote_f32(uint32_t local_saddr, uint32_t rank) {
  uint32_t raddr;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_saddr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float4 ld_remote_f32x4(uint32_t local_saddr, uint32_t rank) {
  uint32_t raddr;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_saddr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(raddr) : "memory");
  return v;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

// ---------------------------------------------------------------------------
// The kernel.  grid = (tiles of 128 weight rows, tiles of BN tokens, K splits).
// ---------------------------------------------------------------------------
struct GemmArgs {
  void* C;
  int ldc, M, N, K, mode, kb_per_split, stages;
  int raster;      // pair kernel: weight strips per group of the tile order (0: strip by strip)
  // Norm folded into the products around it (see the launcher's text).
  const float* ss_in;       // [M, ss_in_tiles] partial sums of squares of the input rows, or null
  int ss_in_tiles, norm_h;
  float eps_in;
  __nv_bfloat16* xw_out;    // [M, N] the new C times the next norm's weight, or null
  const void* nw;           // that weight [N]
  int nw_is_f32;
  float* ss_out;            // [M, tiles of N] partial sums of squares of the new C
  // Rotation and cache write folded into the q/k/v product (K split only): the product's
  // columns are query heads, then key heads, then value heads of `hd` columns each.
  int rope_on, rope_style, rope_nh, rope_nkv, rope_hd, rope_table_stride;
  __nv_bfloat16* rope_q;    // [M, nh * hd]
  __nv_bfloat16* rope_k;    // key pages [pages, nkv, TL_PAGE, hd]
  __nv_bfloat16* rope_v;    // value pages [pages, nkv, hd, TL_PAGE]
  const int* rope_pos;      // [M] position of each token
  const int* rope_seq;      // [M] batch row of each token
  const int* rope_slot;     // cache slot of each batch row
  const int* rope_table;    // page table
  const float* rope_inv_freq;   // [hd / 2] or null
};

// The tail of a block's shared memory, after the stages: barriers and flags (256 bytes), the
// per-warp sums of squares of the fold (1 KB), the tokens' 1/rms (1 KB) and, for token tiles
// of 16 without the SiLU-gate, the cosines and sines of the folded rotation (8 KB).
#define ROPE_TABLE_HALF 64   // pairs of dimensions per token: head sizes up to 128
#define TAIL_BYTES 2304
#define TAIL_ROPE_BYTES (16 * ROPE_TABLE_HALF * 8)
__device__ __forceinline__ float* tail_ssw(uint8_t* tail) { return (float*)tail + 64; }
__device__ __forceinline__ float* tail_rinv(uint8_t* tail) { return (float*)tail + 64 + 256; }
__device__ __forceinline__ float2* tail_cossin(uint8_t* tail) { return (float2*)(tail + TAIL_BYTES); }

// 1 / sqrt(mean(x^2) + eps) of input row m from the partial sums the producer left.
__device__ __forceinline__ float row_rinv(const GemmArgs& a, int m) {
  float ss = 0.0f;
  for (int t = 0; t < a.ss_in_tiles; ++t) ss += __ldcg(a.ss_in + (size_t)m * a.ss_in_tiles + t);
  return 1.0f / sqrtf(ss / (float)a.norm_h + a.eps_in);
}

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const GemmArgs args) {
  TL_TRACE_SCOPE(3, (long long)args.N * 16 + args.mode, 8 + ((args.N >> 7) ^ (args.K >> 9) ^ args.mode));
  // A stage holds KS sub-tiles of 64 K-elements (128 bytes) per operand: two where one weight
  // matrix is read, so that the issuing thread pays its fixed cost per stage (barrier wait,
  // commit, loop: some 400 cycles) once per eight instructions; the SiLU-gate's two matrices
  // make eight instructions per 64 elements already.  Layout: [A sub-tiles][B sub-tiles].
  constexpr int KS = SWIGLU ? 1 : 2;
  constexpr int KSTEP = TILE_K * KS;
  constexpr uint32_t A_BYTES = TILE_N * TILE_K * 2;
  constexpr uint32_t B_BYTES = BN * TILE_K * 2;
  constexpr uint32_t STAGE_BYTES = KS * (A_BYTES * (SWIGLU ? 2 : 1) + B_BYTES);
  constexpr uint32_t B_OFF = KS * A_BYTES * (SWIGLU ? 2 : 1);
  constexpr uint32_t ACC_COLS = BN * (SWIGLU ? 2 : 1);
  constexpr uint32_t TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;   // a power of two >= 32
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(TILE_N >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + 8;
  uint64_t* acc_bar = empty_bar + 8;
  uint32_t* tmem_slot = (uint32_t*)(acc_bar + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* last_flag = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TILE_N, m0 = blockIdx.y * BN;
  const int splits = gridDim.z, split = blockIdx.z;
  const int kb_total = (args.K + KSTEP - 1) / KSTEP;
  const int kb0 = split * args.kb_per_split;
  const int kb1 = min(kb0 + args.kb_per_split, kb_total);
  const int n_kb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 4 && lane == 0) {
    // ---- TMA producer.  The weights do not depend on earlier kernels, so the tiles of the
    // first stages are requested before the wait for those kernels; the activations after it.
    const int pre = n_kb < stages ? n_kb : stages;
    auto load_w = [&](uint8_t* st, uint64_t* bar, int kb) {
#pragma unroll
      for (int h = 0; h < KS; ++h) {
        const int k = kb * KSTEP + h * TILE_K;   // past K the tile is filled with zeros
        tma_load_2d(st + h * A_BYTES, &tm_w, bar, k, n0);
        if (SWIGLU) tma_load_2d(st + A_BYTES, &tm_w, bar, k, args.N + n0);
      }
    };
    auto load_x = [&](uint8_t* st, uint64_t* bar, int kb) {
#pragma unroll
      for (int h = 0; h < KS; ++h)
        tma_load_2d(st + B_OFF + h * B_BYTES, &tm_x, bar, kb * KSTEP + h * TILE_K, m0);
    };
    // Every block walks its K range from another start (and wraps round): with all blocks at the same
    // K offset of their rows at the same time, the requests fall on addresses a multiple of the row
    // length apart and all blocks ask for the same activations at once.  Measured at 8 tokens: q/k/v
    // 11.5 -> 11.1 us, gate-up 38.0 -> 37.3 us, down 21.3 -> 20.9 us; at 64 tokens gate-up 45.9 ->
    // 44.2 us (the multiplier made no difference).  The sums of a block only change their order.
    const int rot = (int)((blockIdx.x * 3u) % (unsigned)n_kb);
    auto kof = [&](int i) { int k = i + rot; if (k >= n_kb) k -= n_kb; return kb0 + k; };
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full_bar[i], STAGE_BYTES);
      load_w(smem + (size_t)i * STAGE_BYTES, &full_bar[i], kof(i));
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i) load_x(smem + (size_t)i * STAGE_BYTES, &full_bar[i], kof(i));
    int s = pre == stages ? 0 : pre;
    uint32_t ph = pre == stages ? 1u : 0u;   // phase of the stage's next use
    for (int i = pre; i < n_kb; ++i) {
      if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, 1)) break;
      uint8_t* st = smem + (size_t)s * STAGE_BYTES;
      mbar_expect_tx(&full_bar[s], STAGE_BYTES);
      load_w(st, &full_bar[s], kof(i));
      load_x(st, &full_bar[s], kof(i));
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < n_kb && ok; ++i) {
      ok = mbar_wait(&full_bar[s], ph, abort_flag, 2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint64_t da = smem_desc_k128(sa);
      const uint64_t da2 = smem_desc_k128(sa + A_BYTES);
      const uint64_t db = smem_desc_k128(sa + B_OFF);
#pragma unroll
      for (int k = 0; k < KSTEP / UMMA_K; ++k) {
        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        // 32 bytes per step inside a sub-tile, then the next sub-tile
        const uint64_t adv_a = (uint64_t)((k >> 2) * (A_BYTES >> 4) + (k & 3) * 2);
        const uint64_t adv_b = (uint64_t)((k >> 2) * (B_BYTES >> 4) + (k & 3) * 2);
        umma_bf16(tmem_base, da + adv_a, db + adv_b, IDESC, acc);
        if (SWIGLU) umma_bf16(tmem_base + BN, da2 + adv_a, db + adv_b, IDESC, acc);
      }
      umma_commit(&empty_bar[s]);   // the stage is free once these instructions have read it
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    if (ok) umma_commit(acc_bar);
  } else if (warp < 4) {
    // ---- epilogue: thread = one weight row = one column of C
    pdl_wait();   // C may be read and written by earlier kernels
    TL_TRACE_RELEASED();
    if (splits > 1) {
      // What the reduction after the cluster barrier needs and the product does not: done now,
      // while the weights stream and these warps have nothing else to do.
      const int cols = min(BN, args.M - m0);
      if (args.ss_in) {   // 1/rms of every token: a warp per token, the partial sums spread over its lanes
        float* rinv_c = tail_rinv(smem + (size_t)stages * STAGE_BYTES);
        for (int c = warp; c < cols; c += 4) {
          float ss = 0.0f;
          for (int t = lane; t < args.ss_in_tiles; t += 32)
            ss += __ldcg(args.ss_in + (size_t)(m0 + c) * args.ss_in_tiles + t);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0) rinv_c[c] = 1.0f / sqrtf(ss / (float)args.norm_h + args.eps_in);
        }
      }
      if (args.rope_on && args.rope_inv_freq) {   // cosine and sine of every (token, pair of dimensions)
        float2* cs_t = tail_cossin(smem + (size_t)stages * STAGE_BYTES);
        const int half = args.rope_hd >> 1;
        for (int e = threadIdx.x; e < cols * half; e += 128) {
          const int c = e / half, i = e - c * half;
          float sn, cs;
          sincosf((float)args.rope_pos[m0 + c] * args.rope_inv_freq[i], &sn, &cs);
          cs_t[c * ROPE_TABLE_HALF + i] = make_float2(cs, sn);
        }
      }
    }
    const bool ok = mbar_wait(acc_bar, 0, abort_flag, 3);
    tc_fence_after();
    const int row = warp * 32 + lane;
    const int n = n0 + row;
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
    float* red = (float*)smem;   // partial tile [columns][128 rows]; the stages are free by now
    float* rinv_s = (float*)smem;   // without a split the same place holds the row scales
    if (ok && splits == 1 && args.ss_in) {
      for (int c = threadIdx.x; c < BN; c += 128)
        rinv_s[c] = m0 + c < args.M ? row_rinv(args, m0 + c) : 0.0f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (ok) {
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16], u[16];
        tmem_ld16(taddr + c0, r);
        if (SWIGLU) tmem_ld16(taddr + BN + c0, u);
        tmem_ld_wait();
        if (splits > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            red[(c0 + j) * TILE_N + row] = __uint_as_float(r[j]);
            if (SWIGLU) red[(BN + c0 + j) * TILE_N + row] = __uint_as_float(u[j]);
          }
        } else if (n < args.N) {
          float* cf = (float*)args.C + (size_t)(m0 + c0) * args.ldc + n;
          __nv_bfloat16* cb = (__nv_bfloat16*)args.C + (size_t)(m0 + c0) * args.ldc + n;
          const int valid = args.M - (m0 + c0);   // columns of this group that are real tokens
          if (args.mode == MODE_ACCUM_F32) {
            float prev[16];   // all loads first, so that they are in flight together
#pragma unroll
            for (int j = 0; j < 16; ++j) prev[j] = j < valid ? cf[(size_t)j * args.ldc] : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < valid) cf[(size_t)j * args.ldc] = prev[j] + __uint_as_float(r[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j >= valid) break;
              const float sc = args.ss_in ? rinv_s[c0 + j] : 1.0f;
              const float v = __uint_as_float(r[j]) * sc;
              if (SWIGLU) cb[(size_t)j * args.ldc] = __float2bfloat16_rn(silu_f(v) * (__uint_as_float(u[j]) * sc));
              else if (args.mode == MODE_STORE_F32) cf[(size_t)j * args.ldc] = v;
              else cb[(size_t)j * args.ldc] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
  }
  __syncwarp();
  if (splits > 1) {
    cluster_sync_all();   // every block's partial tile is in its shared memory
    if (warp < 4) {
      pdl_wait();
      const int row = warp * 32 + lane;
      const int n = n0 + row;
      const uint32_t red_s = smem_u32(smem);
      const int cols = min(BN, args.M - m0);
      const bool live = n < args.N && !*abort_flag;
      float* ssw = tail_ssw(smem + (size_t)stages * STAGE_BYTES);        // [4 warps][64] after the barriers
      const float* rinv_c = tail_rinv(smem + (size_t)stages * STAGE_BYTES);   // [BN] scales of the input rows,
      const float2* cs_t = tail_cossin(smem + (size_t)stages * STAGE_BYTES); // and the rotation's table: both written
      const int rank = (int)cluster_rank();                                 // before the cluster barrier above
      const bool accum = args.mode == MODE_ACCUM_F32 && !SWIGLU;
      int my_cols = 0;
      // Without the folded rotation: a warp takes one column (token) at a time, each lane four
      // consecutive rows of it, so that partial tiles come over in 16-byte loads and C goes out
      // in 16-byte (bfloat16: 8-byte) stores; two columns per turn keep more loads in flight.
      // The folded rotation goes the same way: a lane's four rows are four consecutive dimensions
      // of one head, their partners (half a head away, or the neighbour) are with another lane of
      // the warp or in the same four, and cosine and sine come from the table made above.
      const bool vec4 = (args.ldc & 3) == 0 && (args.N & 3) == 0 && ((uintptr_t)args.C & 15) == 0 &&
                        (!args.xw_out || ((uintptr_t)args.xw_out & 7) == 0) &&
                        (!args.rope_on || (((uintptr_t)args.rope_q | (uintptr_t)args.rope_k) & 7) == 0);
      if (vec4) {
        const int n4 = n0 + 4 * lane;
        const bool live4 = n4 < args.N && !*abort_flag;   // N is a multiple of 4: all four or none
        float nw4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (args.xw_out && live4) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            nw4[e] = args.nw_is_f32 ? ((const float*)args.nw)[n4 + e]
                                    : __bfloat162float(((const __nv_bfloat16*)args.nw)[n4 + e]);
        }
        // One turn of a warp: NC columns, the partial tiles of all splits requested before any is
        // added (a turn costs one round trip through the cluster's shared memory whatever it moves:
        // with two columns a turn, a tile of 64 tokens in two splits took four turns).  The number
        // of splits is a compile-time constant S where it is 2, 4 or 8 (S = 0: any other), so that
        // the loads sit in registers; the sums run in the order of the splits in every case.
        auto reduce_turns = [&](auto s_tag) {
        constexpr int S = decltype(s_tag)::value;
        constexpr int NC = S == 0 ? 2 : ((SWIGLU ? 8 : 16) / S);
        for (int k0 = warp; rank + k0 * splits < cols; k0 += 4 * NC) {
          float4 v[NC], u[NC], prev[NC];
          int cc[NC];
#pragma unroll
          for (int h = 0; h < NC; ++h) {
            const int c = rank + (k0 + 4 * h) * splits;
            cc[h] = c < cols ? c : -1;
            v[h] = u[h] = prev[h] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (cc[h] >= 0 && accum && live4)
              prev[h] = *reinterpret_cast<const float4*>((const float*)args.C + (size_t)(m0 + c) * args.ldc + n4);
          }
          if constexpr (S > 0) {
            float4 pa[NC][S], pb[SWIGLU ? NC : 1][SWIGLU ? S : 1];
#pragma unroll
            for (int h = 0; h < NC; ++h) {
#pragma unroll
              for (int sp = 0; sp < S; ++sp) {
                pa[h][sp] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (SWIGLU) pb[h][sp] = pa[h][sp];
                if (cc[h] < 0) continue;
                pa[h][sp] = ld_remote_f32x4(red_s + (uint32_t)(cc[h] * TILE_N + 4 * lane) * 4u, (uint32_t)sp);
                if (SWIGLU)
                  pb[h][sp] = ld_remote_f32x4(red_s + (uint32_t)((BN + cc[h]) * TILE_N + 4 * lane) * 4u, (uint32_t)sp);
              }
            }
#pragma unroll
            for (int h = 0; h < NC; ++h) {
#pragma unroll
              for (int sp = 0; sp < S; ++sp) {
                v[h].x += pa[h][sp].x; v[h].y += pa[h][sp].y; v[h].z += pa[h][sp].z; v[h].w += pa[h][sp].w;
                if (SWIGLU) { u[h].x += pb[h][sp].x; u[h].y += pb[h][sp].y; u[h].z += pb[h][sp].z; u[h].w += pb[h][sp].w; }
              }
            }
          } else {
#pragma unroll
            for (int h = 0; h < NC; ++h) {
              if (cc[h] < 0) continue;
              for (int sp = 0; sp < splits; ++sp) {
                const float4 a = ld_remote_f32x4(red_s + (uint32_t)(cc[h] * TILE_N + 4 * lane) * 4u, (uint32_t)sp);
                v[h].x += a.x; v[h].y += a.y; v[h].z += a.z; v[h].w += a.w;
                if (SWIGLU) {
                  const float4 b = ld_remote_f32x4(red_s + (uint32_t)((BN + cc[h]) * TILE_N + 4 * lane) * 4u, (uint32_t)sp);
                  u[h].x += b.x; u[h].y += b.y; u[h].z += b.z; u[h].w += b.w;
                }
              }
            }
          }
#pragma unroll
          for (int h = 0; h < NC; ++h) {
            if (cc[h] < 0) continue;
            const int c = cc[h];
            float val[4] = {v[h].x, v[h].y, v[h].z, v[h].w}, up[4] = {u[h].x, u[h].y, u[h].z, u[h].w};
            const float pv[4] = {prev[h].x, prev[h].y, prev[h].z, prev[h].w};
            if (args.ss_in) {
              const float sc = rinv_c[c];
#pragma unroll
              for (int e = 0; e < 4; ++e) { val[e] *= sc; up[e] *= sc; }
            }
            const size_t idx = (size_t)(m0 + c) * args.ldc + n4;
            float sq = 0.0f;
            if (!SWIGLU && args.rope_on) {
              // dimensions d .. d + 3 of head `head`; every lane takes part in the exchange
              const int hd = args.rope_hd, half = hd >> 1;
              const int head = n4 / hd, d = n4 - head * hd, m_tok = m0 + c;
              const bool turns = head < args.rope_nh + args.rope_nkv && args.rope_inv_freq != nullptr;
              float res[4] = {val[0], val[1], val[2], val[3]};
              if (args.rope_style == 0) {
                float other[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) other[e] = __shfl_xor_sync(0xffffffffu, val[e], hd >> 3);
                if (turns) {
                  const bool first = d < half;
                  const float2* t = cs_t + c * ROPE_TABLE_HALF + (first ? d : d - half);
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    res[e] = first ? val[e] * t[e].x - other[e] * t[e].y : other[e] * t[e].y + val[e] * t[e].x;
                }
              } else if (turns) {
                const float2* t = cs_t + c * ROPE_TABLE_HALF + (d >> 1);
                res[0] = val[0] * t[0].x - val[1] * t[0].y; res[1] = val[0] * t[0].y + val[1] * t[0].x;
                res[2] = val[2] * t[1].x - val[3] * t[1].y; res[3] = val[2] * t[1].y + val[3] * t[1].x;
              }
              if (live4) {
                uint2 o;
                o.x = pack_bf16x2(res[0], res[1]);
                o.y = pack_bf16x2(res[2], res[3]);
                if (head < args.rope_nh) {
                  *reinterpret_cast<uint2*>(args.rope_q + (size_t)m_tok * args.rope_nh * hd + n4) = o;
                } else {
                  const int pos = args.rope_pos[m_tok];
                  const int page = args.rope_table[(size_t)args.rope_slot[args.rope_seq[m_tok]] * args.rope_table_stride +
                                                   pos / TL_PAGE];
                  if (page >= 0) {
                    const bool is_k = head < args.rope_nh + args.rope_nkv;
                    const int kvh = head - args.rope_nh - (is_k ? 0 : args.rope_nkv);
                    const size_t base = ((size_t)page * args.rope_nkv + kvh) * (size_t)(TL_PAGE * hd);
                    if (is_k) {
                      *reinterpret_cast<uint2*>(args.rope_k + base + (size_t)(pos % TL_PAGE) * hd + d) = o;
                    } else {
#pragma unroll
                      for (int e = 0; e < 4; ++e)
                        args.rope_v[base + (size_t)(d + e) * TL_PAGE + (pos % TL_PAGE)] = __float2bfloat16_rn(res[e]);
                    }
                  }
                }
              }
            } else if (live4) {
              if (SWIGLU) {
                uint2 o;
                o.x = pack_bf16x2(silu_f(val[0]) * up[0], silu_f(val[1]) * up[1]);
                o.y = pack_bf16x2(silu_f(val[2]) * up[2], silu_f(val[3]) * up[3]);
                *reinterpret_cast<uint2*>((__nv_bfloat16*)args.C + idx) = o;
              } else if (args.mode == MODE_STORE_F32) {
                *reinterpret_cast<float4*>((float*)args.C + idx) = make_float4(val[0], val[1], val[2], val[3]);
              } else if (accum) {
                float cn[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) cn[e] = pv[e] + val[e];
                *reinterpret_cast<float4*>((float*)args.C + idx) = make_float4(cn[0], cn[1], cn[2], cn[3]);
                if (args.xw_out) {
                  uint2 o;
                  o.x = pack_bf16x2(cn[0] * nw4[0], cn[1] * nw4[1]);
                  o.y = pack_bf16x2(cn[2] * nw4[2], cn[3] * nw4[3]);
                  *reinterpret_cast<uint2*>(args.xw_out + (size_t)(m0 + c) * args.N + n4) = o;
                  sq = (cn[0] * cn[0] + cn[1] * cn[1]) + (cn[2] * cn[2] + cn[3] * cn[3]);
                }
              } else {
                uint2 o;
                o.x = pack_bf16x2(val[0], val[1]);
                o.y = pack_bf16x2(val[2], val[3]);
                *reinterpret_cast<uint2*>((__nv_bfloat16*)args.C + idx) = o;
              }
            }
            if (args.xw_out) {   // the tile's 128 rows of this column lie in this one warp
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
              if (lane == 0) args.ss_out[(size_t)(m0 + c) * gridDim.x + blockIdx.x] = sq;
            }
          }
        }
        };
        // Only for token tiles of 64 and more, where a block has many columns to reduce: the loads
        // in flight cost some 40 registers, and with 121 instead of 80 registers a block of the
        // next kernel no longer fits beside two of this one (a decode step at batch 8 took 3.63
        // instead of 3.57 ms when the tiles of 16 tokens were compiled this way too).
        if constexpr (BN >= 64) {
          if (splits == 8) reduce_turns(std::integral_constant<int, 8>{});
          else if (splits == 4) reduce_turns(std::integral_constant<int, 4>{});
          else if (splits == 2) reduce_turns(std::integral_constant<int, 2>{});
          else reduce_turns(std::integral_constant<int, 0>{});
        } else {
          reduce_turns(std::integral_constant<int, 0>{});
        }
      } else {
      // columns rank, rank + splits, ... in groups of 8, so that the loads of a group (old C,
      // partials of every split) are in flight together
      for (int cb = rank; cb < cols; cb += 8 * splits) {
        float v[8], uu[8], prev[8];
        // with the rotation folded in, `uu` holds the partner of the pair (same token, the
        // column that turns together with this one)
        const int rope_half = args.rope_hd >> 1;
        const int prow = args.rope_on ? (args.rope_style == 0 ? (row ^ rope_half) : (row ^ 1)) : row;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int c = cb + q * splits;
          prev[q] = (accum && live && c < cols) ? ((const float*)args.C)[(size_t)(m0 + c) * args.ldc + n] : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int c = cb + q * splits;
          v[q] = uu[q] = 0.0f;
          if (c < cols) {
            for (int sp = 0; sp < splits; ++sp) {
              v[q] += ld_remote_f32(red_s + (uint32_t)(c * TILE_N + row) * 4u, (uint32_t)sp);
              if (SWIGLU) uu[q] += ld_remote_f32(red_s + (uint32_t)((BN + c) * TILE_N + row) * 4u, (uint32_t)sp);
              else if (args.rope_on) uu[q] += ld_remote_f32(red_s + (uint32_t)(c * TILE_N + prow) * 4u, (uint32_t)sp);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int c = cb + q * splits;
          if (c >= cols) break;
          float val = v[q], up = uu[q];
          if (args.ss_in) { val *= rinv_c[c]; up *= rinv_c[c]; }   // `up` may be the rotation partner
          const size_t idx = (size_t)(m0 + c) * args.ldc + n;
          float sq = 0.0f;
          if (live) {
            if (SWIGLU) ((__nv_bfloat16*)args.C)[idx] = __float2bfloat16_rn(silu_f(val) * up);
            else if (args.rope_on) {
              // this column is dimension d of head `head`; rotate q and k at the token's position
              // (angle, sine and cosine in 32-bit) and write q, or k and v into the token's page
              const int hd = args.rope_hd, head = n / hd, d = n - head * hd, m_tok = m0 + c;
              const int pos = args.rope_pos[m_tok];
              float res = val;
              if (head < args.rope_nh + args.rope_nkv && args.rope_inv_freq) {
                const bool first = args.rope_style == 0 ? d < rope_half : (d & 1) == 0;
                const int i = args.rope_style == 0 ? (first ? d : d - rope_half) : d >> 1;
                float sn, cs;
                sincosf((float)pos * args.rope_inv_freq[i], &sn, &cs);
                res = first ? val * cs - up * sn : up * sn + val * cs;
              }
              if (head < args.rope_nh) {
                args.rope_q[(size_t)m_tok * args.rope_nh * hd + n] = __float2bfloat16_rn(res);
              } else {
                const int page = args.rope_table[(size_t)args.rope_slot[args.rope_seq[m_tok]] * args.rope_table_stride +
                                                 pos / TL_PAGE];
                if (page >= 0) {
                  const bool is_k = head < args.rope_nh + args.rope_nkv;
                  const int kvh = head - args.rope_nh - (is_k ? 0 : args.rope_nkv);
                  const size_t base = ((size_t)page * args.rope_nkv + kvh) * (size_t)(TL_PAGE * hd);
                  if (is_k) args.rope_k[base + (size_t)(pos % TL_PAGE) * hd + d] = __float2bfloat16_rn(res);
                  else args.rope_v[base + (size_t)d * TL_PAGE + (pos % TL_PAGE)] = __float2bfloat16_rn(res);
                }
              }
            }
            else if (args.mode == MODE_STORE_F32) ((float*)args.C)[idx] = val;
            else if (accum) {
              const float cn = prev[q] + val;
              ((float*)args.C)[idx] = cn;
              if (args.xw_out) {
                const float w = args.nw_is_f32 ? ((const float*)args.nw)[n]
                                               : __bfloat162float(((const __nv_bfloat16*)args.nw)[n]);
                args.xw_out[(size_t)(m0 + c) * args.N + n] = __float2bfloat16_rn(cn * w);
                sq = cn * cn;
              }
            } else ((__nv_bfloat16*)args.C)[idx] = __float2bfloat16_rn(val);
          }
          if (args.xw_out) {   // sum of squares of this tile's 128 columns, in a fixed order
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) ssw[warp * 64 + my_cols] = sq;
          }
          ++my_cols;
        }
      }
      if (args.xw_out) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if ((int)threadIdx.x < my_cols) {
          const int c = rank + (int)threadIdx.x * splits;
          const float t = ((ssw[threadIdx.x] + ssw[64 + threadIdx.x]) + ssw[128 + threadIdx.x]) + ssw[192 + threadIdx.x];
          args.ss_out[(size_t)(m0 + c) * gridDim.x + blockIdx.x] = t;
        }
      }
      }
    }
    cluster_sync_all();   // nobody leaves while others still read its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// The persistent kernel for many tokens (no K split).  One block per SM walks over output
// tiles; the accumulator is double-buffered in tensor memory, so the four epilogue warps
// write tile i while the issuing thread already runs the instructions of tile i + 1, and
// the TMA ring runs on across tile borders.  Tiles are numbered with the token tile
// fastest, so that blocks running at the same time share weight tiles in L2.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tm_w,
                          const __grid_constant__ CUtensorMap tm_x, const GemmArgs args,
                          int m_tiles, int total_tiles) {
  constexpr uint32_t A_BYTES = TILE_N * TILE_K * 2;
  constexpr uint32_t B_BYTES = BN * TILE_K * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES * (SWIGLU ? 2 : 1) + B_BYTES;
  constexpr uint32_t ACC_COLS = BN * (SWIGLU ? 2 : 1);
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;   // two accumulators; 256 or 512 columns
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "two accumulators must fill a power of two");
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(TILE_N >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + 8;
  uint64_t* acc_full = empty_bar + 8;    // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (args.K + TILE_K - 1) / TILE_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 4 && lane == 0) {
    // ---- TMA producer: one ring of stages across all tiles of this block
    bool waited = false;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int n0 = (tile / m_tiles) * TILE_N, m0 = (tile % m_tiles) * BN;
      for (int kb = 0; kb < kb_total; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, 1)) { tile = total_tiles; break; }
        uint8_t* st = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        const int k = kb * TILE_K;
        tma_load_2d(st, &tm_w, &full_bar[s], k, n0);
        if (SWIGLU) tma_load_2d(st + A_BYTES, &tm_w, &full_bar[s], k, args.N + n0);
        if (!waited) { pdl_wait(); waited = true; }   // weights first, activations after the wait
        tma_load_2d(st + A_BYTES * (SWIGLU ? 2 : 1), &tm_x, &full_bar[s], k, m0);
      }
    }
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer
    uint32_t it = 0, local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const uint32_t buf = local & 1u;
      ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1u) ^ 1u, abort_flag, 4);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * ACC_COLS;
      for (int kb = 0; kb < kb_total; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1u;
        ok = mbar_wait(&full_bar[s], ph, abort_flag, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t da = smem_desc_k128(sa);
        const uint64_t da2 = smem_desc_k128(sa + A_BYTES);
        const uint64_t db = smem_desc_k128(sa + A_BYTES * (SWIGLU ? 2 : 1));
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
          const uint64_t adv = (uint64_t)(k * UMMA_K * 2 >> 4);
          umma_bf16(acc, da + adv, db + adv, IDESC, accum);
          if (SWIGLU) umma_bf16(acc + BN, da2 + adv, db + adv, IDESC, accum);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&acc_full[buf]);
    }
  } else if (warp < 4) {
    // ---- epilogue: thread = one weight row = one column of C
    pdl_wait();
    const int row = warp * 32 + lane;
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int n0 = (tile / m_tiles) * TILE_N, m0 = (tile % m_tiles) * BN;
      const int n = n0 + row;
      const uint32_t buf = local & 1u;
      if (!mbar_wait(&acc_full[buf], (local >> 1) & 1u, abort_flag, 3)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * ACC_COLS;
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16], u[16];
        tmem_ld16(taddr + c0, r);
        if (SWIGLU) tmem_ld16(taddr + BN + c0, u);
        tmem_ld_wait();
        if (n < args.N) {
          float* cf = (float*)args.C + (size_t)(m0 + c0) * args.ldc + n;
          __nv_bfloat16* cb = (__nv_bfloat16*)args.C + (size_t)(m0 + c0) * args.ldc + n;
          const int valid = args.M - (m0 + c0);
          if (args.mode == MODE_ACCUM_F32) {
            float prev[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) prev[j] = j < valid ? cf[(size_t)j * args.ldc] : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < valid) cf[(size_t)j * args.ldc] = prev[j] + __uint_as_float(r[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j >= valid) break;
              const float v = __uint_as_float(r[j]);
              if (SWIGLU) cb[(size_t)j * args.ldc] = __float2bfloat16_rn(silu_f(v) * __uint_as_float(u[j]));
              else if (args.mode == MODE_STORE_F32) cf[(size_t)j * args.ldc] = v;
              else cb[(size_t)j * args.ldc] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);   // 128 arrivals free the accumulator for tile i + 2
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// The persistent kernel on pairs of SMs (tcgen05 with cta_group::2).  The two blocks of a
// cluster share one instruction of 256 weight rows x 256 tokens: each block holds 128 of
// the weight rows and 128 of the tokens in its shared memory and 128 rows of the
// accumulator in its tensor memory, so a block fetches 32 KB per 64 K-elements where the
// one-SM kernel fetches 48 KB.  A stage holds 128 K-elements (64 KB, three stages).  The first block of
// the pair issues the instructions; the barrier that says "stage filled" lives there and
// counts the bytes of both blocks' TMA loads; the instruction's completion is signalled
// to the "stage free" and "accumulator ready" barriers of both blocks at once.
//
// SiLU-gate mode: a block's 128 operand rows are 64 gate rows followed by the 64 up rows
// of the same output columns, so one accumulator serves both; the epilogue threads of the
// gate half and of the up half exchange half of their values through shared memory and
// each write half of the tokens.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_saddr, uint32_t rank) {
  uint32_t raddr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_saddr), "r"(rank));
  return raddr;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA load whose bytes are counted by a barrier of either block of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival at the barrier of the same place in both blocks of the pair, when all
// instructions issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
// All 128 epilogue threads learn whether every one of them passed its wait.
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok)
      : "memory");
  return r != 0;
}

#define PAIR_BN 256       // most tokens per pair tile; a launch picks a multiple of 32 up to this
#define PAIR_K 128        // K elements per stage: two 64-element (128-byte) sub-tiles per operand, so that the
                          // issuing thread's fixed cost per stage (barrier wait, commit, loop) is paid half as often
#define PAIR_SUB 16384    // bytes of one sub-tile slot: 128 rows of 128 bytes
#define PAIR_STAGE 65536  // bytes per stage and block: [A k0][A k1][B k0][B k1]
#define PAIR_XCHG 8192    // SiLU-gate exchange: two buffers of 2 x 8 x 64 floats
#define PAIR_MAX_BLOCKS 160

// A product with fewer tiles than pairs splits K over `splits` pairs per tile, all running
// at once.  The pair with the first K-blocks writes C; the others leave their partial tiles
// here, one slot per block, and raise the block's flag; the writer adds them in split order
// (the same bits every run) and lowers the flags again.
__device__ float tl_pair_partial[PAIR_MAX_BLOCKS * 128 * PAIR_BN];
__device__ unsigned int tl_pair_flag[PAIR_MAX_BLOCKS];

// Which tile a pair takes next.  raster 0: all token tiles of one strip of weight rows, then the next strip.
// raster g > 0: strips in groups of g; inside a group all strips of one token tile, then the next token tile
// (a wave of pairs then shares g strips of weights and pairs / g token tiles instead of one or two strips and
// every token tile).
__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int raster, int& tn, int& tm) {
  if (raster <= 0) { tn = tile / m_tiles; tm = tile % m_tiles; return; }
  const int per_group = raster * m_tiles;
  const int g = tile / per_group, r = tile - g * per_group;
  const int width = min(raster, n_tiles - g * raster);   // the last group may be narrower
  tm = r / width;
  tn = g * raster + r % width;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_x, const GemmArgs args, int m_tiles,
                    int total_tiles, int splits, int bn) {
  constexpr uint32_t ACC_COLS = PAIR_BN;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
  constexpr int PAIR_N = SWIGLU ? 128 : 256;   // output columns per pair tile
  // tokens per tile `bn`: the N of the instruction; each block holds bn / 2 token rows
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) |
                         ((uint32_t)(256 >> 4) << 24);
  const uint32_t stage_tx = 2u * 2u * (PAIR_SUB + (uint32_t)bn * 64u);   // bytes both blocks load per stage

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * PAIR_STAGE);
  uint64_t* empty_bar = full_bar + 8;
  uint64_t* acc_full = empty_bar + 8;    // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* xchg = (float*)(smem + (size_t)stages * PAIR_STAGE + 2048);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (args.K + PAIR_K - 1) / PAIR_K;
  const uint32_t rank = cluster_rank();          // 0 issues the instructions
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  // work item = (tile, split); with splits > 1 the grid holds every item at once
  const int total_items = total_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 256); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  cluster_sync_all();   // both blocks' barriers exist before either touches the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 4 && lane == 0) {
    // ---- TMA producer of this block's halves; the bytes count at the first block's barrier
    bool waited = false;
    int s = 0;
    uint32_t ph = 0;
    for (int item = pair; item < total_items; item += n_pairs) {
      const int tile = item / splits, split = item % splits;
      int tn, tm;
      pair_tile_coords(tile, m_tiles, total_tiles / m_tiles, args.raster, tn, tm);
      const int n0 = tn * PAIR_N, m0 = tm * bn;
      const int kb_b = split * args.kb_per_split, kb_e = min(kb_total, kb_b + args.kb_per_split);
      for (int kb = kb_b; kb < kb_e; ++kb) {
        // (walking each tile's K range from another start, as the few-token kernel does, costs 5 % here:
        // tiles of one wave then no longer meet on the same weights and activations in the L2 cache)
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, 1)) { item = total_items; break; }
        uint8_t* st = smem + (size_t)s * PAIR_STAGE;
        if (rank == 0) mbar_expect_tx(&full_bar[s], stage_tx);
        const uint32_t bar = mapa_u32(smem_u32(&full_bar[s]), 0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // the two 64-element halves of the stage's K range (past K: zeros)
          const int k = kb * PAIR_K + h * TILE_K;
          if (SWIGLU) {
            tma_load_2d_pair(st + h * PAIR_SUB, &tm_w, bar, k, n0 + 64 * (int)rank);
            tma_load_2d_pair(st + h * PAIR_SUB + PAIR_SUB / 2, &tm_w, bar, k, args.N + n0 + 64 * (int)rank);
          } else {
            tma_load_2d_pair(st + h * PAIR_SUB, &tm_w, bar, k, n0 + 128 * (int)rank);
          }
        }
        if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_2d_pair(st + (2 + h) * PAIR_SUB, &tm_x, bar, kb * PAIR_K + h * TILE_K, m0 + (bn >> 1) * (int)rank);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 5 && lane == 0 && rank == 0) {
    // ---- MMA issuer of the pair
    uint32_t local = 0, ph = 0;
    int s = 0;
    bool ok = true;
    for (int item = pair; item < total_items && ok; item += n_pairs, ++local) {
      const int split = item % splits;
      const int kb_b = split * args.kb_per_split, kb_e = min(kb_total, kb_b + args.kb_per_split);
      const uint32_t buf = local & 1u;
      ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1u) ^ 1u, abort_flag, 4);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * ACC_COLS;
      for (int kb = kb_b; kb < kb_e; ++kb) {
        ok = mbar_wait(&full_bar[s], ph, abort_flag, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * PAIR_STAGE);
        const uint64_t da = smem_desc_k128(sa);
        const uint64_t db = smem_desc_k128(sa + 2 * PAIR_SUB);
#pragma unroll
        for (int k = 0; k < PAIR_K / UMMA_K; ++k) {
          // 32 bytes per step inside a sub-tile, then the next sub-tile
          const uint64_t adv = (uint64_t)((k >> 2) * (PAIR_SUB >> 4) + (k & 3) * 2);
          umma_bf16_pair(acc, da + adv, db + adv, idesc, (kb > kb_b || k > 0) ? 1u : 0u);
        }
        umma_commit_pair(&empty_bar[s]);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok) umma_commit_pair(&acc_full[buf]);
    }
  } else if (warp < 4) {
    // ---- epilogue of this block's 128 accumulator rows
    pdl_wait();
    const int row = warp * 32 + lane;
    const uint32_t acc_empty_leader = mapa_u32(smem_u32(&acc_empty[0]), 0);
    float* my_partial = tl_pair_partial + (size_t)blockIdx.x * (128 * PAIR_BN) + row;
    uint32_t local = 0;
    for (int item = pair; item < total_items; item += n_pairs, ++local) {
      const int tile = item / splits, split = item % splits;
      int tn, tm;
      pair_tile_coords(tile, m_tiles, total_tiles / m_tiles, args.raster, tn, tm);
      const int n0 = tn * PAIR_N, m0 = tm * bn;
      const uint32_t buf = local & 1u;
      const bool merge = splits > 1 && split == 0;   // this pair writes C
      bool ok = mbar_wait(&acc_full[buf], (local >> 1) & 1u, abort_flag, 3);
      if (merge && ok && threadIdx.x < (unsigned)(splits - 1)) {
        // thread j waits for the partial tile of split j + 1 (same rank, two blocks further each)
        ok = false;
        for (uint32_t i = 0; i < TL_WAIT_LIMIT && !ok; ++i) {
          unsigned int f;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];"
                       : "=r"(f) : "l"(&tl_pair_flag[blockIdx.x + 2 * (threadIdx.x + 1)]) : "memory");
          ok = f != 0;
          if (!ok) __nanosleep(64);
        }
        if (!ok) { *abort_flag = 5; atomicCAS(&tl_gemm_tc_error, 0, 5); }
      }
      if (!epilogue_all(ok)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * ACC_COLS;
      if (split > 0) {
        for (int c0 = 0; c0 < bn; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) my_partial[(c0 + j) * 128] = __uint_as_float(r[j]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0)
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&tl_pair_flag[blockIdx.x]), "r"(1u) : "memory");
      } else if (SWIGLU) {
        // rows 0-63 hold the gate, rows 64-127 the up value of column n; the gate half
        // writes tokens 0-7 of each 16, the up half tokens 8-15
        const int col = row & 63, up_half = row >> 6;
        const int n = n0 + 64 * (int)rank + col;
        for (int c0 = 0, i = 0; c0 < bn; c0 += 16, ++i) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (merge) {
            for (int sp = 1; sp < splits; ++sp) {
              const float* part = my_partial + (size_t)(2 * sp) * (128 * PAIR_BN) + c0 * 128;
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(part + j * 128));
            }
          }
          float* mine = xchg + (i & 1) * 1024 + (up_half ? 512 : 0);     // what I give away
          float* theirs = xchg + (i & 1) * 1024 + (up_half ? 0 : 512);   // what I get
#pragma unroll
          for (int j = 0; j < 8; ++j) mine[j * 64 + col] = __uint_as_float(r[up_half ? j : 8 + j]);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (n < args.N) {
            const int t0 = m0 + c0 + (up_half ? 8 : 0);
            __nv_bfloat16* cb = (__nv_bfloat16*)args.C + (size_t)t0 * args.ldc + n;
            const int valid = args.M - t0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (j >= valid) break;
              const float other = theirs[j * 64 + col];
              const float g = up_half ? other : __uint_as_float(r[j]);
              const float u = up_half ? __uint_as_float(r[8 + j]) : other;
              cb[(size_t)j * args.ldc] = __float2bfloat16_rn(silu_f(g) * u);
            }
          }
        }
      } else if (args.mode == MODE_ACCUM_F32) {
        // 64 values of C are fetched at once: four round trips to memory per tile, which
        // matters for the last tile, whose epilogue nothing hides
        const int n = n0 + 128 * (int)rank + row;
        for (int c0 = 0; c0 < bn; c0 += 64) {
          float prev[64];
          float* cf = (float*)args.C + (size_t)(m0 + c0) * args.ldc + n;
          const int valid = min(args.M - (m0 + c0), bn - c0);   // the tile's own tokens only
#pragma unroll
          for (int j = 0; j < 64; ++j) prev[j] = (n < args.N && j < valid) ? cf[(size_t)j * args.ldc] : 0.0f;
          float part[64];   // the other splits' sums, added in split order, then to the accumulator
#pragma unroll
          for (int j = 0; j < 64; ++j) part[j] = 0.0f;
          if (merge) {
            for (int sp = 1; sp < splits; ++sp) {
              const float* src = my_partial + (size_t)(2 * sp) * (128 * PAIR_BN) + c0 * 128;
#pragma unroll
              for (int j = 0; j < 64; ++j) part[j] += __ldcg(src + j * 128);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t r[16];
            tmem_ld16(taddr + c0 + 16 * q, r);
            tmem_ld_wait();
            if (n < args.N) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (16 * q + j < valid)
                  cf[(size_t)(16 * q + j) * args.ldc] = prev[16 * q + j] + (__uint_as_float(r[j]) + part[16 * q + j]);
            }
          }
        }
      } else {
        const int n = n0 + 128 * (int)rank + row;
        for (int c0 = 0; c0 < bn; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (merge) {
            for (int sp = 1; sp < splits; ++sp) {
              const float* part = my_partial + (size_t)(2 * sp) * (128 * PAIR_BN) + c0 * 128;
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(part + j * 128));
            }
          }
          if (n < args.N) {
            float* cf = (float*)args.C + (size_t)(m0 + c0) * args.ldc + n;
            __nv_bfloat16* cb = (__nv_bfloat16*)args.C + (size_t)(m0 + c0) * args.ldc + n;
            const int valid = args.M - (m0 + c0);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j >= valid) break;
              const float v = __uint_as_float(r[j]);
              if (args.mode == MODE_STORE_F32) cf[(size_t)j * args.ldc] = v;
              else cb[(size_t)j * args.ldc] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      if (merge) {   // every thread has read the partial tiles: their flags go back to 0
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x < (unsigned)(splits - 1))
          asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&tl_pair_flag[blockIdx.x + 2 * (threadIdx.x + 1)]), "r"(0u) : "memory");
      }
      tc_fence_before();
      mbar_arrive_cluster(acc_empty_leader + 8 * buf);   // 256 arrivals free the accumulator
    }
  }
  __syncwarp();
  tc_fence_before();
  cluster_sync_all();   // neither block leaves, nor frees tensor memory, while the other works
  if (warp == 0) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Host side: tensor maps (cached), tile and split choice, launch.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// [rows, K] bfloat16, row stride ld elements; boxes of 64 K-elements x box_rows rows.
static bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld,
                     int box_rows) {
  typedef std::tuple<const void*, long long, long long, long long, int> Key;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key(ptr, rows, K, ld, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) { *map = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = m;
  *map = m;
  return true;
}

template <int BN, bool SWIGLU>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, GemmArgs a, int splits,
                  size_t smem_budget, cudaStream_t stream) {
  const size_t stage = (SWIGLU ? 1 : 2) * ((size_t)TILE_N * TILE_K * 2 * (SWIGLU ? 2 : 1) + (size_t)BN * TILE_K * 2);
  const size_t tail = TAIL_BYTES + ((BN == 16 && !SWIGLU) ? TAIL_ROPE_BYTES : 0);
  int stages = (int)((smem_budget - 1024 - tail) / stage);
  stages = stages > 8 ? 8 : stages;
  if (stages < 2) return -2;
  a.stages = stages;
  const size_t smem = 1024 + stages * stage + tail;
  static size_t configured = 0;   // per instantiation
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWIGLU>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + TILE_N - 1) / TILE_N, (a.M + BN - 1) / BN, splits);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;   // the splits of one tile share their partials
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, SWIGLU>, tw, tx, a);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int BN, bool SWIGLU>
static int launch_persistent(const CUtensorMap& tw, const CUtensorMap& tx, GemmArgs a, int num_sms,
                             cudaStream_t stream) {
  const size_t stage = (size_t)TILE_N * TILE_K * 2 * (SWIGLU ? 2 : 1) + (size_t)BN * TILE_K * 2;
  int stages = (int)((224 * 1024 - 1024 - 2048) / stage);
  stages = stages > 8 ? 8 : stages;
  if (stages < 2) return -2;
  a.stages = stages;
  const size_t smem = 1024 + stages * stage + 2048;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, SWIGLU>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const int m_tiles = (a.M + BN - 1) / BN;
  const int total = m_tiles * ((a.N + TILE_N - 1) / TILE_N);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(total < num_sms ? total : num_sms);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_persistent_kernel<BN, SWIGLU>, tw, tx, a, m_tiles, total);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// The pair kernel: clusters of two blocks, as many as the GPU holds at once.
template <bool SWIGLU>
static int launch_pair(const CUtensorMap& tw, const CUtensorMap& tx, GemmArgs a, int want_splits, int bn,
                       cudaStream_t stream) {
  const int stages = 3;
  a.stages = stages;
  const size_t smem = 1024 + (size_t)stages * PAIR_STAGE + 2048 + PAIR_XCHG;
  const int m_tiles = (a.M + bn - 1) / bn;
  const int pair_n = SWIGLU ? 128 : 256;
  const int total = m_tiles * ((a.N + pair_n - 1) / pair_n);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  static int max_pairs = -1;   // per instantiation
  if (max_pairs < 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<SWIGLU>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3(2);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<SWIGLU>, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    max_pairs = n < PAIR_MAX_BLOCKS / 2 ? n : PAIR_MAX_BLOCKS / 2;
  }
  if (max_pairs <= 0) return -2;
  // K split over several pairs per tile only while every (tile, split) runs at once
  const int kb_total = (a.K + PAIR_K - 1) / PAIR_K;
  int splits = want_splits;
  while (splits > 1 && (long long)total * splits > max_pairs) --splits;
  a.kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + a.kb_per_split - 1) / a.kb_per_split;   // no empty split
  const int items = total * splits;
  cfg.gridDim = dim3(2 * (items < max_pairs ? items : max_pairs));
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<SWIGLU>, tw, tx, a, m_tiles, total, splits, bn);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

#define MAX_SPLITS 8   // portable cluster size

// How many clusters of `s` blocks of the few-token kernel the GPU is sure to hold at once: what the
// occupancy calculation grants at one block per SM (which is what it answers for kernels that take
// tensor memory), twice that where two blocks share an SM.  The GPCs differ in size, so this is not
// slots / s: at two blocks per SM this pool's B200 holds 46 clusters of 6 but 39 of 7 and 35 of 8.
// -1 if the calculation fails.
template <int BN, bool SWIGLU>
static int clusters_at_once_of(int s, size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, s);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(gemm_tc_kernel<BN, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess) { cudaGetLastError(); return -1; }
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN, SWIGLU>, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
  return n;
}
static int clusters_at_once(int bn, bool swiglu, int s, size_t smem, int per_sm) {
  static int known[5][2][MAX_SPLITS + 1];   // token tiles of 16, 32, 64, 128, 256; 0 = not asked yet
  static std::mutex mu;
  const int bi = bn == 16 ? 0 : bn == 32 ? 1 : bn == 64 ? 2 : bn == 128 ? 3 : 4;
  std::lock_guard<std::mutex> lock(mu);
  int& v = known[bi][swiglu ? 1 : 0][s];
  if (v == 0) {
    int n = -1;
#define ASK(BN_) n = swiglu ? clusters_at_once_of<BN_, true>(s, smem) : clusters_at_once_of<BN_, false>(s, smem)
    switch (bn) {
      case 16: ASK(16); break;
      case 32: ASK(32); break;
      case 64: ASK(64); break;
      case 128: ASK(128); break;
      default: ASK(256); break;
    }
#undef ASK
    v = n <= 0 ? -1 : n;
  }
  return v < 0 ? v : v * per_sm;
}

// What the caller passes to have rotation and cache write done by the q/k/v product.
struct TlRopeArgs {
  void* q_out; void* k_pages; void* v_pages;
  const int* token_pos; const int* token_seq; const int* seq_slot; const int* page_table;
  const float* inv_freq;
  int table_stride, style, nh, nkv, hd;
};

// Returns 0, a CUDA error, or -2 when these sizes or alignments are not taken (the
// caller then uses the CUDA-core kernel).  N counts output columns; in mode 2 W has 2N rows.
//
// A norm between two products can be folded into them.  Producer side (mode 1 only): if
// `xw_out` is given and K is split, the kernel also writes xw_out[m, n] = bf16(C_new[m, n] *
// nw[n]) and ss_out[m, tile] = the sum of C_new[m, n]^2 over the tile's 128 columns, and
// sets *emitted = 1; otherwise *emitted = 0 and the caller runs the norm kernel.  Consumer
// side: with `ss_in` given, X is such an xw and every output is scaled by
// 1 / sqrt(sum_t ss_in[m, t] / norm_h + eps_in) before the mode's operation.
//
// `rope` (a TlRopeArgs, mode 0, K split only): C is not written; instead the columns, read as
// query, key and value heads, are rotated at each token's position and written to q_out and
// into the token's cache page, and *rope_applied = 1.  Otherwise *rope_applied = 0 and the
// caller runs the rotation kernel on C.
extern "C" int tl_gemm_tc(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, int M,
                          int N, int K, int mode, int num_sms, const float* ss_in, int ss_in_tiles,
                          int norm_h, float eps_in, void* xw_out, const void* nw, int nw_is_f32,
                          float* ss_out, int* emitted, const void* rope, int* rope_applied,
                          cudaStream_t stream) {
  if (emitted) *emitted = 0;
  if (rope_applied) *rope_applied = 0;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
    return -2;
  if (mode < 0 || mode > 3) return -1;
  const bool swiglu = mode == MODE_SWIGLU;
  int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const int n_tiles = (N + TILE_N - 1) / TILE_N, m_tiles = (M + bn - 1) / bn;
  const long long tiles = (long long)n_tiles * m_tiles;
  const int kb_total = (K + TILE_K - 1) / TILE_K;
  // stages of the few-token kernel: 128 K-elements, 64 with the SiLU-gate's two matrices
  const int kstep64 = swiglu ? 1 : 2;
  const int kb_np = (K + TILE_K * kstep64 - 1) / (TILE_K * kstep64);
  // two blocks per SM fit while the token tile is small
  const bool two_per_sm = bn <= 64;
  // small token tiles leave room for the blocks of the next kernel, which fetch their first
  // weight tiles while this kernel drains
  const size_t budget = !two_per_sm ? 224 * 1024 : (!swiglu && bn <= 32) ? 88 * 1024 : 112 * 1024;
  const long long slots = (long long)num_sms * (two_per_sm ? 2 : 1);
  int splits = 1;
  if (tiles < slots && (two_per_sm || !ss_in)) {
    // a power of two (clusters of 3, 5, 6 or 7 blocks do not tile the GPCs evenly, and a
    // cluster that has to wait for a second wave doubles the kernel's time), as large as
    // keeps every block resident at once
    while (splits * 2 <= MAX_SPLITS && tiles * splits * 2 <= slots && splits * 2 <= kb_np / 2)
      splits *= 2;
    // 3, 5, 6 or 7 splits where that puts more blocks on the GPU and all their clusters are sure to run
    // at once (measured at 8 tokens: 5120 x 14336 in 6 splits 26.0 us, in 4 splits 28.9 us, in 7, which
    // do not all fit, 36.6 us; 6144 x 5120 in 5 splits 12.5 us, in 4 splits 13.5 us, in 6 19.5 us)
    if (m_tiles == 1) {
      for (int sp = MAX_SPLITS - 1; sp > splits; --sp) {
        if ((sp & (sp - 1)) == 0 || tiles * sp > slots || sp > kb_np / 2) continue;
        if (tiles <= clusters_at_once(bn, swiglu, sp, budget, two_per_sm ? 2 : 1)) { splits = sp; break; }
      }
    }
    // token tiles of 128: the reduction of so wide a tile costs about as much as 16 K-blocks of 64
    // elements (measured: q/k/v at 128 tokens 19.0 us unsplit, 17.0 us in two splits), so the split has
    // to save more than that
    if (!two_per_sm && ((kb_np + splits - 1) / splits) * kstep64 + 16 >= kb_total) splits = 1;
  }
  int kb_per_split = (kb_np + splits - 1) / splits;
  splits = (kb_np + kb_per_split - 1) / kb_per_split;   // no empty split
  const int pairs = num_sms / 2;
  const int pair_n = swiglu ? 128 : 256;
  // token tiles of equal width, a multiple of 32 (300 tokens: two tiles of 160, not 256 + 44)
  const int pair_m_tiles = (M + PAIR_BN - 1) / PAIR_BN;
  const int pair_bn = ((M + pair_m_tiles - 1) / pair_m_tiles + 31) / 32 * 32;
  const long long tiles_p = (long long)((N + pair_n - 1) / pair_n) * pair_m_tiles;
  // K split over idle pairs: the merge of s partial tiles costs about 16 + 24 (s - 1)
  // K-blocks' time (measured)
  int pair_splits = 1;
  if (pairs > 0 && tiles_p * 2 <= pairs) {
    long long best = kb_total;
    for (int sp = 2; sp <= 8 && tiles_p * sp <= pairs && sp <= kb_total / 4; ++sp) {
      const long long cost = (kb_total + sp - 1) / sp + 16 + 24 * (sp - 1);
      if (cost < best) { best = cost; pair_splits = sp; }
    }
  }
  // Many tokens: the persistent kernels with two accumulators.  Not for 129 to 256 tokens of a
  // matrix with so few rows that most pairs would idle while the one-SM kernel with its K splits
  // fills the GPU (measured at 4096 rows and 129 / 256 tokens: K = 4096 23.1 / 29.1 us by pairs, 15.5 /
  // 18.1 us by single SMs; K = 14336 39.2 / 47.5 against 34.5 / 38.0 us; at 5120 rows and more the pairs win).
  bool persistent = M > 128 && !ss_in;
  if (persistent && M <= 256 && !swiglu && tiles * splits * 5 >= (long long)num_sms * 4 &&
      tiles_p * pair_splits * 10 <= (long long)pairs * 7)
    persistent = false;
  if (persistent) bn = swiglu ? 128 : 256;
  const bool use_pair = persistent;
  if (use_pair) {
    CUtensorMap pw, px;
    if (make_map(&pw, W, (long long)N * (swiglu ? 2 : 1), K, ldw, swiglu ? 64 : 128) &&
        make_map(&px, X, M, K, ldx, pair_bn / 2)) {
      GemmArgs p = {};
      p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.mode = mode;
      // many token tiles: strips of weights in groups of 8, so that a wave of pairs works on 8 strips and 9
      // token tiles instead of 2 or 3 strips and every token tile, whose activations then no longer fit
      // the L2 cache (measured at 8192 tokens: down 774 -> 699 us, gate-up 1497 -> 1375 us, q/k/v 311 -> 281
      // us, 5120 x 14336 1029 -> 830 us; at 4096 tokens 365 -> 357 us for down and no change for the others;
      // at 2048 tokens 1 % slower)
      p.raster = pair_m_tiles >= 24 ? 8 : 0;
      const int rc = swiglu ? launch_pair<true>(pw, px, p, pair_splits, pair_bn, stream)
                            : launch_pair<false>(pw, px, p, pair_splits, pair_bn, stream);
      if (rc != -2) return rc;
    }
  }
  CUtensorMap tw, tx;
  if (!make_map(&tw, W, (long long)N * (swiglu ? 2 : 1), K, ldw, TILE_N)) return -2;
  if (!make_map(&tx, X, M, K, ldx, bn)) return -2;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K;
  a.mode = mode; a.kb_per_split = kb_per_split; a.stages = 0;
  a.ss_in = ss_in; a.ss_in_tiles = ss_in_tiles; a.norm_h = norm_h; a.eps_in = eps_in;
  // the fold and the rotation live in the few-token kernel's K-split reduction only: the
  // persistent kernels neither write xw_out / ss_out nor look at the rope arguments
  const bool emit = xw_out && ss_out && nw && mode == MODE_ACCUM_F32 && splits > 1 && !persistent &&
                    M <= 128 && N % 8 == 0;   // (beyond 128 tokens the products that would take the carry run by pairs)
  a.xw_out = emit ? (__nv_bfloat16*)xw_out : nullptr;
  a.nw = nw; a.nw_is_f32 = nw_is_f32; a.ss_out = emit ? ss_out : nullptr;
  if (emitted) *emitted = emit ? 1 : 0;
  a.rope_on = 0;
  if (rope && mode == MODE_STORE_F32 && splits > 1 && !persistent) {
    const TlRopeArgs* r = (const TlRopeArgs*)rope;
    // measured: a gain for a handful of tokens, a loss from a few dozen on (every thread then
    // computes many sines and reads every partial twice)
    const bool fits = (r->hd == 32 || r->hd == 64 || r->hd == 128) && N == (r->nh + 2 * r->nkv) * r->hd &&
                      M <= 16;
    if (fits) {
      a.rope_on = 1; a.rope_style = r->style; a.rope_nh = r->nh; a.rope_nkv = r->nkv; a.rope_hd = r->hd;
      a.rope_table_stride = r->table_stride;
      a.rope_q = (__nv_bfloat16*)r->q_out; a.rope_k = (__nv_bfloat16*)r->k_pages;
      a.rope_v = (__nv_bfloat16*)r->v_pages; a.rope_pos = r->token_pos; a.rope_seq = r->token_seq;
      a.rope_slot = r->seq_slot; a.rope_table = r->page_table; a.rope_inv_freq = r->inv_freq;
      if (rope_applied) *rope_applied = 1;
    }
  }
  if (persistent)
    return swiglu ? launch_persistent<128, true>(tw, tx, a, num_sms, stream)
                  : launch_persistent<256, false>(tw, tx, a, num_sms, stream);
#define DISPATCH(BN_)                                                                      \
  return swiglu ? launch<BN_, true>(tw, tx, a, splits, budget, stream)                    \
                : launch<BN_, false>(tw, tx, a, splits, budget, stream)
  switch (bn) {
    case 16: DISPATCH(16);
    case 32: DISPATCH(32);
    case 64: DISPATCH(64);
    case 128: DISPATCH(128);
    default: DISPATCH(256);
  }
#undef DISPATCH
}

// Reads and clears the error word that a kernel sets when one of its bounded waits ran
// out (0 = none; 1 producer, 2 issuer, 3 epilogue, 4 accumulator, 5 another pair's partial
// tile).  Synchronises the device.
extern "C" int tl_gemm_tc_take_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, tl_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) {
    cudaMemcpyToSymbol(tl_gemm_tc_error, &zero, sizeof(int));
    static const unsigned int zeros[PAIR_MAX_BLOCKS] = {};
    cudaMemcpyToSymbol(tl_pair_flag, zeros, sizeof(zeros));   // a kernel that gave up may leave flags up
  }
  return v;
}

TL_TRACE_EXPORT(gemm_tc)
