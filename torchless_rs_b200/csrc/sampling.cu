// Token selection on the device: arg-max, and sampling with temperature, top-k and
// top-p in the order of the reference (src/sampler/mod.rs:194-222): logits / T, top-k
// on the scaled logits, softmax, top-p on the probabilities, inverse-CDF draw.
//
// One block per row of logits.  Probabilities are kept as 40-bit fixed-point
// integers of exp(z - max): integer sums do not depend on the order of addition, so
// every threshold and the draw are the same from run to run and equal to a
// sequential pass in index order.  The uniform number of each row comes from the
// host, which derives it from (seed, sequence, step).
//
// Ties: arg-max keeps the highest index among equal maxima, as the reference's max_by does
// (src/sampler/mod.rs:60-68); at a top-k or top-p threshold the tied entries of lowest
// index are kept (top-k: as the reference, :108-117; top-p: the reference's unstable
// sort leaves it open, :147).
#include <cuda_runtime.h>
#include <stdint.h>

#include "pdl.cuh"

#define SAMPLE_THREADS 1024
#define FIX_ONE 1099511627776.0f  // 2^40

typedef unsigned long long u64;

__device__ __forceinline__ uint32_t float_key(float f) {
  // larger float -> larger key; NaN is pushed below everything
  if (f != f) return 0u;
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// --------------------------------------------------------------------------
// arg-max
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
  __shared__ uint32_t sk[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_launch_dependents();
  const float* row = logits + (size_t)blockIdx.x * ld;
  uint32_t best = 0u;
  int best_i = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const uint32_t k = float_key(row[i]);
    if (k > best || (k == best && i > best_i)) { best = k; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const uint32_t ok = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ok > best || (ok == best && oi > best_i)) { best = ok; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sk[warp] = best; si[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sk[lane] : 0u;
    best_i = lane < nw ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const uint32_t ok = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ok > best || (ok == best && oi > best_i)) { best = ok; best_i = oi; }
    }
    if (lane == 0) out[blockIdx.x] = (best_i >= 0 && best_i < V) ? best_i : 0;
  }
}

// The same with several blocks per row, for the few rows of a decode step (one block per row
// leaves most SMs idle and takes as long as its one chain of loads).  A block folds its part
// of the row into one 64-bit word per row with atomicMax: key in the high half, the index
// plus one in the low half, so that among equal keys the highest index wins.  The
// block that finishes a row last writes the result and clears the row's word and counter for
// the next launch (they are static: launches on one stream at a time).
#define ARGMAX_ROWS 4096
#define ARGMAX_THREADS 256
__device__ unsigned long long tl_argmax_word[ARGMAX_ROWS];
__device__ unsigned int tl_argmax_count[ARGMAX_ROWS];

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_parts_kernel(const float* __restrict__ logits, int ld, int V, int per_block, int* __restrict__ out) {
  TL_TRACE_SCOPE(6, V, 6);
  __shared__ unsigned long long sw[ARGMAX_THREADS / 32];
  pdl_wait();
  TL_TRACE_RELEASED();
  pdl_launch_dependents();
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * ld;
  const int begin = blockIdx.x * per_block, end = min(V, begin + per_block);
  unsigned long long best = 0ull;
#pragma unroll 4
  for (int i = begin + threadIdx.x; i < end; i += ARGMAX_THREADS) {
    const unsigned long long w = ((unsigned long long)float_key(row[i]) << 32) | (uint32_t)(i + 1);
    best = w > best ? w : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long ow = __shfl_xor_sync(0xffffffffu, best, o);
    best = ow > best ? ow : best;
  }
  if ((threadIdx.x & 31) == 0) sw[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < ARGMAX_THREADS / 32; ++w) best = sw[w] > best ? sw[w] : best;
    atomicMax(&tl_argmax_word[r], best);
    __threadfence();
    if (atomicAdd(&tl_argmax_count[r], 1u) == gridDim.x - 1) {   // every part of the row is in
      __threadfence();
      const unsigned long long w = atomicExch(&tl_argmax_word[r], 0ull);
      const uint32_t low = (uint32_t)(w & 0xffffffffull);   // index + 1; 0: nothing was folded in
      out[r] = (low != 0u && low <= (uint32_t)V) ? (int)(low - 1u) : 0;
      tl_argmax_count[r] = 0u;
    }
  }
}

extern "C" int tl_argmax(const float* logits, int ld, int rows, int V, int* out,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return -1;
  // few rows: spread each over several blocks, about 148 blocks in all
  const int parts = rows >= 64 ? 1 : min(16, max(1, min(148 / rows, (V + 2047) / 2048)));
  if (parts > 1 && rows <= ARGMAX_ROWS) {
    const int per_block = (V + parts - 1) / parts;
    return tl_launch(argmax_parts_kernel, dim3(parts, rows), dim3(ARGMAX_THREADS), 0, stream, logits, ld, V,
                     per_block, out);
  }
  return tl_launch(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, out);
}

// --------------------------------------------------------------------------
// sampling
// --------------------------------------------------------------------------
struct SampleShared {
  u64 wsum[256];
  uint32_t cnt[256];
  u64 warp_tot[32];
  float red[33];
  u64 bcast_u64[2];
  int bcast_int[2];
};

__device__ __forceinline__ float blk_max(float v, SampleShared& sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sm.red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (int)(blockDim.x >> 5) ? sm.red[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (lane == 0) sm.red[32] = t;
  }
  __syncthreads();
  return sm.red[32];
}

// Inclusive scan of one value per thread over the block, in thread order.
// Returns the inclusive prefix; *total receives the block total.
__device__ __forceinline__ u64 blk_scan(u64 v, SampleShared& sm, u64* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sm.warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    u64 t = lane < (int)(blockDim.x >> 5) ? sm.warp_tot[lane] : 0ull;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 n = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += n;
    }
    sm.warp_tot[lane] = t;  // inclusive totals of the warps
  }
  __syncthreads();
  const u64 off = warp ? sm.warp_tot[warp - 1] : 0ull;
  *total = sm.warp_tot[(blockDim.x >> 5) - 1];
  return v + off;
}

// Histogram updates of a whole warp: lanes that hit the same bin are found with match_any and
// one of them adds for all (most logits share their leading bits, so plain atomics would
// queue a thousand threads on two or three bins).  Every lane of the warp must call these;
// `bin` < 0 takes no part.
__device__ __forceinline__ void warp_count(uint32_t* cnt, int bin) {
  if (!__any_sync(0xffffffffu, bin >= 0)) return;   // after the first digits few entries still carry the prefix
  const unsigned peers = __match_any_sync(0xffffffffu, bin);
  if (bin >= 0 && (int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&cnt[bin], (uint32_t)__popc(peers));
}
__device__ __forceinline__ void warp_count_weight(uint32_t* cnt, u64* wsum, int bin, u64 w) {
  if (!__any_sync(0xffffffffu, bin >= 0)) return;   // (as above: most warps have nothing to add in the later passes)
  const unsigned peers = __match_any_sync(0xffffffffu, bin);
  // the weights have 41 bits: three sums of 16-bit (and 9-bit) pieces cannot overflow 32 bits
  const uint32_t a = __reduce_add_sync(peers, (uint32_t)(w & 0xffffull));
  const uint32_t b = __reduce_add_sync(peers, (uint32_t)((w >> 16) & 0xffffull));
  const uint32_t c = __reduce_add_sync(peers, (uint32_t)(w >> 32));
  if (bin >= 0 && (int)(threadIdx.x & 31) == __ffs(peers) - 1) {
    atomicAdd(&cnt[bin], (uint32_t)__popc(peers));
    atomicAdd(&wsum[bin], (u64)a + ((u64)b << 16) + ((u64)c << 32));
  }
}

// Calls f(i, row[i], valid) for every entry of the row, every lane of a warp the same number
// of times (entries past the end come with valid = false).  Four consecutive entries per
// thread and 16-byte loads when the row allows it, so that a pass is not a chain of single
// loads that each wait for L2.
template <typename F>
__device__ __forceinline__ void for_each_entry(const float* row, int V, F f) {
  const int tid = threadIdx.x;
  const int V4 = (((uintptr_t)row & 15) == 0) ? (V & ~3) : 0;
  for (int i0 = 0; i0 < V4; i0 += blockDim.x * 4) {
    const int i = i0 + tid * 4;
    const bool valid = i < V4;
    const float4 x = valid ? *reinterpret_cast<const float4*>(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    f(i, x.x, valid); f(i + 1, x.y, valid); f(i + 2, x.z, valid); f(i + 3, x.w, valid);
  }
  for (int i0 = V4; i0 < V; i0 += blockDim.x) {
    const int i = i0 + tid;
    const bool valid = i < V;
    f(i, valid ? row[i] : 0.0f, valid);
  }
}

struct RowView {
  const float* row;
  int V;
  float T;
  float m;            // max of z
  // top-k state
  bool use_k;
  uint32_t k_thr;     // key of the k-th largest z
  int k_cut;          // entries equal to k_thr are kept up to this index
  // top-p state
  bool use_p;
  u64 p_thr;
  int p_cut;
};

__device__ __forceinline__ float z_from(const RowView& rv, float x) { return x / rv.T; }

__device__ __forceinline__ bool kept_k(const RowView& rv, float z, int i) {
  if (!rv.use_k) return true;
  const uint32_t k = float_key(z);
  return k > rv.k_thr || (k == rv.k_thr && i <= rv.k_cut);
}

__device__ __forceinline__ u64 fix_of(const RowView& rv, float z) {
  return (u64)(expf(z - rv.m) * FIX_ONE);
}

// The first index, in index order, at which the running sum of weight(i) exceeds `target`
// (`fallback` if the whole sum does not).  Each thread takes SCAN_E consecutive entries per
// round, so a round of the block covers 8192 entries with one scan.
#define SCAN_E 8
template <typename Weight>
__device__ int first_exceeding(const float* row, int V, u64 target, SampleShared& sm, int fallback,
                               Weight weight) {
  u64 carry = 0;
  int found = fallback;
  const bool vec = ((uintptr_t)row & 15) == 0;
  for (int base = 0; base < V; base += blockDim.x * SCAN_E) {
    const int i0 = base + threadIdx.x * SCAN_E;
    float x[SCAN_E];
    if (vec && i0 + SCAN_E <= V) {
      const float4 a = *reinterpret_cast<const float4*>(row + i0), b = *reinterpret_cast<const float4*>(row + i0 + 4);
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < SCAN_E; ++e) x[e] = i0 + e < V ? row[i0 + e] : 0.0f;
    }
    u64 w[SCAN_E], mine = 0;
#pragma unroll
    for (int e = 0; e < SCAN_E; ++e) {
      w[e] = i0 + e < V ? weight(i0 + e, x[e]) : 0ull;
      mine += w[e];
    }
    u64 total;
    const u64 inc = blk_scan(mine, sm, &total) + carry;
    u64 run = inc - mine;
    if (mine && inc > target && run <= target) {   // the crossing lies in this thread's entries
#pragma unroll
      for (int e = 0; e < SCAN_E; ++e) {
        const bool before = run <= target;
        run += w[e];
        if (before && run > target) sm.bcast_int[0] = i0 + e;
      }
    }
    const bool done = carry + total > target;
    carry += total;
    __syncthreads();
    if (done) { found = sm.bcast_int[0]; break; }
  }
  __syncthreads();
  return found;
}

// Index of the `need`-th entry (1-based, in index order) for which pred holds.
template <typename Pred>
__device__ int nth_in_order(const float* row, int V, int need, SampleShared& sm, Pred pred) {
  return first_exceeding(row, V, (u64)(need - 1), sm, V - 1,
                         [&](int i, float x) { return pred(i, x) ? 1ull : 0ull; });
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, float temperature, int top_k,
              float top_p, const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ SampleShared sm;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  RowView rv;
  rv.row = logits + (size_t)blockIdx.x * ld;
  rv.V = V;
  rv.T = temperature;
  rv.use_k = top_k > 0 && top_k < V;
  rv.use_p = top_p > 0.0f && top_p < 1.0f;
  rv.k_thr = 0u; rv.k_cut = V; rv.p_thr = 0ull; rv.p_cut = V;

  // ---- max of the scaled logits
  float m = -INFINITY;
  for_each_entry(rv.row, V, [&](int, float x, bool valid) {
    const float z = z_from(rv, x);
    if (valid && z == z) m = fmaxf(m, z);
  });
  rv.m = blk_max(m, sm);

  // ---- top-k: key of the k-th largest scaled logit by radix selection
  if (rv.use_k) {
    uint32_t prefix = 0u, mask = 0u;
    int remaining = top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += blockDim.x) sm.cnt[b] = 0u;
      __syncthreads();
      for_each_entry(rv.row, V, [&](int, float x, bool valid) {   // whole warps: see warp_count
        const uint32_t k = float_key(z_from(rv, x));
        warp_count(sm.cnt, (valid && (k & mask) == prefix) ? (int)((k >> shift) & 255u) : -1);
      });
      __syncthreads();
      if (tid == 0) {
        int rem = remaining, b = 255;
        for (; b > 0; --b) {
          if ((int)sm.cnt[b] >= rem) break;
          rem -= (int)sm.cnt[b];
        }
        sm.bcast_int[0] = b;
        sm.bcast_int[1] = rem;
      }
      __syncthreads();
      prefix |= ((uint32_t)sm.bcast_int[0]) << shift;
      mask |= 255u << shift;
      remaining = sm.bcast_int[1];
      __syncthreads();
    }
    rv.k_thr = prefix;
    // `remaining` entries equal to the threshold are kept, lowest indices first
    const uint32_t thr = prefix;
    const RowView rvc = rv;
    rv.k_cut = nth_in_order(rv.row, V, remaining, sm,
                            [&](int, float x) { return float_key(z_from(rvc, x)) == thr; });
  }

  // ---- sum of the kept fixed-point weights
  u64 part = 0;
  for_each_entry(rv.row, V, [&](int i, float x, bool valid) {
    const float z = z_from(rv, x);
    if (valid && z == z && kept_k(rv, z, i)) part += fix_of(rv, z);
  });
  u64 S;
  blk_scan(part, sm, &S);
  __syncthreads();

  // ---- top-p: smallest weight that still belongs to the nucleus
  if (rv.use_p) {
    u64 target = (u64)ceil((double)top_p * (double)S);
    if (target > S) target = S;
    if (target < 1ull) target = 1ull;
    u64 prefix = 0ull, mask = 0ull, above = 0ull;  // `above` = weight strictly above the prefix
    for (int shift = 40; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += blockDim.x) { sm.cnt[b] = 0u; sm.wsum[b] = 0ull; }
      __syncthreads();
      for_each_entry(rv.row, V, [&](int i, float x, bool valid) {   // whole warps: see warp_count
        int b = -1;
        u64 w = 0;
        const float z = z_from(rv, x);
        if (valid && z == z && kept_k(rv, z, i)) {
          w = fix_of(rv, z);
          if ((w & mask) == prefix) b = (int)((w >> shift) & 255ull);
        }
        warp_count_weight(sm.cnt, sm.wsum, b, w);
      });
      __syncthreads();
      if (tid == 0) {
        u64 acc = above;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + sm.wsum[b] >= target) break;
          acc += sm.wsum[b];
        }
        sm.bcast_int[0] = b;
        sm.bcast_u64[0] = acc;
      }
      __syncthreads();
      prefix |= ((u64)sm.bcast_int[0]) << shift;
      mask |= 255ull << shift;
      above = sm.bcast_u64[0];
      __syncthreads();
    }
    rv.p_thr = prefix;
    int need = 1;
    if (prefix > 0ull && target > above) {
      const u64 n = (target - above + prefix - 1ull) / prefix;
      need = n > (u64)V ? V : (int)n;
      if (need < 1) need = 1;
    }
    const RowView rvc = rv;
    const u64 thr = prefix;
    rv.p_cut = nth_in_order(rv.row, V, need, sm, [&](int i, float x) {
      const float z = z_from(rvc, x);
      return z == z && kept_k(rvc, z, i) && fix_of(rvc, z) == thr;
    });
    S = above + (u64)need * prefix;
  }

  // ---- draw: first kept index whose running weight exceeds floor(r * S)
  float r = uniform[blockIdx.x];
  r = r < 0.0f ? 0.0f : (r >= 1.0f ? 0.99999994f : r);
  u64 target = (u64)((double)r * (double)S);
  if (target >= S) target = S ? S - 1ull : 0ull;
  const RowView rvd = rv;
  const int chosen = first_exceeding(rv.row, V, target, sm, -1, [&](int i, float x) {
    const float z = z_from(rvd, x);
    if (!(z == z) || !kept_k(rvd, z, i)) return 0ull;
    const u64 w = fix_of(rvd, z);
    if (rvd.use_p && !(w > rvd.p_thr || (w == rvd.p_thr && i <= rvd.p_cut))) return 0ull;
    return w;
  });
  if (tid == 0) out[blockIdx.x] = chosen >= 0 ? chosen : V - 1;  // the reference's fallback, :237
}

// temperature must be > 0; rows with temperature <= 0 go through tl_argmax.
extern "C" int tl_sample(const float* logits, int ld, int rows, int V, float temperature,
                         int top_k, float top_p, const float* uniform, int* out,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0 || !(temperature > 0.0f)) return -1;
  return tl_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V,
                   temperature, top_k, top_p, uniform, out);
}

TL_TRACE_EXPORT(sampling)
