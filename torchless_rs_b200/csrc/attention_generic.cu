// Attention over the paged cache on CUDA cores, for prefill and decode alike, with
// every head size that is a multiple of 16 up to 256 and any number of heads and
// groups.  It is the attention of the true 32-bit path and the fallback of the
// bfloat16 path.
//
// One block per (token, query head).  The token's position p and its sequence's page
// table give the keys: i in [max(0, p - W + 1), p] with a window W, else [0, p]
// (reference: scores, softmax and weighted sum of src/model/modules/attention.rs:78-121;
// window inequality of src/model/models/gpt_oss.rs:168-176).  Keys are taken 128 at a
// time, counted from the first visible key, with a running maximum and sum kept in
// 32-bit, so the result of a position is the same in whatever step or batch it is
// computed.
#include "common.cuh"

#define ATT_THREADS 128
#define MAX_HD 256

#if TL_DTYPE == 0
#define AVEC 4
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
#else
#define AVEC 8
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
#endif

__global__ void __launch_bounds__(ATT_THREADS)
attn_generic_kernel(const act_t* __restrict__ q, const act_t* __restrict__ k_pages,
                    const act_t* __restrict__ v_pages, act_t* __restrict__ out,
                    const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                    const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                    int table_stride, int nh, int nkv, int hd, int window, float scale) {
  __shared__ float qs[MAX_HD];
  __shared__ float ps[ATT_THREADS];
  __shared__ int pg[ATT_THREADS];  // page of each key of the chunk
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (nh / nkv);
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int* table = page_table + (size_t)slot * table_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t page_elems = (size_t)nkv * TL_PAGE * hd;
  const size_t head_off = (size_t)kvh * TL_PAGE * hd;

  for (int d = tid; d < hd; d += ATT_THREADS) qs[d] = to_f32(q[(size_t)t * nh * hd + h * hd + d]);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f;
  float acc0 = 0.0f, acc1 = 0.0f;  // dims tid and tid + 128
  for (int base = lo; base <= pos; base += ATT_THREADS) {
    const int i = base + tid;
    const bool valid = i <= pos;
    float s = -INFINITY;
    int page = -1;
    if (valid) {
      page = table[i / TL_PAGE];
      const act_t* krow = k_pages + (size_t)page * page_elems + head_off + (size_t)(i % TL_PAGE) * hd;
      float dot = 0.0f;
      for (int d = 0; d < hd; d += AVEC) {
        float kv[AVEC];
        load_row_vec(krow + d, kv);
#pragma unroll
        for (int e = 0; e < AVEC; ++e) dot = fmaf(qs[d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    const float cmax = block_max(s, scratch);
    const float m_new = fmaxf(m_run, cmax);
    const float p = valid ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    pg[tid] = page;
    const float csum = block_sum(p, scratch);  // has the barriers that publish ps and pg
    const float alpha = expf(m_run - m_new);   // 0 at the first chunk (m_run = -inf)
    l_run = l_run * alpha + csum;
    m_run = m_new;
    const int cnt = (pos - base + 1 < ATT_THREADS) ? pos - base + 1 : ATT_THREADS;
    if (tid < hd) {
      acc0 *= alpha;
      acc1 *= alpha;
      const bool two = tid + ATT_THREADS < hd;
      for (int j = 0; j < cnt; ++j) {
        const int key = base + j;
        // values lie transposed in a page: [hd][TL_PAGE]
        const act_t* vcol = v_pages + (size_t)pg[j] * page_elems + head_off + (key % TL_PAGE);
        const float pj = ps[j];
        acc0 = fmaf(pj, to_f32(vcol[(size_t)tid * TL_PAGE]), acc0);
        if (two) acc1 = fmaf(pj, to_f32(vcol[(size_t)(tid + ATT_THREADS) * TL_PAGE]), acc1);
      }
    }
    __syncthreads();  // ps and pg are rewritten by the next chunk
  }
  act_t* o = out + (size_t)t * nh * hd + h * hd;
  if (tid < hd) o[tid] = from_f32<act_t>(acc0 / l_run);
  if (tid + ATT_THREADS < hd) o[tid + ATT_THREADS] = from_f32<act_t>(acc1 / l_run);
}

extern "C" int TL_NAME(tl_attn_generic)(const void* q, const void* k_pages, const void* v_pages,
                                        void* out, const int* token_pos, const int* token_seq,
                                        const int* seq_slot, const int* page_table,
                                        int table_stride, int T, int nh, int nkv, int hd,
                                        int window, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd % 16 != 0 || hd < 16 || hd > MAX_HD || nkv <= 0 || nh % nkv != 0) return TL_ERR_UNSUPPORTED;
  dim3 grid(T, nh);
  return tl_launch(attn_generic_kernel, grid, dim3(ATT_THREADS), 0, stream, (const act_t*)q,
                   (const act_t*)k_pages, (const act_t*)v_pages, (act_t*)out, token_pos, token_seq,
                   seq_slot, page_table, table_stride, nh, nkv, hd, window, scale);
}
