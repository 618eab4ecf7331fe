// Attention of the step's tokens over the paged cache, exact-order version.
//
// One warp per (token, query head). Keys are walked in chunks of 32 aligned to absolute positions
// (chunk c = keys 32c .. 32c+31); lane l scores key 32c+l with a sequential dot product over the head
// dimension, the chunk is folded into an online softmax, and each lane accumulates the output
// dimensions l, l+32, ... . The order of every sum depends only on absolute key positions, so a
// token's output does not depend on how the request was cut into steps, on the other requests of
// the batch, or on which pages hold the keys. All arithmetic is fp32.
//
// Semantics: omniserve/model/qwen2_llm.py:96-112 with omniserve/cache/kv_prealloc.py:138-142 —
// scale hd^-1/2 on the scores, query at absolute position p of its own request sees keys 0..p of
// the same request (with a window w: keys p-w+1..p), query head h reads kv head h / (nh/nkv).
#include "common.cuh"

namespace {
constexpr int MAX_HD = 256;
constexpr int WARPS = 4;

template <typename QT, typename KT, typename OT>
__global__ void __launch_bounds__(WARPS * 32) paged_attn_generic_kernel(
    OT* __restrict__ out, const QT* __restrict__ q, int q_row_stride, const KT* __restrict__ k_cache,
    const KT* __restrict__ v_cache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ seq_lens, const int* __restrict__ tok_seq, int T, int nh,
    int nkv, int hd, int page_size, int num_pages, float scale, int window, int* __restrict__ err) {
  __shared__ float qs[WARPS][MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * WARPS + warp;
  if (wid >= (long long)T * nh) return;
  const int t = (int)(wid / nh), h = (int)(wid % nh);
  const int s = tok_seq[t];
  const int q_len = cu_q[s + 1] - cu_q[s];
  const int kv_len = seq_lens[s];
  const int p = kv_len - q_len + (t - cu_q[s]);  // absolute position of this query
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int kvh = h / (nh / nkv);
  const QT* qp = q + (size_t)t * q_row_stride + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(qp[d]);
  __syncwarp();

  constexpr int ND = MAX_HD / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  const int* bt = block_table + (size_t)s * bt_stride;

  for (int c = lo / 32; c <= p / 32; ++c) {
    const int j = c * 32 + lane;
    const bool valid = (j >= lo && j <= p);
    size_t base = 0;
    float sc = -INFINITY;
    if (valid) {
      const int page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicExch(err, 4);
      } else {
        base = (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * hd;
        const KT* kp = k_cache + base;
        float dot = 0.0f;
        for (int d = 0; d < hd; ++d) dot = fmaf(qs[warp][d], to_f32(kp[d]), dot);
        sc = dot * scale;
      }
    }
    const float cmax = warp_max(sc);
    const float m_new = fmaxf(m, cmax);
    if (m_new == -INFINITY) continue;  // only when a page index was bad
    const float pe = (sc == -INFINITY) ? 0.0f : expf(sc - m_new);
    const float csum = warp_sum(pe);
    const float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * alpha + csum;
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= alpha;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pe, jj);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, jj);
      if (pj == 0.0f) continue;  // masked key (uniform across the warp)
      const KT* vp = v_cache + bj;
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vp[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
  OT* op = out + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = from_f32<OT>(acc[i] * inv);
  }
}
}  // namespace

// out [T, nh*hd]; q rows of stride q_row_stride elements (heads contiguous); caches
// [num_pages, nkv, page_size, hd]; block_table [S, bt_stride]; window <= 0 means all keys.
OSB_API int osb_paged_attn_generic(void* out, int out_dtype, const void* q, int q_dtype, int q_row_stride,
                                   const void* k_cache, const void* v_cache, int cache_dtype,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* seq_lens,
                                   const int* tok_seq, int T, int nh, int nkv, int hd, int page_size,
                                   int num_pages, float scale, int window, int* err, cudaStream_t stream) {
  if (T <= 0) return OSB_OK;
  if (hd > MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv != 0) return OSB_ERR_UNSUPPORTED;
  const long long warps = (long long)T * nh;
  const long long blocks = (warps + WARPS - 1) / WARPS;
  if (blocks > 2147483647LL) return OSB_ERR_TOO_LARGE;
  return osb_dispatch(q_dtype, [&](auto qt) {
    typedef OSB_T(qt) QT;
    return osb_dispatch(cache_dtype, [&](auto kt) {
      typedef OSB_T(kt) KT;
      return osb_dispatch(out_dtype, [&](auto ot) {
        typedef OSB_T(ot) OT;
        paged_attn_generic_kernel<QT, KT, OT><<<(int)blocks, WARPS * 32, 0, stream>>>(
            (OT*)out, (const QT*)q, q_row_stride, (const KT*)k_cache, (const KT*)v_cache, block_table, bt_stride,
            cu_q, seq_lens, tok_seq, T, nh, nkv, hd, page_size, num_pages, scale, window, err);
        return osb_last_error();
      });
    });
  });
}
