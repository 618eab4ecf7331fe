// bf16 attention over the paged cache on the tensor cores (m16n8k16 MMA, fp32 scores, softmax and
// accumulators), for the serving path.
//
//  * attn_prefill_kernel: requests that bring two or more tokens (prompt portions, whole prompts).
//    One CTA = 64 query rows of one (request, query head); keys and values stream through shared
//    memory in tiles of 64 keys gathered page by page with cp.async; online softmax.
//  * attn_decode_kernel: requests that bring exactly one token. One CTA = one (request, kv head,
//    split of the keys); the query heads of the group share every key/value load; the four warps
//    take different keys of each tile and are merged at the end. Splits of the key range end at
//    fixed absolute boundaries; their partial results (unnormalised output, running max, sum) go
//    to scratch memory and attn_decode_reduce_kernel merges them in split order.
//
// Semantics as in attn_generic.cu (omniserve/model/qwen2_llm.py:96-112, omniserve/cache/kv_prealloc.py:138-142):
// scale on the scores, query at absolute position p sees keys max(0, p-window+1)..p of its own
// request, query head h reads kv head h / (nh/nkv).
// Cache layout: [pages, kv_heads, page_size, head_dim]; a page id < 0 marks a page given back (its
// keys are outside every window and are read as zeros, then masked).
#include <cooperative_groups.h>

#include "mma_utils.cuh"

namespace cg = cooperative_groups;

namespace {
constexpr int TILE_N = 64;
constexpr int NTHREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

// Copies keys [key0, key0 + TILE_N) of one kv head into the shared tiles ktile and vtile
// ([TILE_N][hd + 8] each). The page size is a power of two; key0 is a multiple of TILE_N, so a tile
// starts on a page boundary (or lies inside one page). The tile's page ids are fetched once per warp
// (lane l holds page l of the tile) and handed to the rows by shuffle. Rows at or beyond kv_end and
// rows of pages that were given back are zero-filled. Every thread runs the same number of
// iterations (hd/16), so the shuffles are warp-uniform.
__device__ __forceinline__ void load_kv_tiles_async(bf16* ktile, bf16* vtile, const bf16* __restrict__ kc,
                                                    const bf16* __restrict__ vc, const int* __restrict__ bt, int kvh,
                                                    int nkv, int log2ps, int hd, int key0, int kv_end, int num_pages,
                                                    int tid) {
  const int lane = tid & 31;
  const int cpr = hd >> 3;  // 16-byte chunks per row
  const int stride = hd + 8;
  const int first_page = key0 >> log2ps;
  const int npages = log2ps >= 6 ? 1 : (TILE_N >> log2ps);
  int my_page = -1;
  if (lane < npages && ((first_page + lane) << log2ps) < kv_end) {
    my_page = bt[first_page + lane];
    if (my_page >= num_pages) my_page = -1;
  }
  const size_t page_stride = ((size_t)nkv << log2ps) * hd;
  const size_t head_off = ((size_t)kvh << log2ps) * hd;
  const int ps_mask = (1 << log2ps) - 1;
  int r = tid / cpr, c = tid - r * cpr;
  const int dr = NTHREADS / cpr, dc = NTHREADS - dr * cpr;
  const int iters = cpr >> 1;  // TILE_N * cpr / NTHREADS
  for (int it = 0; it < iters; ++it) {
    const int key = key0 + r;
    const int page = __shfl_sync(0xffffffffu, my_page, (key >> log2ps) - first_page);
    const bool valid = key < kv_end && page >= 0;
    const size_t off = valid ? (size_t)page * page_stride + head_off + (size_t)(key & ps_mask) * hd + c * 8 : 0;
    cp_async16(ktile + r * stride + c * 8, kc + off, valid);
    cp_async16(vtile + r * stride + c * 8, vc + off, valid);
    r += dr;
    c += dc;
    if (c >= cpr) {
      c -= cpr;
      ++r;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Prefill: 64 query rows per CTA, 16 per warp.
template <int HD_MAX>
__global__ void __launch_bounds__(NTHREADS) attn_prefill_kernel(
    bf16* __restrict__ out, const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ kc,
    const bf16* __restrict__ vc, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
    const int* __restrict__ seq_lens, int nh, int nkv, int hd, int log2ps, int num_pages, float scale_log2,
    int window, int skip_single) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = hd + 8;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);  // [64][stride]
  bf16* kvs = qs + 64 * stride;                  // 2 stages x (K, V) x [TILE_N][stride]
  const int tile_elems = TILE_N * stride;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m_tile = gridDim.x - 1 - blockIdx.x;  // long tiles first
  const int h = blockIdx.y, s = blockIdx.z;
  const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
  if (q_len <= 0 || (skip_single && q_len == 1)) return;
  const int m0 = m_tile * 64;
  if (m0 >= q_len) return;
  const int g = nh / nkv, kvh = h / g;
  const int kv_len = seq_lens[s];
  const int rows_here = min(64, q_len - m0);
  const int p_first = kv_len - q_len + m0;
  const int p_last = p_first + rows_here - 1;
  const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int tile_begin = lo / TILE_N, tile_end = p_last / TILE_N;  // inclusive
  const int* bt = block_table + (size_t)s * bt_stride;
  const int kv_end = p_last + 1;

  {  // Q tile
    const int cpr = hd >> 3;
    for (int i = tid; i < 64 * cpr; i += NTHREADS) {
      const int r = i / cpr, c = i - r * cpr;
      const bool valid = r < rows_here;
      const bf16* src = valid ? q + (size_t)(q0 + m0 + r) * q_row_stride + (size_t)h * hd + c * 8 : q;
      cp_async16(qs + r * stride + c * 8, src, valid);
    }
  }
  load_kv_tiles_async(kvs, kvs + tile_elems, kc, vc, bt, kvh, nkv, log2ps, hd, tile_begin * TILE_N, kv_end, num_pages, tid);
  cp_async_commit();

  constexpr int KS = HD_MAX / 16;  // k-steps of QK^T, pairs of n-tiles of PV
  const int ks_n = hd >> 4;
  unsigned qf[KS][4];
  float o[KS * 2][4];
#pragma unroll
  for (int i = 0; i < KS * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const int g0 = lane >> 2, c2 = (lane & 3) * 2;
  const int row_l[2] = {warp * 16 + g0, warp * 16 + g0 + 8};
  int p_row[2], lo_row[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    p_row[hh] = row_l[hh] < rows_here ? p_first + row_l[hh] : -1;
    lo_row[hh] = (window > 0 && p_row[hh] - window + 1 > 0) ? p_row[hh] - window + 1 : 0;
  }
  const bool warp_active = warp * 16 < rows_here;
  const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: matrix index and row within it

  for (int t = tile_begin; t <= tile_end; ++t) {
    const int st = (t - tile_begin) & 1;
    if (t + 1 <= tile_end) {
      bf16* nk = kvs + (st ^ 1) * 2 * tile_elems;
      load_kv_tiles_async(nk, nk + tile_elems, kc, vc, bt, kvh, nkv, log2ps, hd, (t + 1) * TILE_N, kv_end, num_pages, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* ks = kvs + st * 2 * tile_elems;
    const bf16* vs = ks + tile_elems;
    if (t == tile_begin) {
#pragma unroll
      for (int k = 0; k < KS; ++k)
        if (k < ks_n)
          ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3],
                      qs + (warp * 16 + lr + (lm & 1) * 8) * stride + k * 16 + (lm >> 1) * 8);
    }
    // a warp whose rows all lie before this tile's first key has nothing to do here
    const int key0 = t * TILE_N;
    if (warp_active && key0 <= p_first + min(warp * 16 + 15, rows_here - 1)) {
      float sc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        if (k < ks_n) {
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, ks + (np * 16 + lr + (lm >> 1) * 8) * stride + k * 16 + (lm & 1) * 8);
            mma_bf16_16816(sc[np * 2], qf[k], b0, b1);
            mma_bf16_16816(sc[np * 2 + 1], qf[k], b2, b3);
          }
        }
      }
      // scale, mask, online softmax
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + n * 8 + c2 + e;
            float v = sc[n][hh * 2 + e] * scale_log2;
            if (key > p_row[hh] || key < lo_row[hh]) v = -INFINITY;
            sc[n][hh * 2 + e] = v;
            mx = fmaxf(mx, v);
          }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[hh], mx);
        const float alpha = (m_run[hh] == -INFINITY) ? 0.0f : fast_exp2(m_run[hh] - m_new);
        float sum = 0.0f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float v = sc[n][hh * 2 + e];
            const float p = (v == -INFINITY) ? 0.0f : fast_exp2(v - m_new);
            sc[n][hh * 2 + e] = p;
            sum += p;
          }
        }
        l_run[hh] = l_run[hh] * alpha + sum;
        m_run[hh] = m_new;
#pragma unroll
        for (int i = 0; i < KS * 2; ++i) {
          o[i][hh * 2] *= alpha;
          o[i][hh * 2 + 1] *= alpha;
        }
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        unsigned pa[4];
        pa[0] = pack_bf16(sc[kk * 2][0], sc[kk * 2][1]);
        pa[1] = pack_bf16(sc[kk * 2][2], sc[kk * 2][3]);
        pa[2] = pack_bf16(sc[kk * 2 + 1][0], sc[kk * 2 + 1][1]);
        pa[3] = pack_bf16(sc[kk * 2 + 1][2], sc[kk * 2 + 1][3]);
#pragma unroll
        for (int dp = 0; dp < KS; ++dp) {
          if (dp < ks_n) {
            unsigned b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, vs + (kk * 16 + lr + (lm & 1) * 8) * stride + dp * 16 + (lm >> 1) * 8);
            mma_bf16_16816(o[dp * 2], pa, b0, b1);
            mma_bf16_16816(o[dp * 2 + 1], pa, b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (!warp_active) return;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float l = l_run[hh];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (row_l[hh] >= rows_here) continue;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    bf16* op = out + ((size_t)(q0 + m0 + row_l[hh]) * nh + h) * hd;
#pragma unroll
    for (int i = 0; i < KS * 2; ++i) {
      const int d = i * 8 + c2;
      if (d < hd)
        *reinterpret_cast<__nv_bfloat162*>(op + d) = __floats2bfloat162_rn(o[i][hh * 2] * inv, o[i][hh * 2 + 1] * inv);
    }
  }
}

// Optional fusion of the rotary encoding and the cache write into the decode kernel: the query
// rows are rotated in shared memory, and the CTA whose split holds the new token's position rotates
// that token's key and stores key and value into their page before it loads its tiles. Only for
// groups of at most 16 query heads (one CTA per request and kv head reads the new key).
struct FusedRope {
  const float* cos_t;   // [T, rot/2]; null: no fusion (q already rotated, cache already written)
  const float* sin_t;
  const int* slot_map;  // [T] flat cache slot of every token
  int rot;
};

// ------------------------------------------------------------------------------------------------
// Decode: one token per request. grid = (splits, kv heads x head tiles, requests).
template <int HD_MAX, int STAGES, bool CLUSTER>
__global__ void __launch_bounds__(NTHREADS) attn_decode_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
    int q_row_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
    const int* __restrict__ decode_index, int* __restrict__ counters, int nh, int nkv, int hd, int log2ps,
    int num_pages, float scale_log2, int window, int chunk, int nsplits, FusedRope fr) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_last;
  const int stride = hd + 8;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);  // [16][stride]; later the warps' (max, sum)
  bf16* kvs = qs + 16 * stride;                  // STAGES x (K, V) x [TILE_N][stride]; later the warps' outputs
  const int tile_elems = TILE_N * stride;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, s = blockIdx.z;
  const int g = nh / nkv;
  const int head_tiles = (g + 15) >> 4;
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y - kvh * head_tiles;
  const int q0 = cu_q[s];
  if (cu_q[s + 1] - q0 != 1) return;
  const int rows = min(16, g - ht * 16);
  const int head0 = kvh * g + ht * 16;
  const int kv_len = seq_lens[s];
  const int p = kv_len - 1;
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int first_split = lo / chunk, last_split = p / chunk;
  // a split without keys has nothing to do; inside a cluster it still takes part in the merge
  const bool active = split >= first_split && split <= last_split;
  if (!CLUSTER && !active) return;
  const int k_begin = max(split * chunk, (lo / TILE_N) * TILE_N);
  const int k_end = min((split + 1) * chunk, kv_len);
  const int ntiles = active ? (k_end - k_begin + TILE_N - 1) / TILE_N : 0;
  const int* bt = block_table + (size_t)s * bt_stride;

  // Everything read so far was written by the host before the step. When this kernel stores the new key
  // and value itself (fused rotary form), the tiles of every split but the last do not depend on the
  // kernel before this one either: their first copies start before the wait for that kernel.
  const bool early = fr.cos_t != nullptr && split != last_split;
  auto first_tiles = [&]() {
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
      if (st < ntiles) {
        bf16* dst = kvs + st * 2 * tile_elems;
        load_kv_tiles_async(dst, dst + tile_elems, kc, vc, bt, kvh, nkv, log2ps, hd, k_begin + st * TILE_N, k_end, num_pages, tid);
      }
      cp_async_commit();
    }
  };
  if (early) first_tiles();
  pdl_wait();
  if (fr.cos_t != nullptr && split == last_split && ht == 0) {
    // the new token's key (rotated) and value go into their page before this CTA reads its tiles
    const int slot = fr.slot_map[q0];
    const int page = slot >> log2ps, off = slot & ((1 << log2ps) - 1);
    if (page >= 0 && page < num_pages) {
      const size_t dst = ((((size_t)page * nkv + kvh) << log2ps) + off) * hd;
      bf16* kd = const_cast<bf16*>(kc) + dst;
      bf16* vd = const_cast<bf16*>(vc) + dst;
      const bf16* ksrc = q + (size_t)q0 * q_row_stride + (size_t)(nh + kvh) * hd;
      const bf16* vsrc = q + (size_t)q0 * q_row_stride + (size_t)(nh + nkv + kvh) * hd;
      const int half = fr.rot >> 1;
      const float* cs = fr.cos_t + (size_t)q0 * half;
      const float* sn = fr.sin_t + (size_t)q0 * half;
      for (int d = tid; d < half; d += NTHREADS) {
        const float x1 = __bfloat162float(ksrc[d]), x2 = __bfloat162float(ksrc[d + half]);
        kd[d] = __float2bfloat16_rn(x1 * cs[d] - x2 * sn[d]);
        kd[d + half] = __float2bfloat16_rn(x2 * cs[d] + x1 * sn[d]);
      }
      for (int d = fr.rot + tid; d < hd; d += NTHREADS) kd[d] = ksrc[d];
      for (int d = tid; d < hd; d += NTHREADS) vd[d] = vsrc[d];
    }
    __threadfence();
    __syncthreads();
  }

  // the group's query rows (plain loads: they must not become a copy group of their own). In the fused
  // rotary form a thread takes the 8 elements at d and their partners at d + rot/2 and rotates them on the
  // way, the cos/sin loads in flight together with the q loads: one round trip instead of two.
  const bool rotate_here = fr.cos_t != nullptr && ((fr.rot >> 1) & 7) == 0;
  {
    const int cpr = hd >> 3;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    if (rotate_here) {
      const int half = fr.rot >> 1, hc = half >> 3;            // chunks of 8 in half the rotated span
      const int per_row = hc + (cpr - 2 * hc);                  // rotated pairs, then chunks that are not rotated
      const float* cs = fr.cos_t + (size_t)q0 * half;
      const float* sn = fr.sin_t + (size_t)q0 * half;
      for (int i = tid; i < 16 * per_row; i += NTHREADS) {
        const int r = i / per_row, c = i - r * per_row;
        bf16* dst = qs + r * stride;
        const bf16* src = q + (size_t)q0 * q_row_stride + (size_t)(head0 + r) * hd;
        if (c >= hc) {  // beyond the rotated span
          const int cc = 2 * hc + (c - hc);
          *reinterpret_cast<uint4*>(dst + cc * 8) = r < rows ? *reinterpret_cast<const uint4*>(src + cc * 8) : zero4;
          continue;
        }
        uint4 a = zero4, b = zero4;
        if (r < rows) {
          a = *reinterpret_cast<const uint4*>(src + c * 8);
          b = *reinterpret_cast<const uint4*>(src + half + c * 8);
          const float4 c0 = *reinterpret_cast<const float4*>(cs + c * 8), c1 = *reinterpret_cast<const float4*>(cs + c * 8 + 4);
          const float4 s0 = *reinterpret_cast<const float4*>(sn + c * 8), s1 = *reinterpret_cast<const float4*>(sn + c * 8 + 4);
          const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
          __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x1 = __bfloat1622float2(pa[e]), x2 = __bfloat1622float2(pb[e]);
            pa[e] = __floats2bfloat162_rn(x1.x * cv[2 * e] - x2.x * sv[2 * e], x1.y * cv[2 * e + 1] - x2.y * sv[2 * e + 1]);
            pb[e] = __floats2bfloat162_rn(x2.x * cv[2 * e] + x1.x * sv[2 * e], x2.y * cv[2 * e + 1] + x1.y * sv[2 * e + 1]);
          }
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = a;
        *reinterpret_cast<uint4*>(dst + half + c * 8) = b;
      }
    } else {
      for (int i = tid; i < 16 * cpr; i += NTHREADS) {
        const int r = i / cpr, c = i - r * cpr;
        uint4 v = zero4;
        if (r < rows) v = *reinterpret_cast<const uint4*>(q + (size_t)q0 * q_row_stride + (size_t)(head0 + r) * hd + c * 8);
        *reinterpret_cast<uint4*>(qs + r * stride + c * 8) = v;
      }
    }
  }
  if (!early) first_tiles();

  constexpr int KS = HD_MAX / 16;
  const int ks_n = hd >> 4;
  unsigned qf[KS][4];
  float o[KS * 2][4];
#pragma unroll
  for (int i = 0; i < KS * 2; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const int g0 = lane >> 2, c2 = (lane & 3) * 2;
  const int lm = lane >> 3, lr = lane & 7;

  for (int t = 0; t < ntiles; ++t) {
    const int st = t % STAGES;
    {
      const int tn = t + STAGES - 1;
      if (tn < ntiles) {
        bf16* dst = kvs + (tn % STAGES) * 2 * tile_elems;
        load_kv_tiles_async(dst, dst + tile_elems, kc, vc, bt, kvh, nkv, log2ps, hd, k_begin + tn * TILE_N, k_end, num_pages, tid);
      }
      cp_async_commit();
    }
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const bf16* ks = kvs + st * 2 * tile_elems;
    const bf16* vs = ks + tile_elems;
    if (t == 0) {
      if (fr.cos_t != nullptr && !rotate_here) {  // rotate the query rows in place in shared memory
        const int half = fr.rot >> 1;
        const float* cs = fr.cos_t + (size_t)q0 * half;
        const float* sn = fr.sin_t + (size_t)q0 * half;
        for (int i = tid; i < rows * half; i += NTHREADS) {
          const int r = i / half, d = i - r * half;
          bf16* row = qs + r * stride;
          const float x1 = __bfloat162float(row[d]), x2 = __bfloat162float(row[d + half]);
          row[d] = __float2bfloat16_rn(x1 * cs[d] - x2 * sn[d]);
          row[d + half] = __float2bfloat16_rn(x2 * cs[d] + x1 * sn[d]);
        }
        __syncthreads();
      }
#pragma unroll
      for (int k = 0; k < KS; ++k)
        if (k < ks_n)
          ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], qs + (lr + (lm & 1) * 8) * stride + k * 16 + (lm >> 1) * 8);
    }
    const int kbase = k_begin + t * TILE_N + warp * 16;  // this warp's 16 keys of the tile
    if (kbase < k_end && kbase + 15 >= lo) {
      // two accumulator pairs (even and odd k-steps) halve the chain of dependent MMAs
      float sc[2][4], sd[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[n][e] = sd[n][e] = 0.0f;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        if (k < ks_n) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, ks + (warp * 16 + lr + (lm >> 1) * 8) * stride + k * 16 + (lm & 1) * 8);
          if (k & 1) {
            mma_bf16_16816(sd[0], qf[k], b0, b1);
            mma_bf16_16816(sd[1], qf[k], b2, b3);
          } else {
            mma_bf16_16816(sc[0], qf[k], b0, b1);
            mma_bf16_16816(sc[1], qf[k], b2, b3);
          }
        }
      }
      // every row is the same query position: the mask depends on the key only
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = kbase + n * 8 + c2 + e;
          const bool vis = key < k_end && key >= lo;
          const float v0 = vis ? (sc[n][e] + sd[n][e]) * scale_log2 : -INFINITY;
          const float v1 = vis ? (sc[n][2 + e] + sd[n][2 + e]) * scale_log2 : -INFINITY;
          sc[n][e] = v0;
          sc[n][2 + e] = v1;
          mx0 = fmaxf(mx0, v0);
          mx1 = fmaxf(mx1, v1);
        }
      }
      // m_run is the exponent offset in use; it moves only when the maximum has grown by more than 2^8
      // (or at the first keys), so that the accumulated output is rescaled rarely
      float mx[2] = {mx0, mx1}, alpha[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float v = mx[hh];
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        const bool grow = v > m_run[hh] + 8.0f || (m_run[hh] == -INFINITY && v > -INFINITY);
        alpha[hh] = (grow && m_run[hh] != -INFINITY) ? fast_exp2(m_run[hh] - v) : 1.0f;
        if (grow) m_run[hh] = v;
        const float off = m_run[hh];
        float sum = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float x = sc[n][hh * 2 + e];
            const float pe = (x == -INFINITY) ? 0.0f : fast_exp2(x - off);
            sc[n][hh * 2 + e] = pe;
            sum += pe;
          }
        }
        l_run[hh] = l_run[hh] * alpha[hh] + sum;
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < KS * 2; ++i) {
          o[i][0] *= alpha[0];
          o[i][1] *= alpha[0];
          o[i][2] *= alpha[1];
          o[i][3] *= alpha[1];
        }
      }
      unsigned pa[4];
      pa[0] = pack_bf16(sc[0][0], sc[0][1]);
      pa[1] = pack_bf16(sc[0][2], sc[0][3]);
      pa[2] = pack_bf16(sc[1][0], sc[1][1]);
      pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
      for (int dp = 0; dp < KS; ++dp) {
        if (dp < ks_n) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vs + (warp * 16 + lr + (lm & 1) * 8) * stride + dp * 16 + (lm >> 1) * 8);
          mma_bf16_16816(o[dp * 2], pa, b0, b1);
          mma_bf16_16816(o[dp * 2 + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  pdl_trigger();

  // merge the four warps (each saw different keys) in warp order: per-warp results of the valid rows
  // go to shared memory (row stride hd + 8 floats: the 64-bit stores of a half-warp hit distinct banks)
  const int ostride = hd + 8;
  float* wml = reinterpret_cast<float*>(qs);   // [4][16][2], then the CTA's own [16][2]
  float* wo = reinterpret_cast<float*>(kvs);   // [4][16][ostride], then the CTA's own [16][ostride]
  float* cml = wml + 4 * 16 * 2;
  float* co = wo + 4 * 16 * ostride;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float l = l_run[hh];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int r = g0 + hh * 8;
    if (r < rows) {
      if ((lane & 3) == 0) {
        wml[(warp * 16 + r) * 2] = m_run[hh];
        wml[(warp * 16 + r) * 2 + 1] = l;
      }
#pragma unroll
      for (int i = 0; i < KS * 2; ++i) {
        const int d = i * 8 + c2;
        if (d < hd)
          *reinterpret_cast<float2*>(wo + (warp * 16 + r) * ostride + d) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
      }
    }
  }
  __syncthreads();
  const bool direct = !CLUSTER && first_split == last_split;
  const int drow = decode_index[s];
  const int hq = hd >> 2;
  for (int idx = tid; idx < rows * hq; idx += NTHREADS) {
    const int r = idx / hq, d = (idx - r * hq) * 4;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, wml[(w * 16 + r) * 2]);
    float L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = wml[(w * 16 + r) * 2];
      if (mw == -INFINITY) continue;
      const float f = fast_exp2(mw - M);
      const float4 v = *reinterpret_cast<const float4*>(wo + (w * 16 + r) * ostride + d);
      L += wml[(w * 16 + r) * 2 + 1] * f;
      acc.x += v.x * f;
      acc.y += v.y * f;
      acc.z += v.z * f;
      acc.w += v.w * f;
    }
    const int head = head0 + r;
    if (direct) {
      const float inv = L > 0.0f ? 1.0f / L : 0.0f;
      bf16* op = out + ((size_t)q0 * nh + head) * hd + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    } else if (CLUSTER) {
      *reinterpret_cast<float4*>(co + r * ostride + d) = acc;
      if (d == 0) {
        cml[r * 2] = M;
        cml[r * 2 + 1] = L;
      }
    } else {
      const size_t prow = ((size_t)drow * nh + head) * nsplits + split;
      *reinterpret_cast<float4*>(part_o + prow * hd + d) = acc;
      if (d == 0) {
        part_ml[prow * 2] = M;
        part_ml[prow * 2 + 1] = L;
      }
    }
  }
  if (direct) return;

  if (CLUSTER) {
    // The splits of one (request, kv head) are the CTAs of one cluster: every CTA merges a share of the
    // output columns over all of them through distributed shared memory, in split order.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int csize = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    for (int idx = tid * csize + crank; idx < rows * hq; idx += NTHREADS * csize) {
      const int r = idx / hq, d = (idx - r * hq) * 4;
      float ms[8], ls[8];
      float4 vs4[8];
      float M = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < csize) {
          const float* rml = cluster.map_shared_rank(cml, c);
          const float* rco = cluster.map_shared_rank(co, c);
          ms[c] = rml[r * 2];
          ls[c] = rml[r * 2 + 1];
          vs4[c] = *reinterpret_cast<const float4*>(rco + r * ostride + d);
          M = fmaxf(M, ms[c]);
        }
      }
      float L = 0.0f;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < csize && ms[c] != -INFINITY) {
          const float f = fast_exp2(ms[c] - M);
          L += ls[c] * f;
          acc.x += vs4[c].x * f;
          acc.y += vs4[c].y * f;
          acc.z += vs4[c].z * f;
          acc.w += vs4[c].w * f;
        }
      }
      const float inv = L > 0.0f ? 1.0f / L : 0.0f;
      bf16* op = out + ((size_t)q0 * nh + head0 + r) * hd + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
    cluster.sync();  // nobody's shared memory goes away while another CTA still reads it
    return;
  }

  // Without a cluster: the CTA that finishes last among this (request, kv head) group's splits merges
  // them, in split order, so the result does not depend on which CTA that is. The counter returns to zero.
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* cnt = counters + (size_t)drow * gridDim.y + blockIdx.y;
    const int prev = atomicAdd(cnt, 1);
    s_last = (prev == last_split - first_split);
    if (s_last) *cnt = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int nv = last_split - first_split + 1;
  float* sml = reinterpret_cast<float*>(kvs);  // [rows][nv][2]
  for (int idx = tid; idx < rows * nv; idx += NTHREADS) {
    const int r = idx / nv, sp = idx - r * nv;
    const size_t prow = ((size_t)drow * nh + head0 + r) * nsplits + first_split + sp;
    sml[idx * 2] = __ldcg(part_ml + prow * 2);
    sml[idx * 2 + 1] = __ldcg(part_ml + prow * 2 + 1);
  }
  __syncthreads();
  // four output columns per thread; the loads of up to 8 splits are in flight together
  for (int idx = tid; idx < rows * hq; idx += NTHREADS) {
    const int r = idx / hq, d = (idx - r * hq) * 4;
    const float* ml = sml + (size_t)r * nv * 2;
    float M = -INFINITY;
    for (int sp = 0; sp < nv; ++sp) M = fmaxf(M, ml[sp * 2]);
    const float* po = part_o + (((size_t)drow * nh + head0 + r) * nsplits + first_split) * hd + d;
    float L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int sp0 = 0; sp0 < nv; sp0 += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (sp0 + u < nv) v[u] = __ldcg(reinterpret_cast<const float4*>(po + (size_t)(sp0 + u) * hd));
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (sp0 + u < nv) {
          const float ms = ml[(sp0 + u) * 2];
          const float f = (ms == -INFINITY) ? 0.0f : fast_exp2(ms - M);
          L += ml[(sp0 + u) * 2 + 1] * f;
          acc.x += v[u].x * f;
          acc.y += v[u].y * f;
          acc.z += v[u].z * f;
          acc.w += v[u].w * f;
        }
      }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    bf16* op = out + ((size_t)q0 * nh + head0 + r) * hd + d;
    *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  }
}

template <int HD_MAX>
int launch_prefill(bf16* out, const bf16* q, int q_row_stride, const bf16* kc, const bf16* vc, const int* bt,
                   int bt_stride, const int* cu_q, const int* seq_lens, int S, int nh, int nkv, int hd, int log2ps,
                   int num_pages, float scale_log2, int window, int max_q_len, int skip_single, cudaStream_t stream) {
  const size_t smem = (size_t)(64 + 4 * TILE_N) * (hd + 8) * sizeof(bf16);
  auto k = attn_prefill_kernel<HD_MAX>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const dim3 grid((max_q_len + 63) / 64, nh, S);
  k<<<grid, NTHREADS, smem, stream>>>(out, q, q_row_stride, kc, vc, bt, bt_stride, cu_q, seq_lens, nh, nkv, hd, log2ps,
                                      num_pages, scale_log2, window, skip_single);
  return osb_last_error();
}

template <int HD_MAX, int STAGES>
int launch_decode(bf16* out, float* part_o, float* part_ml, const bf16* q, int q_row_stride, const bf16* kc,
                  const bf16* vc, const int* bt, int bt_stride, const int* cu_q, const int* seq_lens,
                  const int* decode_index, int* counters, int S, int nh, int nkv, int hd, int log2ps, int num_pages,
                  float scale_log2, int window, int chunk, int nsplits, cudaStream_t stream,
                  FusedRope fr = FusedRope{nullptr, nullptr, nullptr, 0}, bool use_cluster = false) {
  // stage buffers; after the main loop they hold the warps' and the CTA's fp32 results
  size_t smem = (size_t)(16 + STAGES * 2 * TILE_N) * (hd + 8) * sizeof(bf16);
  const size_t merge = (size_t)16 * (hd + 8) * sizeof(bf16) + (size_t)5 * 16 * (hd + 8) * sizeof(float);
  if (merge > smem) smem = merge;
  const int g = nh / nkv;
  const dim3 grid(nsplits, nkv * ((g + 15) / 16), S);
  int rc;
  if (use_cluster && nsplits > 1 && nsplits <= 8) {
    auto k = attn_decode_kernel<HD_MAX, STAGES, true>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    rc = osb_launch_cluster(k, grid, dim3(NTHREADS), smem, stream, nsplits, out, part_o, part_ml, q, q_row_stride, kc,
                            vc, bt, bt_stride, cu_q, seq_lens, decode_index, counters, nh, nkv, hd, log2ps, num_pages,
                            scale_log2, window, chunk, nsplits, fr);
  } else {
    auto k = attn_decode_kernel<HD_MAX, STAGES, false>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    rc = osb_launch(k, grid, dim3(NTHREADS), smem, stream, out, part_o, part_ml, q, q_row_stride, kc, vc, bt,
                    bt_stride, cu_q, seq_lens, decode_index, counters, nh, nkv, hd, log2ps, num_pages, scale_log2,
                    window, chunk, nsplits, fr);
  }
  return rc ? rc : osb_last_error();
}
}  // namespace

// Scratch needed by the decode path: floats of part_o and of part_ml for n_decode requests.
OSB_API void osb_attn_decode_scratch(int n_decode, int nh, int nkv, int hd, int nsplits, long long* o_floats,
                                     long long* ml_floats, long long* counter_ints) {
  *o_floats = (long long)n_decode * nh * nsplits * hd;
  *ml_floats = (long long)n_decode * nh * nsplits * 2;
  *counter_ints = (long long)n_decode * nkv * ((nh / nkv + 15) / 16);
}

constexpr int MAX_SPLITS = 128;

// log2 of a page size the tensor-core kernels take (a power of two from 2 up), else -1
static inline int page_log2(int page_size) {
  if (page_size < 2 || (page_size & (page_size - 1))) return -1;
  int l = 0;
  while ((1 << l) < page_size) ++l;
  return l;
}
// out [T, nh*hd] bf16. Requests with one token run through the split-key decode kernel when
// n_decode > 0 (decode_index[s] = index among them; part_o/part_ml/counters sized by
// osb_attn_decode_scratch, counters all zero before the first use (the kernel leaves them zero);
// chunk a multiple of 64, nsplits = ceil(max_kv_len / chunk) <= 128); all others (and all, when
// n_decode == 0) through the prefill kernel. rope_cos/rope_sin [T, rope_rot/2] and rope_slot_map [T],
// when given, make the decode kernel rotate q and k itself and store the new key and value (the
// caller then skips the separate rotary/cache-write kernel); allowed only when n_multi == 0.
// use_cluster: with 2..8 splits, launch the splits of a request as one thread-block cluster and merge
// them through distributed shared memory (no scratch, no second phase through global memory).
OSB_API int osb_paged_attn_bf16(void* out, const void* q, int q_row_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int bt_stride, const int* cu_q, const int* seq_lens,
                                const int* decode_index, int S, int nh, int nkv, int hd, int page_size, int num_pages,
                                float scale, int window, int max_q_len, int n_decode, int n_multi, float* part_o,
                                float* part_ml, int* counters, int chunk, int nsplits, const float* rope_cos,
                                const float* rope_sin, const int* rope_slot_map, int rope_rot, int use_cluster,
                                cudaStream_t stream) {
  if (S <= 0) return OSB_OK;
  if (hd <= 0 || hd % 16 != 0 || hd > 256 || nkv <= 0 || nh % nkv != 0) return OSB_ERR_UNSUPPORTED;
  const int log2ps = page_log2(page_size);
  if (log2ps < 0) return OSB_ERR_UNSUPPORTED;
  if (n_decode > 0 && (chunk <= 0 || chunk % TILE_N != 0 || nsplits <= 0 || nsplits > MAX_SPLITS))
    return OSB_ERR_BAD_SHAPE;
  if (use_cluster && (nsplits < 2 || nsplits > 8)) use_cluster = 0;
  if (n_decode > 0 && nsplits > 1 && !use_cluster && (part_o == nullptr || part_ml == nullptr || counters == nullptr))
    return OSB_ERR_BAD_SHAPE;
  FusedRope fr{rope_cos, rope_sin, rope_slot_map, rope_rot};
  if (rope_cos != nullptr) {
    // the fused form covers steps of single-token requests only, with groups of at most 16 heads
    if (n_multi > 0 || nh / nkv > 16 || rope_sin == nullptr || rope_slot_map == nullptr || rope_rot <= 0 ||
        rope_rot > hd || (rope_rot & 1))
      return OSB_ERR_UNSUPPORTED;
  }
  const float scale_log2 = scale * LOG2E;
  bf16* o = (bf16*)out;
  const bf16 *qq = (const bf16*)q, *kc = (const bf16*)k_cache, *vc = (const bf16*)v_cache;
  int rc = OSB_OK;
  if (n_multi > 0 || n_decode == 0) {
    const int skip = n_decode > 0 ? 1 : 0;
    if (hd <= 64)
      rc = launch_prefill<64>(o, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, hd,
                              log2ps, num_pages, scale_log2, window, max_q_len, skip, stream);
    else if (hd <= 128)
      rc = launch_prefill<128>(o, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, hd,
                               log2ps, num_pages, scale_log2, window, max_q_len, skip, stream);
    else
      rc = launch_prefill<256>(o, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, hd,
                               log2ps, num_pages, scale_log2, window, max_q_len, skip, stream);
    if (rc != 0) return rc;
  }
  if (n_decode > 0) {
    static int n_sms = 0;
    if (n_sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0) n_sms = 148;
    }
    const long long decode_ctas = (long long)nsplits * nkv * ((nh / nkv + 15) / 16) * n_decode;
    const bool two_stages = decode_ctas > 2LL * n_sms;
    if (hd <= 64)
      rc = launch_decode<64, 3>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                nsplits, stream, fr, use_cluster != 0);
    else if (hd <= 128 && two_stages)
      rc = launch_decode<128, 2>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                 decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                 nsplits, stream, fr, use_cluster != 0);
    else if (hd <= 128)
      rc = launch_decode<128, 3>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                 decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                 nsplits, stream, fr, use_cluster != 0);
    else
      rc = launch_decode<256, 2>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                 decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                 nsplits, stream, fr, use_cluster != 0);
  }
  return rc;
}

// ------------------------------------------------------------------------------------------------

// Decode attention for callers that cannot allocate (declared in attn_decode_noalloc.h).
//
// The split-key decode kernel above needs scratch memory for the splits' partial results. Some
// hosts of this library have no way to provide it: a runtime that hands out all device memory at
// start-up and forbids cudaMalloc afterwards, a plug-in running inside another process's memory
// budget, code on a latency path where an allocator call is not allowed. For them this entry point
// keeps the scratch inside the library, in a fixed array in device memory.
namespace {
constexpr long long NOALLOC_SCRATCH_FLOATS = 1ll << 20;  // 4 MiB per GPU that loads the library
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

OSB_API long long osb_attn_decode_noalloc_capacity() { return NOALLOC_SCRATCH_FLOATS; }

OSB_API int osb_attn_decode_noalloc(void* out, const void* q, int q_row_stride, const void* k_cache,
                                    const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                                    const int* seq_lens, const int* decode_index, int S, int nh, int nkv, int hd,
                                    int page_size, int num_pages, float scale, int window, int n_decode, int chunk,
                                    int nsplits, cudaStream_t stream) {
  if (S <= 0 || n_decode <= 0) return OSB_OK;
  if (hd <= 0 || hd % 16 != 0 || hd > 256 || nkv <= 0 || nh % nkv != 0) return OSB_ERR_UNSUPPORTED;
  if (chunk <= 0 || chunk % TILE_N != 0 || nsplits <= 0 || nsplits > MAX_SPLITS) return OSB_ERR_BAD_SHAPE;
  const int log2ps = page_log2(page_size);
  if (log2ps < 0) return OSB_ERR_UNSUPPORTED;
  long long o_floats, ml_floats, counter_ints;
  osb_attn_decode_scratch(n_decode, nh, nkv, hd, nsplits, &o_floats, &ml_floats, &counter_ints);
  // layout of the array: counters | part_o | part_ml, each starting on a 256-byte boundary
  const long long o_offset = (counter_ints + 63) / 64 * 64;
  const long long ml_offset = o_offset + (o_floats + 63) / 64 * 64;
  if (nsplits > 1 && ml_offset + ml_floats > NOALLOC_SCRATCH_FLOATS) return OSB_ERR_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return OSB_ERR_UNSUPPORTED;
  if (g_noalloc_ptr[dev] == nullptr) {
    // In host code the array's name is not a device address; ask the runtime for the address on
    // the current device, once per device.
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = p;
  }
  int* counters = reinterpret_cast<int*>(g_noalloc_ptr[dev]);
  float* part_o = g_noalloc_ptr[dev] + o_offset;
  float* part_ml = g_noalloc_ptr[dev] + ml_offset;
  if (nsplits > 1) {
    // The counters are the one part of the array that must start at zero. A completed call leaves
    // them zero, but the array is shared and keeps whatever the last call left (an aborted launch,
    // another shape), so they are cleared on the stream before every launch.
    e = cudaMemsetAsync(counters, 0, (size_t)counter_ints * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
  }
  const float scale_log2 = scale * LOG2E;
  bf16* o = (bf16*)out;
  const bf16 *qq = (const bf16*)q, *kc = (const bf16*)k_cache, *vc = (const bf16*)v_cache;
  if (hd <= 64)
    return launch_decode<64, 3>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                nsplits, stream);
  if (hd <= 128)
    return launch_decode<128, 3>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                 decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                                 nsplits, stream);
  return launch_decode<256, 2>(o, part_o, part_ml, qq, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                               decode_index, counters, S, nh, nkv, hd, log2ps, num_pages, scale_log2, window, chunk,
                               nsplits, stream);
}
