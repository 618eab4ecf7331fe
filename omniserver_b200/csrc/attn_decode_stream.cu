// Decode attention (one new token per request) that streams keys and values from the cache pages straight
// into MMA operand registers: no shared-memory tiles, no cp.async pipeline, no block-wide barrier in the
// main loop. For head sizes 64 and 128, bf16.
//
// One CTA = one (request, kv head, split of the keys), eight warps. A warp takes blocks of 16 keys of the
// split in turn (warp w: blocks w, w + 8, ...), keeps the next block's loads in flight while it computes the
// current one and asks the L2 for the two after that. Every lane reads 16 bytes (8 consecutive dims) of one key.
// The query heads of the group (at most 8) are the N side of both products, keys and dims the M side, so one
// m16n8k16 MMA covers 16 keys (or 16 dims) for all heads:
//  * S^T[16 keys x 8 heads] = K Q^T: lane (g, c) holds K[keys g, g + 8][dims 32 Db + 8c .. + 7], which are the A
//    fragments of two MMAs whose summation index is permuted (k-slots {2c, 2c+1 | 2c+8, 2c+9} = dims 8c + {0, 1 |
//    2, 3}, then {4, 5 | 6, 7}); the B operand takes the same dims of Q[head g] from shared memory. A dot
//    product does not care about the order of its terms as long as both operands agree.
//  * O^T[16 dims x 8 heads] += V^T P^T: lane (g, c) holds V[keys g, g + 8][dims 32 Db + 8c .. + 7]; movmatrix
//    transposes each 32-bit piece across the warp, which turns it into an A fragment (two consecutive keys of
//    one dim); the row block (Db, jj) has pieces 2jj and 2jj + 1 as its rows 0-7 and 8-15, so that its row g
//    stands for dim 32 Db + 8 (g / 2) + 4 jj + g % 2 (+ 2 for row g + 8). P (keys x heads, out of the first
//    MMA) goes through movmatrix as well to become the B fragment.
// The splits of a request are equal parts of its own visible keys (whole blocks), whatever the longest request
// of the batch is. Masks, the fused rotary form (this kernel rotates q and k and stores the new key and value)
// and the merges (eight warps through shared memory; splits through distributed shared memory of a cluster,
// or through scratch memory by the CTA that finishes last) are those of attn_decode_kernel in attn_mma.cu;
// semantics as there (omniserve/model/qwen2_llm.py:96-112, omniserve/cache/kv_prealloc.py:138-142).
#include <cooperative_groups.h>

#include "mma_utils.cuh"

namespace cg = cooperative_groups;

namespace attn_stream {
constexpr int NW = 8;              // warps per CTA
constexpr int NT = NW * 32;
constexpr int BLK = 16;            // keys per block
constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t MERGE_WAIT_LIMIT = 1u << 20;   // polls of a group's counter before the merging CTA gives up
enum : int { ERR_MERGE_WAIT = 141 };

struct FusedRope {
  const float* cos_t;
  const float* sin_t;
  const int* slot_map;
  int rot;
};

__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
  unsigned d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// through the L2 only (the L1 is not asked to keep lines that are read once)
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// K and V of one block of 16 keys as this lane needs them: [half of the block: keys 8h + g][32-dim block Db]
template <int NDB>
struct KVRegs {
  uint4 k[2][NDB], v[2][NDB];
};


// One (request, kv head, split of the keys): the whole CTA (eight warps). ``wait_for_q`` waits for the kernel in front
// (programmatic dependent launch); nothing of this step's q, k, v is touched before it.
template <int HD, bool CLUSTER, class WaitFn>
__device__ __forceinline__ void attn_stream_unit(
    WaitFn&& wait_for_q, int split_, int by_, int s_, int ny_, unsigned char* smem_raw,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
    int q_row_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
    const int* __restrict__ decode_index, int* __restrict__ counters, int nh, int nkv, int log2ps, int num_pages,
    float scale_log2, int window, int chunk, int nsplits, FusedRope fr, int* __restrict__ err) {
  constexpr int NDB = HD / 32;     // 32-dim blocks
  constexpr int stride = HD + 8;   // q rows in shared memory, bf16
  constexpr int ostride = HD + 8;  // merge rows, fp32
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                     // [16][stride]
  float* wml = reinterpret_cast<float*>(qs + 16 * stride);          // [NW][16][2], then the CTA's own [16][2]
  float* cml = wml + NW * 16 * 2;
  float* wo = cml + 16 * 2;                                         // [NW][16][ostride], then the CTA's own [16][ostride]
  float* co = wo + NW * 16 * ostride;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = split_, s = s_;
  const int grp = nh / nkv;
  const int head_tiles = (grp + 7) >> 3;
  const int kvh = by_ / head_tiles, ht = by_ - kvh * head_tiles;
  const int q0 = cu_q[s];
  if (cu_q[s + 1] - q0 != 1) return;
  const int rows = min(8, grp - ht * 8);
  const int head0 = kvh * grp + ht * 8;
  const int kv_len = seq_lens[s];
  const int p = kv_len - 1;
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  // The visible keys [lo, kv_len) of this request are cut into nsplits equal parts of whole 16-key blocks, from
  // this request's own length: the splits stay balanced whatever the longest request of the batch is.
  (void)chunk;
  const int lo16 = (lo / BLK) * BLK;
  const int per = ((kv_len - lo16 + nsplits - 1) / nsplits + BLK - 1) / BLK * BLK;
  const int first_split = 0, last_split = (p - lo16) / per;
  const bool active = split <= last_split;
  if (!CLUSTER && !active) return;
  const int k_begin = lo16 + split * per;
  const int k_end = min(k_begin + per, kv_len);
  const int nblk = active ? (k_end - k_begin + BLK - 1) / BLK : 0;
  const int* bt = block_table + (size_t)s * bt_stride;
  const int ps_mask = (1 << log2ps) - 1;
  const size_t page_stride = ((size_t)nkv << log2ps) * HD;
  const size_t head_off = ((size_t)kvh << log2ps) * HD;

  // the pages of this lane's two keys (g and g + 8) of block b, or -1 (outside [lo, k_end), page given back)
  auto pages_of = [&](int b) -> int2 {
    int2 pg = make_int2(-1, -1);
    const int key = k_begin + b * BLK + g;
    if (b < nblk) {
      if (key < k_end && key >= lo) pg.x = bt[key >> log2ps];
      if (key + 8 < k_end && key + 8 >= lo) pg.y = bt[(key + 8) >> log2ps];
      if (pg.x >= num_pages) pg.x = -1;
      if (pg.y >= num_pages) pg.y = -1;
    }
    return pg;
  };
  // asks the L2 for block b (no registers held): the loads that follow later then come from the L2. Lanes c = 0, 1
  // take the two 128-byte halves of key g's row, lanes c = 2, 3 those of key g + 8.
  auto prefetch_block = [&](int b, int2 pg) {
    const int page = (c >> 1) ? pg.y : pg.x;
    if (page < 0 || (c & 1) * 64 >= HD) return;
    const int key = k_begin + b * BLK + g + 8 * (c >> 1);
    const size_t off = (size_t)page * page_stride + head_off + (size_t)(key & ps_mask) * HD + (c & 1) * 64;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + off));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + off));
  };
  // loads of block b: zeros for keys outside [lo, k_end) and for pages given back
  auto load_block = [&](int b, int2 pg, KVRegs<NDB>& r) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int key = k_begin + b * BLK + h * 8 + g;
      const int page = h ? pg.y : pg.x;
      const size_t off = page >= 0 ? (size_t)page * page_stride + head_off + (size_t)(key & ps_mask) * HD + c * 8 : 0;
#pragma unroll
      for (int db = 0; db < NDB; ++db) {
        r.k[h][db] = page >= 0 ? ld_cg16(kc + off + db * 32) : make_uint4(0u, 0u, 0u, 0u);
        r.v[h][db] = page >= 0 ? ld_cg16(vc + off + db * 32) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  // Everything read so far was written by the host before the step.
  KVRegs<NDB> cur, nxt;
  // In the fused rotary form no block depends on the kernel before this one: the new token's own key and value,
  // which only the last split sees, do not come from the cache (its row there is stale until this kernel has
  // stored it) but from shared memory, where this CTA puts them, and replace that row of the loaded block.
  const bool early = fr.cos_t != nullptr;
  bf16* ks = qs + 8 * stride;   // rows 8 and 9 of the q tile: heads are the N side, only rows 0-7 hold queries
  bf16* vs = qs + 9 * stride;
  // page ids of this warp's first four blocks in one round trip; then one block further every iteration
  int2 pg1 = pages_of(warp + NW), pg2 = pages_of(warp + 2 * NW), pg3 = pages_of(warp + 3 * NW);
  // With many CTAs the L2 is asked for the next blocks only after this step's q, k, v have been asked for (ahead
  // of them the requests of 128 CTAs stood in their way: 2.11 -> 2.07 ms a step at 64 requests); with few, at once
  // (1.017 -> 1.009 ms at one request).
  const bool crowded = gridDim.x * gridDim.y * gridDim.z >= 128;
  if (early) {
    load_block(warp, pages_of(warp), cur);
    if (!crowded) {
      prefetch_block(warp + NW, pg1);
      prefetch_block(warp + 2 * NW, pg2);
    }
  }
  // Before the wait: what the host or an earlier kernel of the step wrote (the slot of the new token, the rotary
  // tables). After it: this step's q, k, v, every load issued before any is used (a thread has at most one item of
  // each kind), so that the whole preparation costs one round trip to the L2 and not one per piece.
  constexpr int cpr = HD >> 3;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const bool do_kv = fr.cos_t != nullptr && split == last_split;
  const int half = fr.rot >> 1, hc = half >> 3;
  const bool rotate_here = fr.cos_t != nullptr && (half & 7) == 0;   // q rotated on its way into shared memory
  const int per_row = rotate_here ? hc + (cpr - 2 * hc) : cpr;       // this thread's piece of the q tile: (row, piece)
  const int qi_r = tid / per_row, qi_c = tid - qi_r * per_row;
  const bool q_item = tid < 8 * per_row, q_live = q_item && qi_r < rows, q_rot = rotate_here && q_live && qi_c < hc;
  float4 qc0 = make_float4(0.f, 0.f, 0.f, 0.f), qc1 = qc0, qs0 = qc0, qs1 = qc0;
  float k_cs = 0.0f, k_sn = 0.0f;
  int slot = -1;
  if (q_rot) {
    const float* cs = fr.cos_t + (size_t)q0 * half + qi_c * 8;
    const float* sn = fr.sin_t + (size_t)q0 * half + qi_c * 8;
    qc0 = *reinterpret_cast<const float4*>(cs);
    qc1 = *reinterpret_cast<const float4*>(cs + 4);
    qs0 = *reinterpret_cast<const float4*>(sn);
    qs1 = *reinterpret_cast<const float4*>(sn + 4);
  }
  if (do_kv) {
    slot = fr.slot_map[q0];
    if (tid < half) {
      k_cs = fr.cos_t[(size_t)q0 * half + tid];
      k_sn = fr.sin_t[(size_t)q0 * half + tid];
    }
  }
  wait_for_q();   // until here nothing of this step's q, k, v was touched
  const bf16* qsrc = q + (size_t)q0 * q_row_stride + (size_t)(head0 + (q_item ? qi_r : 0)) * HD;
  uint4 qa = zero4, qb = zero4;
  if (q_live) {
    if (q_rot) {
      qa = *reinterpret_cast<const uint4*>(qsrc + qi_c * 8);
      qb = *reinterpret_cast<const uint4*>(qsrc + half + qi_c * 8);
    } else {
      qa = *reinterpret_cast<const uint4*>(qsrc + (rotate_here ? 2 * hc + (qi_c - hc) : qi_c) * 8);
    }
  }
  bf16 kx1 = __float2bfloat16_rn(0.0f), kx2 = kx1, kpl = kx1, vv = kx1;
  if (do_kv) {
    const bf16* ksrc = q + (size_t)q0 * q_row_stride + (size_t)(nh + kvh) * HD;
    const bf16* vsrc = q + (size_t)q0 * q_row_stride + (size_t)(nh + nkv + kvh) * HD;
    if (tid < half) {
      kx1 = ksrc[tid];
      kx2 = ksrc[tid + half];
    }
    if (fr.rot + tid < HD) kpl = ksrc[fr.rot + tid];
    if (tid < HD) vv = vsrc[tid];
  }
  if (early && crowded) {
    prefetch_block(warp + NW, pg1);
    prefetch_block(warp + 2 * NW, pg2);
  }
  if (do_kv) {
    // the new token's key (rotated) and value: into shared memory for this CTA's own block, and, by one CTA of the
    // kv head, into the cache page
    const int page = slot >> log2ps, off = slot & ps_mask;
    const bool store = ht == 0 && page >= 0 && page < num_pages;
    const size_t dst = store ? ((((size_t)page * nkv + kvh) << log2ps) + off) * HD : 0;
    bf16* kd = const_cast<bf16*>(kc) + dst;
    bf16* vd = const_cast<bf16*>(vc) + dst;
    if (tid < half) {
      const float x1 = __bfloat162float(kx1), x2 = __bfloat162float(kx2);
      const bf16 ra = __float2bfloat16_rn(x1 * k_cs - x2 * k_sn), rb = __float2bfloat16_rn(x2 * k_cs + x1 * k_sn);
      ks[tid] = ra;
      ks[tid + half] = rb;
      if (store) {
        kd[tid] = ra;
        kd[tid + half] = rb;
      }
    }
    if (fr.rot + tid < HD) {
      ks[fr.rot + tid] = kpl;
      if (store) kd[fr.rot + tid] = kpl;
    }
    if (tid < HD) {
      vs[tid] = vv;
      if (store) vd[tid] = vv;
    }
  }
  if (!early) {
    load_block(warp, pages_of(warp), cur);
    prefetch_block(warp + NW, pg1);
    prefetch_block(warp + 2 * NW, pg2);
  }

  // the group's query rows into shared memory, rotated on the way in the fused rotary form
  if (q_item) {
    bf16* dstq = qs + qi_r * stride;
    if (q_rot) {
      const float cv[8] = {qc0.x, qc0.y, qc0.z, qc0.w, qc1.x, qc1.y, qc1.z, qc1.w};
      const float sv[8] = {qs0.x, qs0.y, qs0.z, qs0.w, qs1.x, qs1.y, qs1.z, qs1.w};
      __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&qa);
      __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&qb);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x1 = __bfloat1622float2(pa[e]), x2 = __bfloat1622float2(pb[e]);
        pa[e] = __floats2bfloat162_rn(x1.x * cv[2 * e] - x2.x * sv[2 * e], x1.y * cv[2 * e + 1] - x2.y * sv[2 * e + 1]);
        pb[e] = __floats2bfloat162_rn(x2.x * cv[2 * e] + x1.x * sv[2 * e], x2.y * cv[2 * e + 1] + x1.y * sv[2 * e + 1]);
      }
      *reinterpret_cast<uint4*>(dstq + qi_c * 8) = qa;
      *reinterpret_cast<uint4*>(dstq + half + qi_c * 8) = qb;
    } else if (rotate_here && qi_c >= hc) {
      *reinterpret_cast<uint4*>(dstq + (2 * hc + (qi_c - hc)) * 8) = qa;   // zeros in rows beyond the group's heads
    } else if (rotate_here) {
      // a row beyond the group's heads in the rotated span: zeros in both halves
      *reinterpret_cast<uint4*>(dstq + qi_c * 8) = zero4;
      *reinterpret_cast<uint4*>(dstq + half + qi_c * 8) = zero4;
    } else {
      *reinterpret_cast<uint4*>(dstq + qi_c * 8) = qa;
    }
  }
  if (fr.cos_t != nullptr && !rotate_here) {  // a rotated span that is no multiple of 16: rotate in place
    __syncthreads();
    const float* cs = fr.cos_t + (size_t)q0 * half;
    const float* sn = fr.sin_t + (size_t)q0 * half;
    for (int i = tid; i < rows * half; i += NT) {
      const int r = i / half, d = i - r * half;
      bf16* row = qs + r * stride;
      const float x1 = __bfloat162float(row[d]), x2 = __bfloat162float(row[d + half]);
      row[d] = __float2bfloat16_rn(x1 * cs[d] - x2 * sn[d]);
      row[d + half] = __float2bfloat16_rn(x2 * cs[d] + x1 * sn[d]);
    }
  }
  __syncthreads();

  // Heads are the N side of both products (at most 8 per kv head), keys and dims the M side:
  //   S^T[16 keys x 8 heads]  = K[16 keys x dims] Q^T          (A = K straight from the loads, B = Q from smem)
  //   O^T[16 dims x 8 heads] += V^T[16 dims x 16 keys] P^T      (A = V through movmatrix, B = P through movmatrix)
  // Lane (g, c) owns heads 2c, 2c+1: of S^T the keys g and g + 8 of the block; of O^T, in row block (db, jj),
  // the dims 32 db + 8 (g / 2) + 4 jj + g % 2 and that + 2.
  float ot[NDB * 2][4];
#pragma unroll
  for (int i = 0; i < NDB * 2; ++i) ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // per head 2c, 2c+1; l_run: this lane's keys only

  for (int b = warp; b < nblk; b += NW) {
    const int2 pg4 = pages_of(b + 4 * NW);  // used one iteration later
    load_block(b + NW, pg1, nxt);          // in flight while this block is computed (zeros beyond the last block)
    prefetch_block(b + 3 * NW, pg3);
    pg1 = pg2;
    pg2 = pg3;
    pg3 = pg4;
    if (fr.cos_t != nullptr && split == last_split && (p - k_begin) / BLK == b && g == ((p - k_begin) & 7)) {
      // this lane holds the new token's row of the block: take it from shared memory
      if (((p - k_begin) & 8) == 0) {
#pragma unroll
        for (int db = 0; db < NDB; ++db) {
          cur.k[0][db] = *reinterpret_cast<const uint4*>(ks + db * 32 + c * 8);
          cur.v[0][db] = *reinterpret_cast<const uint4*>(vs + db * 32 + c * 8);
        }
      } else {
#pragma unroll
        for (int db = 0; db < NDB; ++db) {
          cur.k[1][db] = *reinterpret_cast<const uint4*>(ks + db * 32 + c * 8);
          cur.v[1][db] = *reinterpret_cast<const uint4*>(vs + db * 32 + c * 8);
        }
      }
    }
    float st[4] = {0.0f, 0.0f, 0.0f, 0.0f}, su[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // two chains of dependent MMAs
#pragma unroll
    for (int db = 0; db < NDB; ++db) {
      const uint4 qv = *reinterpret_cast<const uint4*>(qs + g * stride + db * 32 + c * 8);  // head g
      const unsigned a0[4] = {cur.k[0][db].x, cur.k[1][db].x, cur.k[0][db].y, cur.k[1][db].y};
      const unsigned a1[4] = {cur.k[0][db].z, cur.k[1][db].z, cur.k[0][db].w, cur.k[1][db].w};
      mma_bf16_16816(st, a0, qv.x, qv.y);
      mma_bf16_16816(su, a1, qv.z, qv.w);
    }
    // st[0], st[1]: key g, heads 2c, 2c+1; st[2], st[3]: key g + 8. Every head is the same query position: the
    // mask depends on the key only.
    const int kbase = k_begin + b * BLK;
    const bool vis0 = kbase + g < k_end && kbase + g >= lo, vis1 = kbase + g + 8 < k_end && kbase + g + 8 >= lo;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      st[e] = vis0 ? (st[e] + su[e]) * scale_log2 : -INFINITY;
      st[2 + e] = vis1 ? (st[2 + e] + su[2 + e]) * scale_log2 : -INFINITY;
    }
    float alpha[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {  // head 2c + e: maximum over the block's 16 keys (this lane's two, then the lanes g)
      float v = fmaxf(st[e], st[2 + e]);
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
      // m_run is the exponent offset in use; it moves only when the maximum has grown by more than 2^8
      const bool grow = v > m_run[e] + 8.0f || (m_run[e] == -INFINITY && v > -INFINITY);
      alpha[e] = (grow && m_run[e] != -INFINITY) ? fast_exp2(m_run[e] - v) : 1.0f;
      if (grow) m_run[e] = v;
      const float off = m_run[e];
      const float p0 = st[e] == -INFINITY ? 0.0f : fast_exp2(st[e] - off);
      const float p1 = st[2 + e] == -INFINITY ? 0.0f : fast_exp2(st[2 + e] - off);
      st[e] = p0;
      st[2 + e] = p1;
      l_run[e] = l_run[e] * alpha[e] + p0 + p1;
    }
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < NDB * 2; ++i) {
        ot[i][0] *= alpha[0];
        ot[i][1] *= alpha[1];
        ot[i][2] *= alpha[0];
        ot[i][3] *= alpha[1];
      }
    }
    // P (keys x heads) transposed across the warp is the B operand: keys 2c, 2c+1 (and + 8) of head g
    const unsigned pb0 = movmatrix_trans(pack_bf16(st[0], st[1]));
    const unsigned pb1 = movmatrix_trans(pack_bf16(st[2], st[3]));
#pragma unroll
    for (int db = 0; db < NDB; ++db) {
      const unsigned t00 = movmatrix_trans(cur.v[0][db].x), t01 = movmatrix_trans(cur.v[0][db].y);
      const unsigned t02 = movmatrix_trans(cur.v[0][db].z), t03 = movmatrix_trans(cur.v[0][db].w);
      const unsigned t10 = movmatrix_trans(cur.v[1][db].x), t11 = movmatrix_trans(cur.v[1][db].y);
      const unsigned t12 = movmatrix_trans(cur.v[1][db].z), t13 = movmatrix_trans(cur.v[1][db].w);
      const unsigned va0[4] = {t00, t01, t10, t11};  // rows g: piece 0, rows g + 8: piece 1; keys 0-7 | 8-15
      const unsigned va1[4] = {t02, t03, t12, t13};
      mma_bf16_16816(ot[db * 2], va0, pb0, pb1);
      mma_bf16_16816(ot[db * 2 + 1], va1, pb0, pb1);
    }
    cur = nxt;
  }
  pdl_trigger();

  // merge the warps (each saw different keys) in warp order through shared memory
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float l = l_run[e];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    const int r = 2 * c + e;  // head
    if (r < rows) {
      if (g == 0) {
        wml[(warp * 16 + r) * 2] = m_run[e];
        wml[(warp * 16 + r) * 2 + 1] = l;
      }
#pragma unroll
      for (int db = 0; db < NDB; ++db)
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int d = db * 32 + (g >> 1) * 8 + jj * 4 + (g & 1);
          wo[(warp * 16 + r) * ostride + d] = ot[db * 2 + jj][e];
          wo[(warp * 16 + r) * ostride + d + 2] = ot[db * 2 + jj][2 + e];
        }
    }
  }
  __syncthreads();
  const bool direct = !CLUSTER && first_split == last_split;
  const bool merger = !CLUSTER && split == last_split;   // without a cluster: the CTA of the last split merges
  const int drow = decode_index[s];
  constexpr int hq = HD >> 2;
  static_assert(8 * hq <= NT, "a thread has at most one (head, four dims) of the CTA's result");
  float my_m = -INFINITY, my_l = 0.0f;   // the merging CTA keeps its own partial result in registers
  float4 my_acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int idx = tid; idx < rows * hq; idx += NT) {
    const int r = idx / hq, d = (idx - r * hq) * 4;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, wml[(w * 16 + r) * 2]);
    float L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
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
      bf16* op = out + ((size_t)q0 * nh + head) * HD + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    } else if (CLUSTER) {
      *reinterpret_cast<float4*>(co + r * ostride + d) = acc;
      if (d == 0) {
        cml[r * 2] = M;
        cml[r * 2 + 1] = L;
      }
    } else if (merger) {
      my_m = M;
      my_l = L;
      my_acc = acc;
    } else {
      const size_t prow = ((size_t)drow * nh + head) * nsplits + split;
      *reinterpret_cast<float4*>(part_o + prow * HD + d) = acc;
      if (d == 0) {
        part_ml[prow * 2] = M;
        part_ml[prow * 2 + 1] = L;
      }
    }
  }
  if (direct) return;

  if (CLUSTER) {
    // the splits of one (request, kv head) are the CTAs of one cluster: every CTA merges a share of the
    // output columns over all of them through distributed shared memory, in split order
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int csize = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    for (int idx = tid * csize + crank; idx < rows * hq; idx += NT * csize) {
      const int r = idx / hq, d = (idx - r * hq) * 4;
      float ms[8], ls[8];
      float4 vs4[8];
      float M = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        if (cc < csize) {
          const float* rml = cluster.map_shared_rank(cml, cc);
          const float* rco = cluster.map_shared_rank(co, cc);
          ms[cc] = rml[r * 2];
          ls[cc] = rml[r * 2 + 1];
          vs4[cc] = *reinterpret_cast<const float4*>(rco + r * ostride + d);
          M = fmaxf(M, ms[cc]);
        }
      }
      float L = 0.0f;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        if (cc < csize && ms[cc] != -INFINITY) {
          const float f = fast_exp2(ms[cc] - M);
          L += ls[cc] * f;
          acc.x += vs4[cc].x * f;
          acc.y += vs4[cc].y * f;
          acc.z += vs4[cc].z * f;
          acc.w += vs4[cc].w * f;
        }
      }
      const float inv = L > 0.0f ? 1.0f / L : 0.0f;
      bf16* op = out + ((size_t)q0 * nh + head0 + r) * HD + d;
      *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
    cluster.sync();  // nobody's shared memory goes away while another CTA still reads it
    return;
  }

  // Without a cluster: the CTA of the last split (the highest block index of its group, so the others were handed
  // to SMs before it) merges. The others put their partial results into global memory, add one to the group's
  // counter without waiting for the answer, and are done. The merging CTA keeps its own partial result in
  // registers, waits (bounded) until the counter says that all others have arrived, puts the counter back to zero,
  // and folds the others' results into its own in split order, fetching (max, sum) and outputs of up to eight
  // splits in one round trip. The launcher only takes this path when all CTAs of the grid fit on the GPU at once.
  int* cnt = counters + (size_t)drow * ny_ + by_;
  if (!merger) {
    __threadfence();
    __syncthreads();
    if (tid == 0) atomicAdd(cnt, 1);   // the result is not used: nobody waits for it
    return;
  }
  const int others = last_split - first_split;
  if (tid == 0) {
    bool ok = false;
    for (uint32_t i = 0; i < MERGE_WAIT_LIMIT && !ok; ++i) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
      ok = v >= others;
    }
    if (!ok) atomicExch(err, ERR_MERGE_WAIT);
    *cnt = 0;
  }
  __syncthreads();
  if (tid < rows * hq) {
    const int r = tid / hq, d = (tid - r * hq) * 4;
    const size_t prow0 = ((size_t)drow * nh + head0 + r) * nsplits + first_split;
    float M = my_m, L = my_l;
    float4 acc = my_acc;
    for (int sp0 = 0; sp0 < others; sp0 += 8) {
      float2 ml[8];
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (sp0 + u < others) {
          ml[u] = __ldcg(reinterpret_cast<const float2*>(part_ml + (prow0 + sp0 + u) * 2));
          v[u] = __ldcg(reinterpret_cast<const float4*>(part_o + (prow0 + sp0 + u) * HD + d));
        }
      float Mc = M;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (sp0 + u < others) Mc = fmaxf(Mc, ml[u].x);
      if (Mc == -INFINITY) continue;
      const float keep = M == -INFINITY ? 0.0f : fast_exp2(M - Mc);
      L *= keep;
      acc.x *= keep;
      acc.y *= keep;
      acc.z *= keep;
      acc.w *= keep;
      M = Mc;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (sp0 + u < others && ml[u].x != -INFINITY) {
          const float f = fast_exp2(ml[u].x - M);
          L += ml[u].y * f;
          acc.x += v[u].x * f;
          acc.y += v[u].y * f;
          acc.z += v[u].z * f;
          acc.w += v[u].w * f;
        }
      }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    bf16* op = out + ((size_t)q0 * nh + head0 + r) * HD + d;
    *reinterpret_cast<__nv_bfloat162*>(op) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    *reinterpret_cast<__nv_bfloat162*>(op + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  }
}

}  // namespace attn_stream


namespace {
using namespace attn_stream;

template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(NT, 1) attn_decode_stream_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
    int q_row_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
    const int* __restrict__ decode_index, const int* __restrict__ order, int* __restrict__ counters, int nh, int nkv,
    int log2ps, int num_pages, float scale_log2, int window, int chunk, int nsplits, FusedRope fr, int* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // CTAs are handed to the SMs in the order of their indices: `order` (the requests by falling length) lets the long
  // ones start first, so that, when there are more CTAs than SMs, the short ones fill the gaps at the end
  const int s = order != nullptr ? order[blockIdx.z] : (int)blockIdx.z;
  attn_stream_unit<HD, CLUSTER>([] { pdl_wait(); }, blockIdx.x, blockIdx.y, s, gridDim.y, smem_raw, out, part_o,
                                       part_ml, q, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                       decode_index, counters, nh, nkv, log2ps, num_pages, scale_log2, window, chunk,
                                       nsplits, fr, err);
}

template <int HD>
int launch(bf16* out, float* part_o, float* part_ml, const bf16* q, int q_row_stride, const bf16* kc, const bf16* vc,
           const int* bt, int bt_stride, const int* cu_q, const int* seq_lens, const int* decode_index, const int* order,
           int* counters, int S, int nh, int nkv, int log2ps, int num_pages, float scale_log2, int window, int chunk, int nsplits,
           cudaStream_t stream, FusedRope fr, bool use_cluster, int* err) {
  // q rows, the warps' (max, sum) and outputs, the CTA's own; the last CTA's table of (max, sum) of all splits
  size_t smem = (size_t)16 * (HD + 8) * sizeof(bf16) + (size_t)(NW + 1) * 16 * 2 * sizeof(float) +
                (size_t)(NW + 1) * 16 * (HD + 8) * sizeof(float);
  const int g = nh / nkv;
  const dim3 grid(nsplits, nkv * ((g + 7) / 8), S);
  int rc;
  if (use_cluster && nsplits > 1 && nsplits <= 8) {
    auto k = attn_decode_stream_kernel<HD, true>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    rc = osb_launch_cluster(k, grid, dim3(NT), smem, stream, nsplits, out, part_o, part_ml, q, q_row_stride, kc, vc, bt,
                            bt_stride, cu_q, seq_lens, decode_index, order, counters, nh, nkv, log2ps, num_pages, scale_log2,
                            window, chunk, nsplits, fr, err);
  } else {
    auto k = attn_decode_stream_kernel<HD, false>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    rc = osb_launch(k, grid, dim3(NT), smem, stream, out, part_o, part_ml, q, q_row_stride, kc, vc, bt, bt_stride, cu_q,
                    seq_lens, decode_index, order, counters, nh, nkv, log2ps, num_pages, scale_log2, window, chunk, nsplits, fr,
                    err);
  }
  return rc ? rc : osb_last_error();
}
}  // namespace

// The decode part of osb_paged_attn_bf16 (same arguments, same meaning; requests bringing more than one
// token are skipped) for head sizes 64 and 128 and page sizes that are powers of two; anything else is refused
// with OSB_ERR_UNSUPPORTED. chunk is a multiple of 64; with nsplits > 1 and no cluster, part_o / part_ml /
// counters as for osb_paged_attn_bf16; the CTA of a group's last split then waits (bounded; error 141 in *err) for the
// group's other splits, so the grid (nsplits x kv heads x head tiles x S) must fit on the GPU at once: a larger one is
// refused with OSB_ERR_TOO_LARGE (n_decode: how many of the S requests bring one token; 0: all of them).
// order: null, or a permutation of 0..S-1: the requests in the order in which their CTAs are to start.
OSB_API int osb_attn_decode_stream(void* out, const void* q, int q_row_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* seq_lens,
                                   const int* decode_index, const int* order, int S, int nh, int nkv, int hd, int page_size,
                                   int num_pages,
                                   float scale, int window, float* part_o, float* part_ml, int* counters, int chunk,
                                   int nsplits, const float* rope_cos, const float* rope_sin, const int* rope_slot_map,
                                   int rope_rot, int use_cluster, int n_decode, int* err, cudaStream_t stream) {
  if (S <= 0) return OSB_OK;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0) return OSB_ERR_UNSUPPORTED;
  if (page_size < 1 || (page_size & (page_size - 1))) return OSB_ERR_UNSUPPORTED;
  if ((q_row_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return OSB_ERR_UNSUPPORTED;
  if (chunk <= 0 || chunk % 64 != 0 || nsplits <= 0 || nsplits > 128) return OSB_ERR_BAD_SHAPE;
  if (use_cluster && (nsplits < 2 || nsplits > 8)) use_cluster = 0;
  if (nsplits > 1 && !use_cluster) {
    if (part_o == nullptr || part_ml == nullptr || counters == nullptr || err == nullptr) return OSB_ERR_BAD_SHAPE;
    // the CTA that merges a group's splits waits for the others: all CTAs must be on the GPU at the same time
    static int n_sms = 0;
    if (n_sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0) n_sms = 1;
    }
    // (n_decode: the requests of the step that bring one token; the CTAs of the others end at once)
    if (n_decode <= 0 || n_decode > S) n_decode = S;
    if ((long long)nsplits * nkv * ((nh / nkv + 7) / 8) * n_decode > n_sms) return OSB_ERR_TOO_LARGE;
  }
  FusedRope fr{rope_cos, rope_sin, rope_slot_map, rope_rot};
  if (rope_cos != nullptr) {
    if (nh / nkv > 8 || rope_sin == nullptr || rope_slot_map == nullptr || rope_rot <= 0 || rope_rot > hd || (rope_rot & 1))
      return OSB_ERR_UNSUPPORTED;
  }
  int log2ps = 0;
  while ((1 << log2ps) < page_size) ++log2ps;
  const float scale_log2 = scale * LOG2E;
  if (hd == 64)
    return launch<64>((bf16*)out, part_o, part_ml, (const bf16*)q, q_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
                      block_table, bt_stride, cu_q, seq_lens, decode_index, order, counters, S, nh, nkv, log2ps, num_pages,
                      scale_log2, window, chunk, nsplits, stream, fr, use_cluster != 0, err);
  return launch<128>((bf16*)out, part_o, part_ml, (const bf16*)q, q_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
                     block_table, bt_stride, cu_q, seq_lens, decode_index, order, counters, S, nh, nkv, log2ps, num_pages,
                     scale_log2, window, chunk, nsplits, stream, fr, use_cluster != 0, err);
}
