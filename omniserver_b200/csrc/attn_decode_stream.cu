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
#include "attn_decode_stream.cuh"

namespace {
using namespace attn_stream;

template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(NT, 1) attn_decode_stream_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q,
    int q_row_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
    const int* __restrict__ decode_index, int* __restrict__ counters, int nh, int nkv, int log2ps, int num_pages,
    float scale_log2, int window, int chunk, int nsplits, FusedRope fr) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_last;
  attn_stream_unit<HD, CLUSTER, false>([] { pdl_wait(); }, blockIdx.x, blockIdx.y, blockIdx.z, gridDim.y, smem_raw, &s_last, out, part_o,
                                       part_ml, q, q_row_stride, kc, vc, block_table, bt_stride, cu_q, seq_lens,
                                       decode_index, counters, nh, nkv, log2ps, num_pages, scale_log2, window, chunk,
                                       nsplits, fr);
}

template <int HD>
int launch(bf16* out, float* part_o, float* part_ml, const bf16* q, int q_row_stride, const bf16* kc, const bf16* vc,
           const int* bt, int bt_stride, const int* cu_q, const int* seq_lens, const int* decode_index, int* counters,
           int S, int nh, int nkv, int log2ps, int num_pages, float scale_log2, int window, int chunk, int nsplits,
           cudaStream_t stream, FusedRope fr, bool use_cluster) {
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
                            bt_stride, cu_q, seq_lens, decode_index, counters, nh, nkv, log2ps, num_pages, scale_log2,
                            window, chunk, nsplits, fr);
  } else {
    auto k = attn_decode_stream_kernel<HD, false>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    rc = osb_launch(k, grid, dim3(NT), smem, stream, out, part_o, part_ml, q, q_row_stride, kc, vc, bt, bt_stride, cu_q,
                    seq_lens, decode_index, counters, nh, nkv, log2ps, num_pages, scale_log2, window, chunk, nsplits, fr);
  }
  return rc ? rc : osb_last_error();
}
}  // namespace

#ifdef OSB_ATTN_TIMELINE
OSB_API int osb_attn_stream_timeline(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_stream_timeline, sizeof(long long) * (size_t)n);
}
#endif

// The decode part of osb_paged_attn_bf16 (same arguments, same meaning; requests bringing more than one
// token are skipped) for head sizes 64 and 128 and page sizes that are powers of two; anything else is refused
// with OSB_ERR_UNSUPPORTED. chunk is a multiple of 64; with nsplits > 1 and no cluster, part_o / part_ml /
// counters as for osb_paged_attn_bf16 (the splits table of the merging CTA needs rows * nsplits <= 8 * 16 * (hd + 8) / 2).
OSB_API int osb_attn_decode_stream(void* out, const void* q, int q_row_stride, const void* k_cache, const void* v_cache,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* seq_lens,
                                   const int* decode_index, int S, int nh, int nkv, int hd, int page_size, int num_pages,
                                   float scale, int window, float* part_o, float* part_ml, int* counters, int chunk,
                                   int nsplits, const float* rope_cos, const float* rope_sin, const int* rope_slot_map,
                                   int rope_rot, int use_cluster, cudaStream_t stream) {
  if (S <= 0) return OSB_OK;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0) return OSB_ERR_UNSUPPORTED;
  if (page_size < 1 || (page_size & (page_size - 1))) return OSB_ERR_UNSUPPORTED;
  if ((q_row_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return OSB_ERR_UNSUPPORTED;
  if (chunk <= 0 || chunk % 64 != 0 || nsplits <= 0 || nsplits > 128) return OSB_ERR_BAD_SHAPE;
  if (use_cluster && (nsplits < 2 || nsplits > 8)) use_cluster = 0;
  if (nsplits > 1 && !use_cluster && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return OSB_ERR_BAD_SHAPE;
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
                      block_table, bt_stride, cu_q, seq_lens, decode_index, counters, S, nh, nkv, log2ps, num_pages,
                      scale_log2, window, chunk, nsplits, stream, fr, use_cluster != 0);
  return launch<128>((bf16*)out, part_o, part_ml, (const bf16*)q, q_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
                     block_table, bt_stride, cu_q, seq_lens, decode_index, counters, S, nh, nkv, log2ps, num_pages,
                     scale_log2, window, chunk, nsplits, stream, fr, use_cluster != 0);
}
