// Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores.
//
// One CTA = 128 query rows of one (request, query head). Keys and values stream through shared
// memory in tiles of 128 keys, fetched page by page with TMA (128-byte swizzle) straight from the
// cache pages. S = Q K^T and O += P V are tcgen05.mma instructions, each kind issued by one thread of a
// warp of its own; S (three buffers) and O live in tensor memory. Four softmax warps (one thread per query row) read a row
// of S with tcgen05.ld into registers, keep the running maximum and sum in fp32 and write P as
// bf16 back into tensor memory over the S it came from (two values per 32-bit column), from where
// the second MMA takes it as its A operand: P never touches shared memory, and the softmax of
// tile t+1 runs while the tensor cores work on P V of tile t and Q K^T of the tiles after. O is rescaled
// in tensor memory only when a row's maximum has grown by more than 2^8 since the offset in use
// was set (the offset stays consistent, so the result is exact up to rounding).
// Roles: warp 0 TMA producer of Q and keys, warp 6 of values, warp 1 issues Q K^T (up to three tiles ahead),
// warp 7 issues P V, warps 2-5 softmax and epilogue. All mbarrier
// waits are bounded; on a time-out the CTA records a code in *err, waits for its copies in flight,
// frees its tensor memory and returns.
//
// Semantics as attn_generic.cu / attn_mma.cu (omniserve/model/qwen2_llm.py:96-112,
// omniserve/cache/kv_prealloc.py:138-142): scale on the scores, query at absolute position p sees keys
// max(0, p-window+1)..p of its own request, query head h reads kv head h / (nh/nkv).
#include "tc_utils.cuh"

namespace {
using namespace tc;

constexpr int BLOCK_M = 128, TILE_N = 128;
constexpr int NUM_THREADS = 256;
constexpr int STAGES = 3;  // K tiles, V tiles and S buffers in flight: tile t uses number t % STAGES of each
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows of 128 bytes
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens, int nh, int nkv, int log2ps,
    float scale_log2, int window, int skip_single, int m_tiles, int* __restrict__ err) {
  constexpr int NA = HD / 64;                 // 64-element atoms along the head dimension
  constexpr int Q_BYTES = NA * ATOM_BYTES;    // [atom][128 rows][128 B]
  constexpr int KV_BYTES = NA * ATOM_BYTES;   // one K or V tile: [atom][128 keys][128 B]
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, O_COL = STAGES * TILE_N;  // S buffers of 128 columns, P over the first 64 of its S; then O
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = base;
  unsigned char* k_smem = q_smem + Q_BYTES;                  // STAGES tiles
  unsigned char* v_smem = k_smem + STAGES * KV_BYTES;     // STAGES tiles
  // s_full[i]: Q K^T of a tile complete (S may be read, the K tile may be overwritten);
  // pv_done[i]: P V of a tile complete (the V tile and the S buffer that held P may be overwritten, O may be read)
  __shared__ uint64_t q_full, k_full[STAGES], v_full[STAGES], s_full[STAGES], p_full[STAGES], pv_done[STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blocks are numbered so that the tiles with the most keys (the last rows of the longest portions) start first
  const int per_tile = gridDim.x / m_tiles;
  const int m_tile = m_tiles - 1 - (int)blockIdx.x / per_tile;
  const int hs = (int)blockIdx.x % per_tile;
  const int h = hs % nh, s = hs / nh;
  const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
  if (q_len <= 0 || (skip_single && q_len == 1)) return;
  const int m0 = m_tile * BLOCK_M;
  if (m0 >= q_len) return;
  const int g = nh / nkv, kvh = h / g;
  const int kv_len = seq_lens[s];
  const int rows_here = min(BLOCK_M, q_len - m0);
  const int p_first = kv_len - q_len + m0;
  const int p_last = p_first + rows_here - 1;
  const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int lo_last = (window > 0 && p_last - window + 1 > 0) ? p_last - window + 1 : 0;
  const int tile_begin = lo / TILE_N, n_tiles = p_last / TILE_N - tile_begin + 1;
  const int* bt = block_table + (size_t)s * bt_stride;
  const int ps = 1 << log2ps;
  const int box_rows = ps < TILE_N ? ps : TILE_N;  // keys per TMA box: a page, or a tile's worth of a larger page
  const int n_boxes = TILE_N / box_rows;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* vabort = &abort_flag;

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers: warp 0 keys (and Q), warp 6 values
    const int which = warp == 0 ? 0 : 1;
    if (which == 0 && lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
      for (int a = 0; a < NA; ++a) tma_load_2d(q_smem + a * ATOM_BYTES, &map_q, &q_full, h * HD + a * 64, q0 + m0);
    }
    unsigned char* tiles = which ? v_smem : k_smem;
    const CUtensorMap* map = which ? &map_v : &map_k;
    // lane = (box b, atom a) of a tile: boxes * NA <= 32, a box being at least 8 keys
    const int b = lane / NA, a = lane - b * NA;
    auto page_of = [&](int t) -> int {
      const int key = (tile_begin + t) * TILE_N + b * box_rows;
      return (t < n_tiles && b < n_boxes && key <= p_last) ? bt[key >> log2ps] : -1;
    };
    int issued = 0;
    int page = page_of(0);
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t % STAGES;
      const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
      const int key0 = (tile_begin + t) * TILE_N;
      const int next_page = page_of(t + 1);  // in flight while this tile's copies are issued
      // whole boxes (pages) up to the last key this CTA may look at; a box that starts beyond it is skipped
      const int boxes = min(n_boxes, (p_last - key0) / box_rows + 1);
      uint64_t* empty = which ? &pv_done[st] : &s_full[st];
      uint64_t* full = which ? &v_full[st] : &k_full[st];
      if (lane == 0) {
        if (!mbar_wait(empty, ph ^ 1u, vabort)) {
          if (!*vabort) atomicExch(err, 111);
          *vabort = 1;
        } else {
          mbar_expect_tx(full, (uint32_t)(boxes * NA * box_rows * 128));
        }
      }
      __syncwarp();
      if (*vabort) break;
      if (lane < boxes * NA)
        tma_load_4d(tiles + st * KV_BYTES + a * ATOM_BYTES + b * box_rows * 128, map, full, a * 64,
                    (key0 + b * box_rows) & (ps - 1), kvh, page);
      page = next_page;
      issued = t + 1;
    }
    if (*vabort && lane == 0) {
      for (int t = max(0, issued - STAGES); t < issued; ++t) {
        const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
        uint64_t* full = which ? &v_full[t % STAGES] : &k_full[t % STAGES];
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(full, ph); ++w) {
        }
      }
      if (which == 0)
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(&q_full, 0); ++w) {
        }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer of S = Q K^T, up to STAGES tiles ahead
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BLOCK_M, TILE_N, 0, 0);
      bool ok = mbar_wait(&q_full, 0, vabort);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int st = t % STAGES;
        const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
        // the keys have landed, and the product that read P out of this S buffer (tile t - STAGES) has completed
        if (!mbar_wait(&k_full[st], ph, vabort) || !mbar_wait(&pv_done[st], ph ^ 1u, vabort)) {
          ok = false;
          break;
        }
        fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t ad = desc_kmajor(q_smem + (ks >> 2) * ATOM_BYTES) + (uint64_t)((ks & 3) * 2);
          const uint64_t bd = desc_kmajor(k_smem + st * KV_BYTES + (ks >> 2) * ATOM_BYTES) + (uint64_t)((ks & 3) * 2);
          umma_bf16(tmem + S_COL0 + (uint32_t)(st * TILE_N), ad, bd, idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
      }
      if (!ok) {
        if (!*vabort) atomicExch(err, 112);
        *vabort = 1;
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ issuer of O += P V
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(BLOCK_M, HD, 0, 1);  // B = V: N (head dim) contiguous
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int st = t % STAGES;
        const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
        if (!mbar_wait(&p_full[st], ph, vabort) || !mbar_wait(&v_full[st], ph, vabort)) {
          ok = false;
          break;
        }
        fence_after();
        const uint32_t p_tmem = tmem + S_COL0 + (uint32_t)(st * TILE_N);
#pragma unroll
        for (int ks = 0; ks < TILE_N / 16; ++ks) {
          const uint64_t bd = desc_mnmajor(v_smem + st * KV_BYTES, ATOM_BYTES) + (uint64_t)(ks * (16 * 128 / 16));
          umma_bf16_ts(tmem + O_COL, p_tmem + (uint32_t)(ks * 8), bd, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[st]);
      }
      if (!ok) {
        if (!*vabort) atomicExch(err, 112);
        *vabort = 1;
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------------ softmax and epilogue: warps 2..5
    const int qd = warp & 3;             // TMEM lane quarter of this warp
    const int r = qd * 32 + lane;        // query row of this thread
    const int p_row = r < rows_here ? p_first + r : -1;
    const int lo_row = (window > 0 && p_row - window + 1 > 0) ? p_row - window + 1 : 0;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    float m_used = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t % STAGES;
      if (!mbar_wait(&s_full[st], (uint32_t)(t / STAGES) & 1u, vabort)) ok = false;
      if (!__all_sync(0xffffffffu, ok)) {
        ok = false;
        break;
      }
      fence_after();
      const int key0 = (tile_begin + t) * TILE_N;
      const uint32_t s_addr = tmem + lane_addr + S_COL0 + (uint32_t)(st * TILE_N);
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + (uint32_t)(c * 32), v[c]);
      tmem_ld_wait();
      // a tile wholly below the diagonal and inside every row's window needs no mask
      const bool unmasked = key0 + TILE_N - 1 <= p_first && key0 >= lo_last;
      if (!unmasked) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c * 32 + j;
            if (key > p_row || key < lo_row) v[c][j] = 0xff800000u;  // -inf
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        mx0 = fmaxf(mx0, __uint_as_float(v[0][j]));
        mx1 = fmaxf(mx1, __uint_as_float(v[1][j]));
        mx2 = fmaxf(mx2, __uint_as_float(v[2][j]));
        mx3 = fmaxf(mx3, __uint_as_float(v[3][j]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;  // the scale is positive
      // the exponent offset in use moves only when the maximum has grown enough (or at the first keys)
      const bool grow = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx > -INFINITY);
      const float m_new = grow ? mx : m_used;
      const float alpha = (grow && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        // O belongs to the tensor cores until the product of the tile before has completed
        if (!mbar_wait(&pv_done[(t - 1) % STAGES], (uint32_t)((t - 1) / STAGES) & 1u, vabort)) ok = false;
        if (!__all_sync(0xffffffffu, ok)) {
          ok = false;
          break;
        }
        fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_addr + O_COL + (uint32_t)c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st32(tmem + lane_addr + O_COL + (uint32_t)c0, o);
        }
      }
      l_run *= alpha;
      m_used = m_new;
      // P = exp2(S * scale - offset), two bf16 per column, over the first half of this S buffer;
      // rows that have seen no key yet (offset -inf) are all masked here: exp2(-inf) = 0 with any finite offset
      const float offset = m_used == -INFINITY ? 0.0f : m_used;
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(v[c][j]), scale_log2, -offset));
          const float p1 = ex2_approx(fmaf(__uint_as_float(v[c][j + 1]), scale_log2, -offset));
          sum0 += p0;
          sum1 += p1;
          __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          v[c >> 1][(c & 1) * 16 + (j >> 1)] = *reinterpret_cast<uint32_t*>(&b);
        }
        if (c == 1) tmem_st32(s_addr, v[0]);
      }
      tmem_st32(s_addr + 32u, v[1]);
      l_run += sum0 + sum1;
      // The last tile may end before its 128 keys do: rows of the V tile from the first key that was
      // not loaded (shared memory never written, or an older tile) or that lies at or beyond the request's
      // length (whatever the page held before) have P = 0, and 0 x (Inf or NaN) must not reach O: clear them.
      if (t == n_tiles - 1) {
        const int loaded = min(n_boxes, (p_last - key0) / box_rows + 1) * box_rows;
        const int first_bad = min(kv_len - key0, loaded);
        if (first_bad < TILE_N) {
          if (!mbar_wait(&v_full[st], (uint32_t)(t / STAGES) & 1u, vabort)) ok = false;
          if (!__all_sync(0xffffffffu, ok)) {
            ok = false;
            break;
          }
          if (r >= first_bad)
            for (int a = 0; a < NA; ++a)
#pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(v_smem + st * KV_BYTES + a * ATOM_BYTES + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
          fence_async_smem();
        }
      }
      tmem_st_wait();
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    // epilogue: O / l
    if (ok) {
      if (!mbar_wait(&pv_done[(n_tiles - 1) % STAGES], (uint32_t)((n_tiles - 1) / STAGES) & 1u, vabort)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      fence_after();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_addr + O_COL + (uint32_t)c0, o);
        tmem_ld_wait();
        if (r < rows_here) {
          bf16* op = out + ((size_t)(q0 + m0 + r) * nh + h) * HD + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 u;
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              hh[e] = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * e]) * inv, __uint_as_float(o[j + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(op + j) = u;
          }
        }
      }
    } else if (lane == 0) {
      if (!*vabort) atomicExch(err, 113);
      *vabort = 1;
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, bf16* out, const int* bt, int bt_stride,
           const int* cu_q, const int* seq_lens, int S, int nh, int nkv, int log2ps, float scale_log2, int window,
           int max_q_len, int skip_single, int* err, cudaStream_t stream) {
  // at least 120 KB so that one CTA is resident per SM: each takes all 512 tensor-memory columns
  constexpr size_t need = (size_t)(HD / 64) * ATOM_BYTES * (1 + 2 * STAGES) + 1024;
  constexpr size_t smem = need > 120 * 1024 ? need : 120 * 1024;
  auto k = attn_prefill_tc_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int m_tiles = (max_q_len + BLOCK_M - 1) / BLOCK_M;
  const dim3 grid((unsigned)m_tiles * (unsigned)nh * (unsigned)S);
  k<<<grid, NUM_THREADS, smem, stream>>>(mq, mk, mv, out, bt, bt_stride, cu_q, seq_lens, nh, nkv, log2ps, scale_log2,
                                         window, skip_single, m_tiles, err);
  return osb_last_error();
}
}  // namespace


// out [T, nh*hd] bf16; q = the first nh*hd columns of rows of q_row_stride elements; caches
// [pages, nkv, page_size, hd] bf16. Head sizes 64 and 128, page sizes that are powers of two from 8
// up; anything else is refused with OSB_ERR_UNSUPPORTED (the caller then uses the mma.sync kernel).
// Requests bringing one token are skipped when skip_single is set.
OSB_API int osb_attn_prefill_tc(void* out, const void* q, int q_row_stride, int T, const void* k_cache,
                                const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                                const int* seq_lens, int S, int nh, int nkv, int hd, int page_size, int num_pages,
                                float scale, int window, int max_q_len, int skip_single, int* err,
                                cudaStream_t stream) {
  if (S <= 0 || T <= 0) return OSB_OK;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0 || !(scale > 0.0f)) return OSB_ERR_UNSUPPORTED;
  if (page_size < 8 || (page_size & (page_size - 1))) return OSB_ERR_UNSUPPORTED;
  if ((q_row_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return OSB_ERR_UNSUPPORTED;
  int log2ps = 0;
  while ((1 << log2ps) < page_size) ++log2ps;
  CUtensorMap mq, mk, mv;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)q_row_stride, (cuuint64_t)T};
    const cuuint64_t strides[1] = {(cuuint64_t)q_row_stride * 2};
    const cuuint32_t box[2] = {64, 128};
    int rc = tc::make_map_bf16(&mq, q, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)page_size, (cuuint64_t)nkv, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)page_size * hd * 2,
                                   (cuuint64_t)nkv * page_size * hd * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)(page_size < 128 ? page_size : 128), 1, 1};
    int rc = tc::make_map_bf16(&mk, k_cache, 4, dims, strides, box);
    if (rc) return rc;
    rc = tc::make_map_bf16(&mv, v_cache, 4, dims, strides, box);
    if (rc) return rc;
  }
  const float scale_log2 = scale * LOG2E;
  if (hd == 64)
    return launch<64>(mq, mk, mv, (bf16*)out, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, log2ps, scale_log2,
                      window, max_q_len, skip_single, err, stream);
  return launch<128>(mq, mk, mv, (bf16*)out, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, log2ps, scale_log2,
                     window, max_q_len, skip_single, err, stream);
}
