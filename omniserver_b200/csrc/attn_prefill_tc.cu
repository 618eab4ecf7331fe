// Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores.
//
// A unit of work is 128 query rows of one (request, query head). Keys and values stream through shared
// memory in tiles of 128 keys, fetched page by page with TMA (128-byte swizzle) straight from the
// cache pages. S = Q K^T and O += P V are tcgen05.mma instructions, each kind issued by one thread of a
// warp of its own; two S buffers, two P buffers and O live in tensor memory. A softmax thread (one per query
// row) reads a row of S with tcgen05.ld into registers (the S buffer is free again at once, so Q K^T runs two
// tiles ahead), keeps the running sum in fp32 and writes P as bf16 into a P buffer (two values per 32-bit
// column), from where the second MMA takes it as its A operand: P never touches shared memory. O is rescaled
// in tensor memory only when a row's maximum has grown by more than 2^8 since the offset in use
// was set (the offset stays consistent, so the result is exact up to rounding).
// The softmax of one 128 x 128 tile is a chain of about 1,700 cycles in one thread per row (128 exponentials on
// the special-function unit, 8 cycles per warp instruction, and the arithmetic around them), longer than the
// tile's two products. So two groups of four softmax warps take the key tiles in turn: a row's exponent offset
// passes from one group's thread to the other's through shared memory as soon as the tile's maximum is known
// (the short, serial part), and the exponentials of tile t+1 run beside those of tile t, two warps per
// scheduler. Each group keeps its own running sum, brought to the common offset at the end. The output leaves
// through shared memory so that rows are written in whole lines.
// The grid is one CTA per SM at most; a CTA works through several items (the longest first, see item_index)
// without setting up again: barriers, tensor memory and the K/V pipeline run on across items.
// Roles: warp 0 TMA producer of keys, warp 2 of values, warp 1 issues Q K^T, warp 3 loads Q and issues P V
// (these four give registers to the others), warps 4-7 and 8-11 the two softmax groups. All mbarrier waits are
// bounded; on a time-out the CTA records a code in *err, waits for its copies in flight, frees its tensor
// memory and returns.
//
// Semantics as attn_generic.cu / attn_mma.cu (omniserve/model/qwen2_llm.py:96-112,
// omniserve/cache/kv_prealloc.py:138-142): scale on the scores, query at absolute position p sees keys
// max(0, p-window+1)..p of its own request, query head h reads kv head h / (nh/nkv).
#include "tc_utils.cuh"

namespace {
using namespace tc;

constexpr int BLOCK_M = 128, TILE_N = 128;
constexpr int NUM_THREADS = 384;
constexpr int SOFTMAX_REGS = 216, OTHER_REGS = 64;   // 256 x 216 + 128 x 64 registers of the 64 K
constexpr int STAGES = 3;  // K tiles, V tiles and S buffers in flight: tile t uses number t % STAGES of each
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows of 128 bytes
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

// One unit of work: 128 query rows of one (request, query head).
struct Item {
  int h, kvh, q0, m0, rows_here, kv_len, p_first, p_last, lo_last, tile_begin, n_tiles;
  const int* bt;
};

// Items are numbered so that those with the most keys (the last rows of the longest portions) come first. A CTA
// takes item blockIdx.x, then, while there are more items than CTAs, goes back and forth over the rest
// (item 2G-1-x, 2G+x, ...), so that the CTA with the longest first item gets the shortest second one.
__device__ __forceinline__ int item_index(int pass) {
  const int G = (int)gridDim.x, x = (int)blockIdx.x;
  return pass * G + ((pass & 1) ? G - 1 - x : x);
}

// `units` (or null): the (request, 128-row tile) pairs that have work, those with the most keys first; item idx is then
// head idx % nh of unit idx / nh. Without it every (tile, request, head) of the batch is an item and most may be empty.
__device__ __forceinline__ bool item_of(int idx, Item& it, const int* __restrict__ block_table, int bt_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ seq_lens, int nh, int nkv,
                                        int window, int skip_single, int m_tiles, int per_tile,
                                        const int2* __restrict__ units) {
  int m_tile, s;
  if (units != nullptr) {
    const int u = idx / nh;
    it.h = idx - u * nh;
    const int2 un = units[u];
    s = un.x;
    m_tile = un.y;
  } else {
    m_tile = m_tiles - 1 - idx / per_tile;
    const int hs = idx % per_tile;
    s = hs / nh;
    it.h = hs - s * nh;
  }
  it.q0 = cu_q[s];
  const int q_len = cu_q[s + 1] - it.q0;
  it.m0 = m_tile * BLOCK_M;
  if (q_len <= 0 || (skip_single && q_len == 1) || it.m0 >= q_len) return false;
  it.kvh = it.h / (nh / nkv);
  it.kv_len = seq_lens[s];
  it.rows_here = min(BLOCK_M, q_len - it.m0);
  it.p_first = it.kv_len - q_len + it.m0;
  it.p_last = it.p_first + it.rows_here - 1;
  const int lo = (window > 0 && it.p_first - window + 1 > 0) ? it.p_first - window + 1 : 0;
  it.lo_last = (window > 0 && it.p_last - window + 1 > 0) ? it.p_last - window + 1 : 0;
  it.tile_begin = lo / TILE_N;
  it.n_tiles = it.p_last / TILE_N - it.tile_begin + 1;
  it.bt = block_table + (size_t)s * bt_stride;
  return true;
}

// Barrier of the eight softmax warps that also tells every one of them whether any saw `v`.
__device__ __forceinline__ bool softmax_bar_or(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 2, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)v)
      : "memory");
  return r != 0;
}

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens, int nh, int nkv, int log2ps,
    float scale_log2, int window, int skip_single, int m_tiles, int n_items, const int2* __restrict__ units,
    int* __restrict__ err) {
  constexpr int NA = HD / 64;                 // 64-element atoms along the head dimension
  constexpr int Q_BYTES = NA * ATOM_BYTES;    // [atom][128 rows][128 B]
  constexpr int KV_BYTES = NA * ATOM_BYTES;   // one K or V tile: [atom][128 keys][128 B]
  constexpr uint32_t TMEM_COLS = 512;
  // two S buffers of 128 columns (fp32), two P buffers of 64 columns (two bf16 per column), then O
  constexpr uint32_t S_COL0 = 0, P_COL0 = 2 * TILE_N, O_COL = 3 * TILE_N;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = base;
  unsigned char* k_smem = q_smem + Q_BYTES;                  // STAGES tiles
  unsigned char* v_smem = k_smem + STAGES * KV_BYTES;     // STAGES tiles
  // The tiles a CTA works through are counted across its items: tile u uses K/V stage u % STAGES and S/P buffer u % 2.
  // k_free / s_full: Q K^T of a tile complete (the K tile may be overwritten / S may be read);
  // s_free: the softmax warps hold the tile's S in registers (the S buffer may be overwritten);
  // p_full: P of a tile is in tensor memory; v_free / p_free: P V of a tile complete (the V tile / the P buffer
  // may be overwritten, O may be read); epi_done: an item's output has left tensor and shared memory (the next
  // item's Q may be loaded; its first P V, which overwrites O, follows from that)
  __shared__ uint64_t q_full, epi_done, k_full[STAGES], v_full[STAGES], k_free[STAGES], v_free[STAGES];
  __shared__ uint64_t s_full[2], s_free[2], p_full[2], p_free[2];
  // max_done[u % 2]: the rows' exponent offsets after tile u are in row_offset (the group of tile u + 1 may go on)
  __shared__ uint64_t max_done[2];
  __shared__ float row_offset[BLOCK_M];   // per query row: the exponent offset in use (log2 units), -inf before the first key
  __shared__ float row_sum[2][BLOCK_M];   // per group and row: its sum of P at the final offset
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_tile = n_items / m_tiles;
  const int ps = 1 << log2ps;
  const int box_rows = ps < TILE_N ? ps : TILE_N;  // keys per TMA box: a page, or a tile's worth of a larger page
  const int n_boxes = TILE_N / box_rows;

  if (lane == 0 && warp < 3) prefetch_tensormap(warp == 0 ? &map_k : warp == 1 ? &map_q : &map_v);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&epi_done, 8);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_free[i], 1);
      mbar_init(&v_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&p_free[i], 1);
    }
    mbar_init(&max_done[0], BLOCK_M);
    mbar_init(&max_done[1], BLOCK_M);
    mbar_init_fence();
  }
  if (threadIdx.x < BLOCK_M) row_offset[threadIdx.x] = -INFINITY;
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  // until here nothing was read that the kernel before this one in the stream may still be writing (q, the pages)
  pdl_wait();
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* vabort = &abort_flag;
  Item it;
  auto next_item = [&](int& pass) -> bool {   // the same sequence of items in every warp
    for (;;) {
      const int idx = item_index(pass++);
      if (idx >= n_items) return false;
      if (item_of(idx, it, block_table, bt_stride, cu_q, seq_lens, nh, nkv, window, skip_single, m_tiles, per_tile, units))
        return true;
    }
  };

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(OTHER_REGS));
  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------------ TMA producers: warp 0 keys, warp 2 values
    const int which = warp == 0 ? 0 : 1;
    unsigned char* tiles = which ? v_smem : k_smem;
    const CUtensorMap* map = which ? &map_v : &map_k;
    // lane = (box b, atom a) of a tile: boxes * NA <= 32, a box being at least 8 keys
    const int b = lane / NA, a = lane - b * NA;
    int u0 = 0;   // tiles of the items before this one
    int issued = 0;
    for (int pass = 0; next_item(pass) && !*vabort; u0 += it.n_tiles) {
      auto page_of = [&](int t) -> int {
        const int key = (it.tile_begin + t) * TILE_N + b * box_rows;
        return (t < it.n_tiles && b < n_boxes && key <= it.p_last) ? it.bt[key >> log2ps] : -1;
      };
      int page = page_of(0);
      for (int t = 0; t < it.n_tiles; ++t) {
        const int u = u0 + t, st = u % STAGES;
        const uint32_t ph = (uint32_t)(u / STAGES) & 1u;
        const int key0 = (it.tile_begin + t) * TILE_N;
        const int next_page = page_of(t + 1);  // in flight while this tile's copies are issued
        // whole boxes (pages) up to the last key this item may look at; a box that starts beyond it is skipped
        const int boxes = min(n_boxes, (it.p_last - key0) / box_rows + 1);
        uint64_t* empty = which ? &v_free[st] : &k_free[st];
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
                      (key0 + b * box_rows) & (ps - 1), it.kvh, page);
        page = next_page;
        issued = u + 1;
      }
    }
    // after a failure: every copy that was issued lands before the CTA goes (a tile's barrier completes with it)
    if (*vabort && lane == 0) {
      for (int u = max(0, issued - STAGES); u < issued; ++u) {
        uint64_t* full = which ? &v_full[u % STAGES] : &k_full[u % STAGES];
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(full, (uint32_t)(u / STAGES) & 1u); ++w) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer of S = Q K^T, up to two tiles ahead
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BLOCK_M, TILE_N, 0, 0);
      bool ok = true;
      int u0 = 0, n_done = 0;
      for (int pass = 0; ok && next_item(pass); u0 += it.n_tiles, ++n_done) {
        ok = mbar_wait(&q_full, (uint32_t)n_done & 1u, vabort);
        for (int t = 0; t < it.n_tiles && ok; ++t) {
          const int u = u0 + t, st = u % STAGES;
          // the keys have landed, and the softmax warps have taken tile u - 2 out of this S buffer
          if (!mbar_wait(&k_full[st], (uint32_t)(u / STAGES) & 1u, vabort) ||
              !mbar_wait(&s_free[u & 1], ((uint32_t)(u >> 1) & 1u) ^ 1u, vabort)) {
            ok = false;
            break;
          }
          fence_after();
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t ad = desc_kmajor(q_smem + (ks >> 2) * ATOM_BYTES) + (uint64_t)((ks & 3) * 2);
            const uint64_t bd = desc_kmajor(k_smem + st * KV_BYTES + (ks >> 2) * ATOM_BYTES) + (uint64_t)((ks & 3) * 2);
            umma_bf16(tmem + S_COL0 + (uint32_t)((u & 1) * TILE_N), ad, bd, idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[u & 1]);
          umma_commit(&k_free[st]);
        }
      }
      if (!ok) {
        if (!*vabort) atomicExch(err, 112);
        *vabort = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ warp 3: loads Q, issues O += P V
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(BLOCK_M, HD, 0, 1);  // B = V: N (head dim) contiguous
      bool ok = true;
      int u0 = 0, n_done = 0, q_issued = 0;
      for (int pass = 0; ok && next_item(pass); u0 += it.n_tiles, ++n_done) {
        // Q goes where the item before staged its output: wait until that has left
        if (n_done > 0 && !mbar_wait(&epi_done, (uint32_t)(n_done - 1) & 1u, vabort)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&q_full, Q_BYTES);
        for (int a = 0; a < NA; ++a)
          tma_load_2d(q_smem + a * ATOM_BYTES, &map_q, &q_full, it.h * HD + a * 64, it.q0 + it.m0);
        q_issued = n_done + 1;
        for (int t = 0; t < it.n_tiles && ok; ++t) {
          const int u = u0 + t, st = u % STAGES;
          if (!mbar_wait(&p_full[u & 1], (uint32_t)(u >> 1) & 1u, vabort) ||
              !mbar_wait(&v_full[st], (uint32_t)(u / STAGES) & 1u, vabort)) {
            ok = false;
            break;
          }
          fence_after();
          const uint32_t p_tmem = tmem + P_COL0 + (uint32_t)((u & 1) * (TILE_N / 2));
#pragma unroll
          for (int ks = 0; ks < TILE_N / 16; ++ks) {
            const uint64_t bd = desc_mnmajor(v_smem + st * KV_BYTES, ATOM_BYTES) + (uint64_t)(ks * (16 * 128 / 16));
            umma_bf16_ts(tmem + O_COL, p_tmem + (uint32_t)(ks * 8), bd, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(&p_free[u & 1]);
          umma_commit(&v_free[st]);
        }
      }
      if (!ok) {
        if (!*vabort) atomicExch(err, 112);
        *vabort = 1;
        for (uint32_t w = 0; q_issued > 0 && w < WAIT_LIMIT && !mbar_try_wait(&q_full, (uint32_t)(q_issued - 1) & 1u); ++w) {
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
    // ------------------------------------------------------------------ softmax and epilogue: two groups of four warps
    const int grp = (warp - 4) >> 2;     // group 0 takes the even tiles of the CTA's count, group 1 the odd ones
    const int qd = warp & 3;             // TMEM lane quarter of this warp
    const int r = qd * 32 + lane;        // query row of this thread
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + S_COL0 + (uint32_t)(grp * TILE_N);
    const uint32_t p_addr = tmem + lane_addr + P_COL0 + (uint32_t)(grp * (TILE_N / 2));
    int u0 = 0;
    bool stop = false;
    for (int pass = 0; !stop && next_item(pass); u0 += it.n_tiles) {
      const int p_row = r < it.rows_here ? it.p_first + r : -1;
      const int lo_row = (window > 0 && p_row - window + 1 > 0) ? p_row - window + 1 : 0;
      const int u_last = u0 + it.n_tiles - 1;
      // my_off: the offset this thread's sum l_run is expressed at (what it last saw or set)
      float my_off = -INFINITY, l_run = 0.0f;
      bool ok = true;
      for (int t = (u0 & 1) == grp ? 0 : 1; t < it.n_tiles; t += 2) {
        const int u = u0 + t;                             // u % 2 == grp
        const uint32_t ph2 = (uint32_t)(u >> 1) & 1u;     // phase of this group's S/P barriers
        if (!mbar_wait(&s_full[grp], ph2, vabort)) ok = false;
        if (!__all_sync(0xffffffffu, ok)) {
          ok = false;
          break;
        }
        fence_after();
        const int key0 = (it.tile_begin + t) * TILE_N;
        uint32_t v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + (uint32_t)(c * 32), v[c]);
        tmem_ld_wait();
        // the row is in registers: the S buffer is free for the tile after the next
        fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[grp]);
        // a tile wholly below the diagonal and inside every row's window needs no mask
        const bool unmasked = key0 + TILE_N - 1 <= it.p_first && key0 >= it.lo_last;
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
        // the row's offset after the tile before, which the other group's thread of this row has set
        if (t > 0) {
          if (!mbar_wait(&max_done[(u - 1) & 1], (uint32_t)((u - 1) >> 1) & 1u, vabort)) ok = false;
          if (!__all_sync(0xffffffffu, ok)) {
            ok = false;
            break;
          }
        }
        const float m_used = row_offset[r];   // -inf at an item's first tile
        // the exponent offset in use moves only when the maximum has grown enough (or at the first keys)
        const bool grow = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx > -INFINITY);
        const float m_new = grow ? mx : m_used;
        row_offset[r] = m_new;
        mbar_arrive(&max_done[grp]);    // releases the write above to the thread that waits for this tile's offsets
        // this thread's sum at the new offset: first to what the other group left, then to what this tile sets
        if (my_off != m_new) l_run = my_off == -INFINITY ? 0.0f : l_run * ex2_approx(my_off - m_new);
        my_off = m_new;
        const float alpha = (grow && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
        if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
          // O belongs to the tensor cores until the product of the tile before has completed; the product of this
          // tile waits for this thread's P, the products after it for this one: nothing else touches O meanwhile
          if (!mbar_wait(&p_free[(u - 1) & 1], (uint32_t)((u - 1) >> 1) & 1u, vabort)) ok = false;
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
        // the product that read this P buffer last (tile u - 2) has completed
        if (u >= 2) {
          if (!mbar_wait(&p_free[grp], ph2 ^ 1u, vabort)) ok = false;
          if (!__all_sync(0xffffffffu, ok)) {
            ok = false;
            break;
          }
          fence_after();
        }
        // P = exp2(S * scale - offset), two bf16 per column of this group's P buffer;
        // rows that have seen no key yet (offset -inf) are all masked here: exp2(-inf) = 0 with any finite offset
        const float offset = m_new == -INFINITY ? 0.0f : m_new;
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
          if (c == 1) tmem_st32(p_addr, v[0]);
        }
        tmem_st32(p_addr + 32u, v[1]);
        l_run += sum0 + sum1;
        // The last tile may end before its 128 keys do: rows of the V tile from the first key that was
        // not loaded (shared memory never written, or an older tile) or that lies at or beyond the request's
        // length (whatever the page held before) have P = 0, and 0 x (Inf or NaN) must not reach O: clear them.
        if (t == it.n_tiles - 1) {
          const int loaded = min(n_boxes, (it.p_last - key0) / box_rows + 1) * box_rows;
          const int first_bad = min(it.kv_len - key0, loaded);
          if (first_bad < TILE_N) {
            const int st = u % STAGES;
            if (!mbar_wait(&v_full[st], (uint32_t)(u / STAGES) & 1u, vabort)) ok = false;
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
        if (lane == 0) mbar_arrive(&p_full[grp]);
      }
      // both groups bring their sums to the offset after the last tile and exchange them
      if (ok && (u_last & 1) != grp) {   // the other group had the last tile
        if (!mbar_wait(&max_done[u_last & 1], (uint32_t)(u_last >> 1) & 1u, vabort)) ok = false;
      }
      {
        const float m_fin = row_offset[r];
        if (my_off != m_fin) l_run = my_off == -INFINITY ? 0.0f : l_run * ex2_approx(my_off - m_fin);
        row_sum[grp][r] = l_run;
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");   // the eight softmax warps
      if (grp == 0) row_offset[r] = -INFINITY;          // for the next item; its first tile is read after the barrier below
      if (item_index(pass) >= n_items) pdl_trigger();   // the last item of this CTA (or only empty ones follow)
      // epilogue: O / l as bf16 through the shared memory that held Q (every product that read it has completed),
      // each group half of the head's columns, so that the rows go out in whole 16-byte pieces side by side:
      // written straight from the tensor-memory layout (one row per lane) every store instruction would touch 32 rows
      constexpr int CPR = HD / 8;          // 16-byte pieces per row; piece c of row r lies at slot c ^ (r % CPR)
      ok = __all_sync(0xffffffffu, ok);
      if (ok && !mbar_wait(&p_free[u_last & 1], (uint32_t)(u_last >> 1) & 1u, vabort)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        fence_after();
        const float l = row_sum[0][r] + row_sum[1][r];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
        for (int c0 = grp * (HD / 2); c0 < (grp + 1) * (HD / 2); c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_addr + O_COL + (uint32_t)c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              hh[e] = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * e]) * inv, __uint_as_float(o[j + 2 * e + 1]) * inv);
            const int c = (c0 + j) >> 3;
            *reinterpret_cast<uint4*>(q_smem + r * (HD * 2) + ((c ^ (r & (CPR - 1))) << 4)) = w;
          }
        }
        fence_before();
      } else if (lane == 0) {
        if (!*vabort) atomicExch(err, 113);
        *vabort = 1;
      }
      stop = softmax_bar_or(!ok || *vabort != 0);
      if (!stop) {
        const int ts = (int)threadIdx.x - 128;
        const int c = ts % CPR;
#pragma unroll
        for (int row = ts / CPR; row < BLOCK_M; row += 256 / CPR)
          if (row < it.rows_here)
            *reinterpret_cast<uint4*>(out + ((size_t)(it.q0 + it.m0 + row) * nh + it.h) * HD + c * 8) =
                *reinterpret_cast<const uint4*>(q_smem + row * (HD * 2) + ((c ^ (row & (CPR - 1))) << 4));
        // what this warp read of O (tensor memory) and of the staged rows is in its registers or on its way out
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_done);
      }
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
           int max_q_len, int skip_single, const int2* units, int n_units, int* err, cudaStream_t stream) {
  // at least 120 KB so that one CTA is resident per SM: each takes all 512 tensor-memory columns
  constexpr size_t need = (size_t)(HD / 64) * ATOM_BYTES * (1 + 2 * STAGES) + 1024;
  constexpr size_t smem = need > 120 * 1024 ? need : 120 * 1024;
  auto k = attn_prefill_tc_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int m_tiles = (max_q_len + BLOCK_M - 1) / BLOCK_M;
  const int n_items = units != nullptr ? n_units * nh : m_tiles * nh * S;
  if (n_items <= 0) return OSB_OK;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 1;
  }
  // one CTA per SM at most (each takes all tensor memory and most of the shared memory), several items each if need be
  const dim3 grid((unsigned)(n_items < num_sms ? n_items : num_sms));
  return osb_launch(k, grid, dim3(NUM_THREADS), smem, stream, mq, mk, mv, out, bt, bt_stride, cu_q, seq_lens, nh, nkv,
                    log2ps, scale_log2, window, skip_single, m_tiles, n_items, units, err);
}
}  // namespace


// out [T, nh*hd] bf16; q = the first nh*hd columns of rows of q_row_stride elements; caches
// [pages, nkv, page_size, hd] bf16. Head sizes 64 and 128, page sizes that are powers of two from 8
// up; anything else is refused with OSB_ERR_UNSUPPORTED (the caller then uses the mma.sync kernel).
// Requests bringing one token are skipped when skip_single is set. units (or null) [n_units][2] int32: the (request,
// 128-row tile of its portion) pairs to compute, in the order in which they are to start; the caller lists every pair
// that has rows (a pair that has none is skipped).
OSB_API int osb_attn_prefill_tc(void* out, const void* q, int q_row_stride, int T, const void* k_cache,
                                const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                                const int* seq_lens, int S, int nh, int nkv, int hd, int page_size, int num_pages,
                                float scale, int window, int max_q_len, int skip_single, const int* units, int n_units,
                                int* err, cudaStream_t stream) {
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
                      window, max_q_len, skip_single, reinterpret_cast<const int2*>(units), n_units, err, stream);
  return launch<128>(mq, mk, mv, (bf16*)out, block_table, bt_stride, cu_q, seq_lens, S, nh, nkv, log2ps, scale_log2,
                     window, max_q_len, skip_single, reinterpret_cast<const int2*>(units), n_units, err, stream);
}
