// Decode-step layers as persistent kernels: one CTA per SM, all resident at once (cooperative launch).
//
// A decode step of a few rows is bound by reading the weights once. Run as one kernel per projection, every
// kernel pays its start (launch, first loads in flight) and its tail again, and the memory pipe drains at each
// boundary. Here one warp per CTA streams the CTA's share of every weight matrix through a ring of
// shared-memory tiles with bulk asynchronous copies, stage after stage without a pause: the weights do not
// depend on the activations, so the stream runs ahead across the points where the CTAs have to wait for one
// another. A second warp streams activations that other CTAs wrote (the input of a projection that follows a
// grid barrier) through tiles of their own. Eight warps consume the tiles with m16n8k16 MMAs (weight rows on
// the M side, up to 8 batch rows on the N side, the K range of a tile split over the warps and summed in a
// fixed order through shared memory). An RMS norm in front of a projection is computed by every CTA itself.
// Between stages the CTAs meet at a barrier in global memory; every wait is bounded and reports through the
// error flag instead of hanging.
//
// Kernels:
//   norm_linear_decode_kernel   y = (rmsnorm(res + x) * w) W^T + b          (no CTA waits for another)
//   ffn_decode_fused_kernel     r = res + x;  h = rmsnorm(r) * w;  act = silu(h Wg^T) * (h Wu^T)
//                               -- grid barrier --  y = act Wd^T
//   attn_decode_fused_kernel    norm, qkv -- barrier -- rotary, cache write, attention over the cache (the
//                               device function of attn_decode_stream.cuh) -- barrier -- y = attn Wo^T
//   decode_layers_fused_kernel  the last two, layer after layer, as one launch
// Formulas: omniserve/kernels/fused_ops.py:21-29, 43-57 (add + norm), 111-119 (silu * up);
// omniserve/model/qwen2_llm.py:75-113 (attention), 116-134 (feed-forward), 137-157 (the residual stream).
#include <type_traits>

#include "attn_decode_stream.cuh"
#include "mma_utils.cuh"
#include "tc_utils.cuh"

namespace {

constexpr int NCW = 8;               // consumer warps
constexpr int NCT = NCW * 32;        // consumer threads
constexpr int W_WARP = NCW;          // the warp that streams the weights
constexpr int A_WARP = NCW + 1;      // the warp that streams activations other CTAs wrote (kernels that have such stages)
constexpr int NTHREADS = NCT + 32;
constexpr int NTHREADS_ACT = NCT + 64;
// With the attention inside, the consumer warps need more registers than an even share of the file gives
// nine warps (one scheduler would hold three of them): such a kernel is launched with twelve warps, the
// last four give registers back (three of them end at once) and the consumers take them.
constexpr int NTHREADS_WIDE = NCT + 128;
constexpr int CONSUMER_REGS = 224, PRODUCER_REGS = 56;   // 2 * 224 + 56 = 3 * 168 per scheduler
// How the shared memory is cut: weight tiles of RS rows by at most MAX_KTW * 128 elements along K, NST
// of them in flight; activation tiles of MAX_B rows by the same length, AST in flight.
// NT: MMA column tiles of 8 batch rows each (kernels for up to 8 * NT rows; the reduction buffers grow with it).
template <int RS_, int MAX_KTW_, int NST_, int AST_, int NT_ = 1>
struct Geometry {
  static constexpr int RS = RS_, PG = RS_ / 2, MAX_KTW = MAX_KTW_, NST = NST_, AST = AST_, NT = NT_;
  static constexpr int RED_FLOATS = 2 * NCW * 128 * NT;   // two buffers of every warp's accumulators
  static constexpr int MAX_KC = MAX_KTW * NCW * 16;
  // row stride in a tile; = 32 mod 128, so the 8-byte fragment loads of four rows fall on different banks
  static constexpr int SROW = MAX_KC * 2 + 32;
  static constexpr int SLOT = RS * SROW, ASLOT = 8 * NT * SROW;   // an activation tile holds all batch rows
  static constexpr int MAX_ST = 8;   // bound of NST and AST: the barrier arrays
  static_assert(NST <= MAX_ST && AST <= MAX_ST && (MAX_KC * 2) % 128 == 0, "");
};
constexpr int MAX_B = 8;             // batch rows: the N side of one MMA
constexpr uint32_t GRID_WAIT_LIMIT = 1u << 21;

enum : int { ERR_TILE_WAIT = 131, ERR_SLOT_WAIT = 132, ERR_GRID_WAIT = 133, ERR_DRAIN = 134 };

#ifdef OSB_FUSED_TIMELINE
__device__ long long g_fused_timeline[160 * 16];
__device__ __forceinline__ long long gtime() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FTL(i) do { if ((threadIdx.x & 31) == 0 && (threadIdx.x == 0 || threadIdx.x == NCT) && blockIdx.x < 160) \
    g_fused_timeline[blockIdx.x * 16 + (i)] = gtime(); } while (0)
#else
#define FTL(i) do { } while (0)
#endif

__host__ __device__ constexpr int largest_divisor_le(int n, int cap) {
  int best = 1;
  for (int d = 1; d <= cap; ++d)
    if (n % d == 0) best = d;
  return best;
}

struct FfnParams {
  const bf16* x;          // [B, H] branch output of the part before
  const float* res_in;    // [B, H] or null
  float* res_out;         // [B, H]
  const bf16* norm_w;     // [H]
  const bf16* w_gate_up;  // [2I, H], gate rows first
  const bf16* w_down;     // [H, I]
  bf16* act;              // [B, I] scratch
  bf16* y;                // [B, H]
  unsigned long long* bar;  // arrivals at all grid barriers so far: a multiple of the grid size between launches
  int* err;
  float eps;
  int B, H, I;
};

struct Shared {
  uint64_t full[8], empty[8];
  uint64_t afull[8], aempty[8];
  uint64_t act_ready;      // a phase per streamed activation: it is complete in global memory
  int s_last;              // attention: this CTA merges the splits of its (request, kv head)
  volatile int abort_flag;
};

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(tc::smem_addr(dst)), "l"(src), "r"(bytes), "r"(tc::smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(tc::smem_addr(dst)), "l"(src), "r"(bytes), "r"(tc::smem_addr(bar))
               : "memory");
}
template <uint32_t R> __device__ __forceinline__ void reg_take() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}
template <uint32_t R> __device__ __forceinline__ void reg_give() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}
// After generic-proxy stores to global memory that another CTA will read with bulk asynchronous copies (the
// async proxy), before the barrier that tells it so.
__device__ __forceinline__ void publish_for_bulk_copies() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }
__device__ __forceinline__ uint2 lds64(const uint8_t* p) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(tc::smem_addr(p)));
  return v;
}

// The rows [r0, r1) of `total` that CTA c of G owns: sizes differ by at most one.
__device__ __forceinline__ void cta_rows(int total, int c, int G, int& r0, int& r1) {
  r0 = (int)((long long)total * c / G);
  r1 = (int)((long long)total * (c + 1) / G);
}

// A bounded wait on one of the CTA's barriers; the first thread that runs out of patience makes every
// later wait of the CTA return at once. The control flow goes on unchanged (every bar.sync is still
// reached by all its threads), on data that is no longer meaningful, and the host sees the error flag.
__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, Shared* sh, int* err, int code) {
  if (!tc::mbar_wait(bar, parity, (volatile int*)&sh->abort_flag) && !sh->abort_flag) {
    sh->abort_flag = 1;
    atomicExch(err, code);
  }
}

// ------------------------------------------------------------------ a stream of tiles (one warp)
// Used twice: the weights (tiles of RS rows), and activations that other CTAs wrote (tiles of B rows).
template <int NST, int SLOT, int SROW, int RS, bool ONCE>   // ONCE: the bytes are read once per step (weights): first out of the L2
struct Streamer {
  Shared* sh;
  uint64_t *full, *empty;
  uint8_t* slots;
  uint32_t idx;
  uint64_t policy;
  int lane;
  int* err;

  // One tile: lane l < n copies `bytes` from src(l) to row l of the next slot.
  template <class Src>
  __device__ __forceinline__ void tile(int n, uint32_t bytes, Src src) {
    const uint32_t slot = idx % NST, round = idx / NST;
    wait_or_abort(&empty[slot], (round & 1u) ^ 1u, sh, err, ERR_SLOT_WAIT);
    if (lane == 0) tc::mbar_expect_tx(&full[slot], bytes * (uint32_t)n);
    __syncwarp();
    if (lane < n) {
      void* dst = slots + (size_t)slot * SLOT + (size_t)lane * SROW;
      if constexpr (ONCE) bulk_copy(dst, src(lane), bytes, &full[slot], policy);
      else bulk_copy(dst, src(lane), bytes, &full[slot]);
    }
    ++idx;
  }

  // rows [r0, r1) of W [*, K] in groups of RS rows, each group in `nch` pieces of `kc` elements along K
  __device__ void rows(const bf16* W, int K, int r0, int r1, int nch, int kc) {
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      for (int ch = 0; ch < nch; ++ch)
        tile(nr, (uint32_t)kc * 2u, [&](int l) { return W + (size_t)(rg + l) * K + (size_t)ch * kc; });
    }
  }
  // pairs [p0, p1): row p of W [2I, K] in tile rows 0 .. PG-1 beside row I + p in tile rows PG ..
  __device__ void pairs(const bf16* W, int K, int I, int p0, int p1, int nch, int kc) {
    constexpr int PG = RS / 2;
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      for (int ch = 0; ch < nch; ++ch)
        tile(RS, (uint32_t)kc * 2u, [&](int l) {
          // a short last tile repeats its last pair: the rows exist and are not used
          const int q = pg + min(l < PG ? l : l - PG, np - 1);
          return W + (size_t)((l < PG ? 0 : I) + q) * K + (size_t)ch * kc;
        });
    }
  }
  // the activation x [B, K] once for every row group of a stage that has `groups` of them
  __device__ void activation(const bf16* x, int K, int B, int groups, int nch, int kc) {
    for (int gidx = 0; gidx < groups; ++gidx)
      for (int ch = 0; ch < nch; ++ch)
        tile(B, (uint32_t)kc * 2u, [&](int l) { return x + (size_t)l * K + (size_t)ch * kc; });
  }

  // Before the CTA ends after giving up: the copies that nobody waited for must have landed.
  __device__ void drain() {
    if (lane != 0) return;
    for (uint32_t k = (idx > NST ? idx - NST : 0); k < idx; ++k) {
      bool ok = false;
      for (uint32_t i = 0; i < tc::WAIT_LIMIT && !ok; ++i) ok = tc::mbar_try_wait(&full[k % NST], (k / NST) & 1u);
      if (!ok) atomicExch(err, ERR_DRAIN);
    }
  }
};

// ------------------------------------------------------------------ the consumers
template <class Geo>
struct Consumer {
  static constexpr int NSTAGE = Geo::NST, ASTAGE = Geo::AST, SROW = Geo::SROW, RS = Geo::RS;
  static constexpr int SLOT_BYTES = Geo::SLOT, ASLOT_BYTES = Geo::ASLOT;
  Shared* sh;
  uint8_t* slots;
  uint8_t* aslots;
  float* red;      // [2][NCW][128]
  uint32_t idx;    // weight tiles consumed
  uint32_t aidx;   // activation tiles consumed
  uint32_t nred;   // reductions done
  int warp, lane;
  int wk;          // which of the NCW ranges along K of a tile this warp sums: rotated from CTA to CTA
  int* err;
  // An activation that other CTAs wrote is complete in global memory (the grid barrier was passed): the
  // activation warp may stream it. Called by all consumer threads.
  __device__ __forceinline__ void act_begin() {
    if (warp == 0 && lane == 0) tc::mbar_arrive(&sh->act_ready);
  }

  // c += (tile rows) x (this warp's K range of the tile) . xf[XOFF ..]. MMA row r < 8 is tile row r, MMA
  // row 8 + r is tile row HI + r (8 for plain rows, PG for pairs); rows past the tile's end read its last row.
  template <int KTW, int HI, int XOFF, int NX>
  __device__ __forceinline__ void mma_tile(float (&c)[4], const uint32_t (&xf)[NX][2]) {
    const uint32_t slot = idx % NSTAGE, round = idx / NSTAGE;
    wait_or_abort(&sh->full[slot], round & 1u, sh, err, ERR_TILE_WAIT);
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* base = slots + (size_t)slot * SLOT_BYTES + (size_t)(wk * KTW * 16 + 4 * t) * 2;
    const uint8_t* lo_p = base + (size_t)g * SROW;
    const uint8_t* hi_p = base + (size_t)min(HI + g, RS - 1) * SROW;
    float c2[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // two chains of dependent MMAs instead of one
#pragma unroll
    for (int j = 0; j < KTW; ++j) {
      // the summation index inside a k-tile is permuted so that one 8-byte load holds both halves
      const uint2 lo = lds64(lo_p + j * 32), hi = lds64(hi_p + j * 32);
      const unsigned a[4] = {lo.x, hi.x, lo.y, hi.y};
      if (j & 1) mma_bf16_16816(c2, a, xf[XOFF + j][0], xf[XOFF + j][1]);
      else mma_bf16_16816(c, a, xf[XOFF + j][0], xf[XOFF + j][1]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] += c2[i];
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sh->empty[slot]);
    ++idx;
  }

  // the NCH tiles of one row group, piece after piece along K, with the activation's fragments in registers
  template <int KTW, int NCH, int HI, int NX, int CH = 0>
  __device__ __forceinline__ void row_group_local(float (&c)[4], const uint32_t (&xf)[NX][2]) {
    mma_tile<KTW, HI, CH * KTW>(c, xf);
    if constexpr (CH + 1 < NCH) row_group_local<KTW, NCH, HI, NX, CH + 1>(c, xf);
  }

  // the same with the activation's fragments taken from the streamed tiles, one beside every weight tile
  template <int KTW, int NCH, int HI>
  __device__ __forceinline__ void row_group_streamed(float (&c)[4]) {
    const int g = lane >> 2, t = lane & 3;
    for (int ch = 0; ch < NCH; ++ch) {
      const uint32_t slot = aidx % ASTAGE, round = aidx / ASTAGE;
      wait_or_abort(&sh->afull[slot], round & 1u, sh, err, ERR_TILE_WAIT);
      uint32_t xf[KTW][2];
      const uint8_t* xp = aslots + (size_t)slot * ASLOT_BYTES + (size_t)g * SROW + (size_t)(wk * KTW * 16 + 4 * t) * 2;
#pragma unroll
      for (int j = 0; j < KTW; ++j) {
        const uint2 v = lds64(xp + j * 32);
        xf[j][0] = v.x;
        xf[j][1] = v.y;
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->aempty[slot]);
      ++aidx;
      mma_tile<KTW, HI, 0>(c, xf);
    }
  }

  // Sum of the warps' accumulators: afterwards thread i < 128 of the consumers holds element
  // (MMA row i / 8, batch row i % 8); with `other` the element 64 further on too (MMA row + 8).
  __device__ __forceinline__ float reduce(const float (&c)[4], float* other) {
    float* buf = red + (nred & 1u) * (NCW * 128);
    const int g = lane >> 2, t = lane & 3;
    *reinterpret_cast<float2*>(buf + warp * 128 + g * 8 + 2 * t) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(buf + warp * 128 + 64 + g * 8 + 2 * t) = make_float2(c[2], c[3]);
    consumer_sync();
    ++nred;
    const int i = warp * 32 + lane;
    float s = 0.0f, s2 = 0.0f;
    if (i < 128) {
#pragma unroll
      for (int w = 0; w < NCW; ++w) s += buf[w * 128 + i];
      if (other && i < 64) {
#pragma unroll
        for (int w = 0; w < NCW; ++w) s2 += buf[w * 128 + 64 + i];
      }
    }
    if (other) *other = s2;
    return s;
  }

  // ---- the same for NT column tiles of 8 batch rows: one load of the weights' fragments feeds NT MMAs, which
  // are as many independent chains
  template <int KTW, int HI, int XOFF, int NT, int NX>
  __device__ __forceinline__ void mma_tile_nt(float (&c)[NT][4], const uint32_t (&xf)[NT][NX][2]) {
    const uint32_t slot = idx % NSTAGE, round = idx / NSTAGE;
    wait_or_abort(&sh->full[slot], round & 1u, sh, err, ERR_TILE_WAIT);
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* base = slots + (size_t)slot * SLOT_BYTES + (size_t)(wk * KTW * 16 + 4 * t) * 2;
    const uint8_t* lo_p = base + (size_t)g * SROW;
    const uint8_t* hi_p = base + (size_t)min(HI + g, RS - 1) * SROW;
#pragma unroll
    for (int j = 0; j < KTW; ++j) {
      const uint2 lo = lds64(lo_p + j * 32), hi = lds64(hi_p + j * 32);
      const unsigned a[4] = {lo.x, hi.x, lo.y, hi.y};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(c[nt], a, xf[nt][XOFF + j][0], xf[nt][XOFF + j][1]);
    }
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sh->empty[slot]);
    ++idx;
  }
  template <int KTW, int NCH, int HI, int NT, int NX, int CH = 0>
  __device__ __forceinline__ void row_group_local_nt(float (&c)[NT][4], const uint32_t (&xf)[NT][NX][2]) {
    mma_tile_nt<KTW, HI, CH * KTW>(c, xf);
    if constexpr (CH + 1 < NCH) row_group_local_nt<KTW, NCH, HI, NT, NX, CH + 1>(c, xf);
  }
  // the activation's fragments of all column tiles from the streamed tiles (row 8 nt + g of the tile)
  template <int KTW, int NCH, int NT>
  __device__ __forceinline__ void row_group_streamed_nt(float (&c)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    for (int ch = 0; ch < NCH; ++ch) {
      const uint32_t slot = aidx % ASTAGE, round = aidx / ASTAGE;
      wait_or_abort(&sh->afull[slot], round & 1u, sh, err, ERR_TILE_WAIT);
      uint32_t xf[NT][KTW][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint8_t* xp = aslots + (size_t)slot * ASLOT_BYTES + (size_t)(nt * 8 + g) * SROW + (size_t)(wk * KTW * 16 + 4 * t) * 2;
#pragma unroll
        for (int j = 0; j < KTW; ++j) {
          const uint2 v = lds64(xp + j * 32);
          xf[nt][j][0] = v.x;
          xf[nt][j][1] = v.y;
        }
      }
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->aempty[slot]);
      ++aidx;
      mma_tile_nt<KTW, 8, 0>(c, xf);
    }
  }
  // Sum of the warps' accumulators of all column tiles: thread i < 128 gets, per tile, element (MMA row i / 8,
  // batch row 8 nt + i % 8) in s, and with PAIR (i < 64) the element of MMA row + 8 in s2.
  template <int NT, bool PAIR>
  __device__ __forceinline__ void reduce_nt(const float (&c)[NT][4], float (&s)[NT], float (&s2)[NT]) {
    float* buf = red + (nred & 1u) * (NCW * 128 * NT);
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      *reinterpret_cast<float2*>(buf + (nt * NCW + warp) * 128 + g * 8 + 2 * t) = make_float2(c[nt][0], c[nt][1]);
      *reinterpret_cast<float2*>(buf + (nt * NCW + warp) * 128 + 64 + g * 8 + 2 * t) = make_float2(c[nt][2], c[nt][3]);
    }
    consumer_sync();
    ++nred;
    const int i = warp * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s[nt] = s2[nt] = 0.0f;
      if (i < 128) {
#pragma unroll
        for (int w = 0; w < NCW; ++w) s[nt] += buf[(nt * NCW + w) * 128 + i];
        if (PAIR && i < 64) {
#pragma unroll
          for (int w = 0; w < NCW; ++w) s2[nt] += buf[(nt * NCW + w) * 128 + 64 + i];
        }
      }
    }
  }
  template <int NT>
  __device__ __forceinline__ static void zero(float (&c)[NT][4]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.0f;
  }
  // rows [r0, r1): epi(row, n, sum) for batch rows n < B <= 8 * NT
  template <int KTW, int NCH, int NT, int NX, class Epi>
  __device__ __forceinline__ void rows_local_nt(const uint32_t (&xf)[NT][NX][2], int r0, int r1, int B, Epi epi) {
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[NT][4], s[NT], s2[NT];
      zero(c);
      row_group_local_nt<KTW, NCH, 8>(c, xf);
      reduce_nt<NT, false>(c, s, s2);
      const int i = warp * 32 + lane, row = i >> 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + (i & 7);
        if (i < 128 && row < nr && n < B) epi(rg + row, n, s[nt]);
      }
    }
  }
  template <int KTW, int NCH, int NT, int NX, class Epi>
  __device__ __forceinline__ void pairs_local_nt(const uint32_t (&xf)[NT][NX][2], int p0, int p1, int B, Epi epi) {
    constexpr int PG = Geo::PG;
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      float c[NT][4], s[NT], s2[NT];
      zero(c);
      row_group_local_nt<KTW, NCH, PG>(c, xf);
      reduce_nt<NT, true>(c, s, s2);
      const int i = warp * 32 + lane, pair = i >> 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + (i & 7);
        if (i < 64 && pair < np && n < B) epi(pg + pair, n, s[nt], s2[nt]);
      }
    }
  }
  template <int KTW, int NCH, int NT, class Epi>
  __device__ __forceinline__ void rows_streamed_nt(int r0, int r1, int B, Epi epi) {
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[NT][4], s[NT], s2[NT];
      zero(c);
      row_group_streamed_nt<KTW, NCH>(c);
      reduce_nt<NT, false>(c, s, s2);
      const int i = warp * 32 + lane, row = i >> 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + (i & 7);
        if (i < 128 && row < nr && n < B) epi(rg + row, n, s[nt]);
      }
    }
  }

  // ---- whole stages. epi(row, n, sum) is called by the thread that holds output (row, batch row n < B).
  // rows [r0, r1) of a projection whose activation's fragments are in registers
  template <int KTW, int NCH, int NX, class Epi>
  __device__ __forceinline__ void rows_local(const uint32_t (&xf)[NX][2], int r0, int r1, int B, Epi epi) {
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      row_group_local<KTW, NCH, 8>(c, xf);
      const float s = reduce(c, nullptr);
      const int i = warp * 32 + lane;
      const int row = i >> 3, n = i & 7;
      if (i < 128 && row < nr && n < B) epi(rg + row, n, s);
    }
  }
  // pairs [p0, p1) of a gated projection: epi(pair, n, gate sum, up sum)
  template <int KTW, int NCH, int NX, class Epi>
  __device__ __forceinline__ void pairs_local(const uint32_t (&xf)[NX][2], int p0, int p1, int B, Epi epi) {
    constexpr int PG = Geo::PG;
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      row_group_local<KTW, NCH, PG>(c, xf);
      float up;
      const float gate = reduce(c, &up);
      const int i = warp * 32 + lane;
      const int pair = i >> 3, n = i & 7;
      if (i < 64 && pair < np && n < B) epi(pg + pair, n, gate, up);
    }
  }
  // rows [r0, r1) of a projection whose activation the activation warp streams (after act_begin())
  template <int KTW, int NCH, class Epi>
  __device__ __forceinline__ void rows_streamed(int r0, int r1, int B, Epi epi) {
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      row_group_streamed<KTW, NCH, 8>(c);
      const float s = reduce(c, nullptr);
      const int i = warp * 32 + lane;
      const int row = i >> 3, n = i & 7;
      if (i < 128 && row < nr && n < B) epi(rg + row, n, s);
    }
  }
};

// All CTAs meet: every CTA adds one to a counter that only grows and waits until it reaches `target`
// (the next multiple of the grid size). Called by one thread per CTA, between two consumer_sync(): the
// barrier before orders the other threads' stores before the release here.
__device__ __forceinline__ void grid_arrive(unsigned long long* bar, Shared* sh) {
  if (sh->abort_flag) return;
  asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(bar) : "memory");
}
__device__ void grid_wait(unsigned long long* bar, unsigned long long target, Shared* sh, int* err) {
  if (sh->abort_flag) return;
  for (uint32_t i = 0; i < GRID_WAIT_LIMIT; ++i) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(bar) : "memory");
    if (v >= target) return;
  }
  sh->abort_flag = 1;
  atomicExch(err, ERR_GRID_WAIT);
}
__device__ __forceinline__ void grid_barrier(unsigned long long* bar, unsigned long long target, Shared* sh, int* err) {
  grid_arrive(bar, sh);
  grid_wait(bar, target, sh, err);
}

template <class Geo>
__device__ __forceinline__ void init_shared(Shared* sh) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < Geo::NST; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], NCW);
    }
    for (int s = 0; s < Geo::AST; ++s) {
      tc::mbar_init(&sh->afull[s], 1);
      tc::mbar_init(&sh->aempty[s], NCW);
    }
    tc::mbar_init(&sh->act_ready, 1);
    sh->abort_flag = 0;
    tc::mbar_init_fence();
  }
  __syncthreads();
}

// r = residual + x (fp32), h = rmsnorm(r) * w rounded to bf16 into shared memory rows of H * 2 + 32 bytes:
// consumer warp n does batch row n (rows from B on are zeros). `nw` holds this lane's norm weights, loaded
// by the caller. The sum is written to res_out where that is given.
template <int HT>
__device__ __forceinline__ void norm_rows(const bf16* x, const float* res_in, float* res_out, const uint2 (&nw)[HT],
                                          float eps, int B, uint8_t* xs, int warp, int lane) {
  constexpr int H = HT * NCW * 16, XS = H * 2 + 32;
  const int n = warp;
  uint8_t* xrow = xs + (size_t)n * XS;
  if (n < B) {
    float r[HT][4];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < HT; ++i) {
      const int e = (i * 32 + lane) * 4;
      const uint2 xv = __ldcg(reinterpret_cast<const uint2*>(x + (size_t)n * H + e));
      const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.x));
      const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.y));
      r[i][0] = x01.x; r[i][1] = x01.y; r[i][2] = x23.x; r[i][3] = x23.y;
      if (res_in) {
        const float4 q = __ldcg(reinterpret_cast<const float4*>(res_in + (size_t)n * H + e));
        r[i][0] = q.x + r[i][0]; r[i][1] = q.y + r[i][1]; r[i][2] = q.z + r[i][2]; r[i][3] = q.w + r[i][3];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += r[i][j] * r[i][j];
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < HT; ++i) {
      const int e = (i * 32 + lane) * 4;
      if (res_out) *reinterpret_cast<float4*>(res_out + (size_t)n * H + e) = make_float4(r[i][0], r[i][1], r[i][2], r[i][3]);
      const uint2 wv = nw[i];
      const float2 w01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.x));
      const float2 w23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.y));
      uint2 o;
      o.x = pack_bf16(r[i][0] * rstd * w01.x, r[i][1] * rstd * w01.y);
      o.y = pack_bf16(r[i][2] * rstd * w23.x, r[i][3] * rstd * w23.y);
      *reinterpret_cast<uint2*>(xrow + e * 2) = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < HT; ++i) *reinterpret_cast<uint2*>(xrow + (i * 32 + lane) * 8) = make_uint2(0u, 0u);
  }
}

// this warp's fragments of the normalised rows, for all pieces along K
template <int HT, int KTW, int NCH>
__device__ __forceinline__ void load_local_x(uint32_t (&xf)[HT][2], const uint8_t* xs, int wk, int lane) {
  constexpr int H = HT * NCW * 16, XS = H * 2 + 32, KC = KTW * NCW * 16;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int j = 0; j < KTW; ++j) {
      const int k0 = ch * KC + (wk * KTW + j) * 16 + 4 * t;
      const uint2 v = lds64(xs + (size_t)g * XS + k0 * 2);
      xf[ch * KTW + j][0] = v.x;
      xf[ch * KTW + j][1] = v.y;
    }
}

// The norm in front of a projection, by every CTA itself: r = res_in + x, h = rmsnorm(r) * w into shared memory
// (CTA 0 also writes r to res_out), then this warp's fragments of h. `wait_pdl`: the kernel's first use of
// anything the kernel before it wrote; the norm's weights are fetched before that wait.
template <int HT, int KTW, int NCH>
__device__ __forceinline__ void norm_to_fragments(uint32_t (&xf)[HT][2], const bf16* x, const float* res_in, float* res_out,
                                                  const bf16* norm_w, float eps, int B, uint8_t* xs, int warp, int lane,
                                                  int wk, bool wait_pdl) {
  uint2 nw[HT];
#pragma unroll
  for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(norm_w + (i * 32 + lane) * 4);
  if (wait_pdl) pdl_wait();
  norm_rows<HT>(x, res_in, blockIdx.x == 0 ? res_out : nullptr, nw, eps, B, xs, warp, lane);
  consumer_sync();
  load_local_x<HT, KTW, NCH>(xf, xs, wk, lane);
}

// The same for 8 * NT batch rows: fragments per column tile.
template <int HT, int KTW, int NCH, int NT>
__device__ __forceinline__ void norm_to_fragments_nt(uint32_t (&xf)[NT][HT][2], const bf16* x, const float* res_in,
                                                     float* res_out, const bf16* norm_w, float eps, int B, uint8_t* xs,
                                                     int warp, int lane, int wk, bool wait_pdl) {
  constexpr int H = HT * NCW * 16, XS = H * 2 + 32;
  uint2 nw[HT];
#pragma unroll
  for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(norm_w + (i * 32 + lane) * 4);
  if (wait_pdl) pdl_wait();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    norm_rows<HT>(x + (size_t)nt * 8 * H, res_in ? res_in + (size_t)nt * 8 * H : nullptr,
                  blockIdx.x == 0 ? res_out + (size_t)nt * 8 * H : nullptr, nw, eps, B - nt * 8, xs + (size_t)nt * 8 * XS, warp,
                  lane);
  consumer_sync();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) load_local_x<HT, KTW, NCH>(xf[nt], xs + (size_t)nt * 8 * XS, wk, lane);
}

// The consumers of all CTAs meet (see grid_arrive / grid_wait). `for_bulk_copies`: what this CTA stored is read
// by other CTAs' bulk copies next.
struct GridSync {
  unsigned long long* bar;
  unsigned long long target;   // kept by thread 0
  unsigned G;
  Shared* sh;
  int* err;
  // after the kernel's wait for the kernel before it: no CTA passes the first barrier before this one arrives,
  // so the counter is less than a grid size past the multiple that the launch started from
  __device__ __forceinline__ void begin() {
    if (threadIdx.x == 0) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(bar) : "memory");
      target = v - v % (unsigned long long)G;
    }
  }
  __device__ __forceinline__ void arrive(bool for_bulk_copies) {
    if (for_bulk_copies) publish_for_bulk_copies();
    consumer_sync();
    if (threadIdx.x == 0) {
      grid_arrive(bar, sh);
      target += (unsigned long long)G;
    }
  }
  __device__ __forceinline__ void wait() {
    if (threadIdx.x == 0) grid_wait(bar, target, sh, err);
    consumer_sync();
  }
  __device__ __forceinline__ void sync(bool for_bulk_copies) {
    arrive(for_bulk_copies);
    wait();
  }
};

// What the attention stage needs beside q, k, v of the step: the cache and the step's tables, as
// osb_attn_decode_stream takes them.
struct AttnTables {
  bf16* k_cache;
  bf16* v_cache;
  const int* block_table;
  const int* cu_q;
  const int* seq_lens;
  const int* decode_index;
  int* counters;
  float* part_o;
  float* part_ml;
  attn_stream::FusedRope rope;
  float scale_log2;
  int bt_stride, nh, nkv, log2ps, num_pages, window, nsplits;
};

// Rotary encoding, the new key and value into the cache, attention over the cache: units (request, kv head,
// split of the keys), one per CTA and turn; the CTA that finishes a (request, kv head) last merges its splits.
// Called after gs.arrive(): the first unit looks up its pages and starts its first loads before it waits
// for the other CTAs' q, k, v.
template <int HD>
__device__ __forceinline__ void attention_stage(const AttnTables& a, const bf16* qkv, int NQKV, bf16* attn, int B,
                                                GridSync& gs, uint8_t* scratch, Shared* sh) {
  const int grp = a.nh / a.nkv;
  const int ny = a.nkv * ((grp + 7) >> 3);
  const int units = B * ny * a.nsplits;
  bool waited = false;
  auto wait_qkv = [&] {
    if (!waited) {
      gs.wait();
      waited = true;
    }
  };
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int split = u % a.nsplits, rest = u / a.nsplits;
    attn_stream::attn_stream_unit<HD, false, true>(
        wait_qkv, split, rest % ny, rest / ny, ny, scratch, &sh->s_last, attn, a.part_o, a.part_ml, qkv, NQKV, a.k_cache,
        a.v_cache, a.block_table, a.bt_stride, a.cu_q, a.seq_lens, a.decode_index, a.counters, a.nh, a.nkv, a.log2ps,
        a.num_pages, a.scale_log2, a.window, 0, a.nsplits, a.rope);
    wait_qkv();        // a unit that has nothing to do returns before it waits
    consumer_sync();   // the scratch in shared memory is used again by the next unit and by the tiles after it
  }
  wait_qkv();
}

// Shared memory of every kernel here: weight tiles, activation tiles (the normalised rows and the attention's
// scratch use the same bytes at other times), the reduction buffers, the barriers.
template <class Geo>
struct Carve {
  uint8_t *slots, *aslots, *xs;
  float* red;
  Shared* sh;
  __device__ __forceinline__ explicit Carve(uint8_t* smem) {
    slots = smem;
    aslots = slots + Geo::NST * Geo::SLOT;
    xs = aslots;
    red = reinterpret_cast<float*>(aslots + Geo::AST * Geo::ASLOT);
    sh = reinterpret_cast<Shared*>(red + Geo::RED_FLOATS);
  }
};

template <class Geo> using WeightStreamOf = Streamer<Geo::NST, Geo::SLOT, Geo::SROW, Geo::RS, true>;
template <class Geo> using ActStreamOf = Streamer<Geo::AST, Geo::ASLOT, Geo::SROW, Geo::RS, false>;

// How a K of KT * 128 elements is cut into pieces of a tile's length
template <int KT, class Geo>
struct Pieces {
  static constexpr int KTW = largest_divisor_le(KT, Geo::MAX_KTW), NCH = KT / KTW, KC = KTW * NCW * 16;
};

__device__ __forceinline__ float silu_mul(float gate, float up) { return (gate / (1.0f + expf(-gate))) * up; }

// The feed-forward half: r = res_in + x; h = rmsnorm(r) * w; act = silu(h Wg^T) * (h Wu^T) -- grid barrier --
// y = act Wd^T. The consumers' part; `first`: nothing of this kernel has waited for the kernel before it yet.
template <int HT, int IT, class Geo>
__device__ __forceinline__ void ffn_half(Consumer<Geo>& co, GridSync& gs, uint8_t* xs, const bf16* x, const float* res_in,
                                         float* res_out, const bf16* norm_w, float eps, bf16* act, bf16* y, int B, int p0,
                                         int p1, int r0, int r1, bool first) {
  constexpr int H = HT * NCW * 16, I = IT * NCW * 16;
  typedef Pieces<HT, Geo> PH;
  typedef Pieces<IT, Geo> PI;
  constexpr int NT = Geo::NT;
  auto store_act = [&](int pair, int n, float gate, float up) { act[(size_t)n * I + pair] = __float2bfloat16_rn(silu_mul(gate, up)); };
  auto store_y = [&](int row, int n, float s) { y[(size_t)n * H + row] = __float2bfloat16_rn(s); };
  {
    uint32_t xf[NT][HT][2];
    norm_to_fragments_nt<HT, PH::KTW, PH::NCH>(xf, x, res_in, res_out, norm_w, eps, B, xs, co.warp, co.lane, co.wk, first);
    if (first) gs.begin();
    FTL(2);
    if constexpr (NT == 1) co.template pairs_local<PH::KTW, PH::NCH>(xf[0], p0, p1, B, store_act);
    else co.template pairs_local_nt<PH::KTW, PH::NCH>(xf, p0, p1, B, store_act);
  }
  FTL(4);
  gs.sync(true);   // also: every warp has its fragments out of xs, whose memory the activation tiles use next
  FTL(6);
  if (first) pdl_trigger();
  co.act_begin();
  if constexpr (NT == 1) co.template rows_streamed<PI::KTW, PI::NCH>(r0, r1, B, store_y);
  else co.template rows_streamed_nt<PI::KTW, PI::NCH, NT>(r0, r1, B, store_y);
}

template <int HT, int IT, class Geo>
__global__ void __launch_bounds__(NTHREADS_ACT, 1) ffn_decode_fused_kernel(const __grid_constant__ FfnParams p) {
  constexpr int H = HT * NCW * 16, I = IT * NCW * 16;
  typedef Pieces<HT, Geo> PH;
  typedef Pieces<IT, Geo> PI;
  static_assert(Geo::NT * MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows share the activation tiles' memory");
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int p0, p1, r0, r1;
  cta_rows(I, cta, G, p0, p1);
  cta_rows(H, cta, G, r0, r1);

  if (warp == W_WARP) {
    // the weights depend on nothing that runs before this kernel: the stream starts at once
    WeightStreamOf<Geo> ws{sh, sh->full, sh->empty, m.slots, 0u, policy_evict_first(), lane, p.err};
    FTL(10);
    ws.pairs(p.w_gate_up, H, I, p0, p1, PH::NCH, PH::KC);
    FTL(11);
    ws.rows(p.w_down, I, r0, r1, PI::NCH, PI::KC);
    FTL(12);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  if (warp == A_WARP) {
    ActStreamOf<Geo> as{sh, sh->afull, sh->aempty, m.aslots, 0u, 0ull, lane, p.err};
    wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
    as.activation(p.act, I, p.B, (r1 - r0 + Geo::RS - 1) / Geo::RS, PI::NCH, PI::KC);
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  Consumer<Geo> co{sh, m.slots, m.aslots, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  GridSync gs{p.bar, 0ull, (unsigned)G, sh, p.err};
  FTL(0);
  ffn_half<HT, IT, Geo>(co, gs, m.xs, p.x, p.res_in, p.res_out, p.norm_w, p.eps, p.act, p.y, p.B, p0, p1, r0, r1, true);
  FTL(9);
  __syncthreads();
}

struct NormLinearParams {
  const bf16* x;        // [B, H] branch output of the part before
  const float* res_in;  // [B, H] or null
  float* res_out;       // [B, H]
  const bf16* norm_w;   // [H], or null: no norm (then no res_in, no res_out)
  const bf16* w;        // [N, H]
  const bf16* bias;     // [N] or null
  bf16* y;              // [B, N]
  int* err;
  float eps;
  int B, N;
};

// y = (rmsnorm(res_in + x) * norm_w) W^T + bias for a few rows: every CTA normalises the rows itself while
// its rows of W are already on their way; no CTA waits for another. Without norm_w: y = x W^T + bias.
template <int HT, class Geo>
__global__ void __launch_bounds__(NTHREADS, 1) norm_linear_decode_kernel(const __grid_constant__ NormLinearParams p) {
  constexpr int H = HT * NCW * 16, NT = Geo::NT, XS = H * 2 + 32;
  typedef Pieces<HT, Geo> PH;
  static_assert(NT * MAX_B * XS <= Geo::AST * Geo::ASLOT, "the normalised rows use the activation tiles' memory");
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int r0, r1;
  cta_rows(p.N, cta, G, r0, r1);

  if (warp == W_WARP) {
    WeightStreamOf<Geo> ws{sh, sh->full, sh->empty, m.slots, 0u, policy_evict_first(), lane, p.err};
    ws.rows(p.w, H, r0, r1, PH::NCH, PH::KC);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  Consumer<Geo> co{sh, m.slots, m.xs, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  uint32_t xf[NT][HT][2];   // batch rows 8 nt .. 8 nt + 7
  if (p.norm_w != nullptr) {
    norm_to_fragments_nt<HT, PH::KTW, PH::NCH>(xf, p.x, p.res_in, p.res_out, p.norm_w, p.eps, p.B, m.xs, warp, lane, co.wk, true);
  } else {
    // no norm in front: the rows' fragments come straight from global memory
    pdl_wait();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int ch = 0; ch < PH::NCH; ++ch)
#pragma unroll
        for (int j = 0; j < PH::KTW; ++j) {
          const int k0 = ch * PH::KC + (co.wk * PH::KTW + j) * 16 + 4 * t;
          uint2 v = make_uint2(0u, 0u);
          if (nt * 8 + g < p.B) v = __ldcg(reinterpret_cast<const uint2*>(p.x + (size_t)(nt * 8 + g) * H + k0));
          xf[nt][ch * PH::KTW + j][0] = v.x;
          xf[nt][ch * PH::KTW + j][1] = v.y;
        }
  }
  pdl_trigger();
  auto store = [&](int row, int n, float s) {
    if (p.bias) s += __bfloat162float(p.bias[row]);
    p.y[(size_t)n * p.N + row] = __float2bfloat16_rn(s);
  };
  if constexpr (NT == 1) co.template rows_local<PH::KTW, PH::NCH>(xf[0], r0, r1, p.B, store);
  else co.template rows_local_nt<PH::KTW, PH::NCH>(xf, r0, r1, p.B, store);
  __syncthreads();
}

// The attention half of a layer for a decode step of up to 8 requests:
//   r = res_in + x; h = rmsnorm(r) * w; qkv = h Wqkv^T + b       (rows of Wqkv split over the CTAs)
//   -- grid barrier --  attention_stage()  -- grid barrier --
//   y = attn Wo^T                                                 (rows of Wo split over the CTAs)
// The rows of Wo are on their way into shared memory while the attention runs.
// Formulas: omniserve/model/qwen2_llm.py:75-113.
template <int HT, int OT, int HD, class Geo>
__device__ __forceinline__ void attn_half(Consumer<Geo>& co, GridSync& gs, const Carve<Geo>& m, const bf16* x,
                                          const float* res_in, float* res_out, const bf16* norm_w, float eps,
                                          const bf16* b_qkv, int NQKV, bf16* qkv, bf16* attn, bf16* y, int B,
                                          const AttnTables& tables, int q0, int q1, int r0, int r1, bool first) {
  constexpr int H = HT * NCW * 16;
  typedef Pieces<HT, Geo> PH;
  typedef Pieces<OT, Geo> PO;
  {
    uint32_t xf[HT][2];
    norm_to_fragments<HT, PH::KTW, PH::NCH>(xf, x, res_in, res_out, norm_w, eps, B, m.xs, co.warp, co.lane, co.wk, first);
    if (first) gs.begin();
    co.template rows_local<PH::KTW, PH::NCH>(xf, q0, q1, B, [&](int row, int n, float s) {
      if (b_qkv) s += __bfloat162float(b_qkv[row]);
      qkv[(size_t)n * NQKV + row] = __float2bfloat16_rn(s);
    });
  }
  gs.arrive(false);
  attention_stage<HD>(tables, qkv, NQKV, attn, B, gs, m.aslots, m.sh);
  gs.sync(true);
  if (first) pdl_trigger();
  co.act_begin();
  co.template rows_streamed<PO::KTW, PO::NCH>(r0, r1, B, [&](int row, int n, float s) {
    y[(size_t)n * H + row] = __float2bfloat16_rn(s);
  });
}

struct AttnHalfParams {
  const bf16* x;          // [B, H] branch output of the part before
  const float* res_in;    // [B, H] or null
  float* res_out;         // [B, H]
  const bf16* norm_w;     // [H]
  const bf16* w_qkv;      // [NQKV, H]: q heads, k heads, v heads
  const bf16* b_qkv;      // [NQKV] or null
  const bf16* w_o;        // [H, nh * hd]
  bf16* qkv;              // [B, NQKV] scratch
  bf16* attn;             // [B, nh * hd] scratch
  bf16* y;                // [B, H]
  unsigned long long* bar;
  int* err;
  float eps;
  int B, NQKV;
  AttnTables t;
};

// the attention's q rows, per-warp (max, sum) and outputs use the activation tiles and the reduction buffers
template <int HD, class Geo>
__host__ __device__ constexpr bool attention_scratch_fits() {
  return 16 * (HD + 8) * 2 + NCW * 16 * 2 * 4 + 16 * 2 * 4 + NCW * 16 * (HD + 8) * 4 <= Geo::AST * Geo::ASLOT + Geo::RED_FLOATS * 4;
}

template <int HT, int OT, int HD, class Geo>
__global__ void __launch_bounds__(NTHREADS_WIDE, 1) attn_decode_fused_kernel(const __grid_constant__ AttnHalfParams p) {
  constexpr int H = HT * NCW * 16, OD = OT * NCW * 16;
  typedef Pieces<HT, Geo> PH;
  typedef Pieces<OT, Geo> PO;
  static_assert(MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows share the activation tiles' memory");
  static_assert(attention_scratch_fits<HD, Geo>(), "the attention's scratch does not fit");
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int q0, q1, r0, r1;
  cta_rows(p.NQKV, cta, G, q0, q1);
  cta_rows(H, cta, G, r0, r1);

  if (warp >= W_WARP) reg_give<PRODUCER_REGS>();   // all four warps of the last warp group, at one place
  if (warp > A_WARP) return;
  if (warp == A_WARP) {
    ActStreamOf<Geo> as{sh, sh->afull, sh->aempty, m.aslots, 0u, 0ull, lane, p.err};
    wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
    as.activation(p.attn, OD, p.B, (r1 - r0 + Geo::RS - 1) / Geo::RS, PO::NCH, PO::KC);
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  if (warp == W_WARP) {
    WeightStreamOf<Geo> ws{sh, sh->full, sh->empty, m.slots, 0u, policy_evict_first(), lane, p.err};
    ws.rows(p.w_qkv, H, q0, q1, PH::NCH, PH::KC);
    ws.rows(p.w_o, OD, r0, r1, PO::NCH, PO::KC);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  reg_take<CONSUMER_REGS>();
  Consumer<Geo> co{sh, m.slots, m.aslots, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  GridSync gs{p.bar, 0ull, (unsigned)G, sh, p.err};
  attn_half<HT, OT, HD, Geo>(co, gs, m, p.x, p.res_in, p.res_out, p.norm_w, p.eps, p.b_qkv, p.NQKV, p.qkv, p.attn, p.y, p.B,
                             p.t, q0, q1, r0, r1, true);
  __syncthreads();
}

// One layer of the schedule for decode_layers_fused_kernel: device pointers and constants.
struct LayerDesc {
  const bf16 *norm_attn, *w_qkv, *b_qkv, *w_o, *norm_ffn, *w_gate_up, *w_down;
  bf16 *k_cache, *v_cache;
  float eps_attn, eps_ffn;
  int window, num_pages, log2ps, pad_;
};

struct LayersParams {
  const LayerDesc* layers;
  int n_layers;
  const bf16* x;        // [B, H] what the embedding gave
  const float* res_in;  // [B, H] or null
  float* res_a;         // [B, H] the residual stream, written in turn: res_a by the first norm, res_b by the second, ...
  float* res_b;
  bf16* y;              // [B, H] every half's output; the last one is the kernel's result
  bf16 *qkv, *attn, *act;   // scratch: [B, NQKV], [B, nh * hd], [B, I]
  unsigned long long* bar;
  int* err;
  int B, NQKV;
  AttnTables t;         // k_cache, v_cache, window, num_pages, log2ps: taken from the layer's record instead
};

// A run of pre-norm layers (attention half, feed-forward half) for a decode step of up to 8 requests as ONE
// kernel: attn_half and ffn_half layer after layer, five grid barriers per layer, with the weights of all
// layers as one uninterrupted stream through shared memory. The residual stream alternates between two
// buffers (CTA 0 writes the sum that every CTA computes), the halves hand their output on in y.
template <int HT, int OT, int IT, int HD, class Geo>
__global__ void __launch_bounds__(NTHREADS_WIDE, 1) decode_layers_fused_kernel(const __grid_constant__ LayersParams p) {
  constexpr int H = HT * NCW * 16, OD = OT * NCW * 16, I = IT * NCW * 16;
  typedef Pieces<HT, Geo> PH;
  typedef Pieces<OT, Geo> PO;
  typedef Pieces<IT, Geo> PI;
  static_assert(MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows share the activation tiles' memory");
  static_assert(attention_scratch_fits<HD, Geo>(), "the attention's scratch does not fit");
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int q0, q1, r0, r1, p0, p1;
  cta_rows(p.NQKV, cta, G, q0, q1);
  cta_rows(H, cta, G, r0, r1);
  cta_rows(I, cta, G, p0, p1);

  if (warp >= W_WARP) reg_give<PRODUCER_REGS>();   // all four warps of the last warp group, at one place
  if (warp > A_WARP) return;
  if (warp == A_WARP) {
    ActStreamOf<Geo> as{sh, sh->afull, sh->aempty, m.aslots, 0u, 0ull, lane, p.err};
    const int groups = (r1 - r0 + Geo::RS - 1) / Geo::RS;
    for (int l = 0; l < p.n_layers; ++l) {
      wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
      as.activation(p.attn, OD, p.B, groups, PO::NCH, PO::KC);
      wait_or_abort(&sh->act_ready, 1u, sh, p.err, ERR_GRID_WAIT);
      as.activation(p.act, I, p.B, groups, PI::NCH, PI::KC);
    }
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  if (warp == W_WARP) {
    WeightStreamOf<Geo> ws{sh, sh->full, sh->empty, m.slots, 0u, policy_evict_first(), lane, p.err};
    for (int l = 0; l < p.n_layers; ++l) {
      const LayerDesc& L = p.layers[l];
      ws.rows(L.w_qkv, H, q0, q1, PH::NCH, PH::KC);
      ws.rows(L.w_o, OD, r0, r1, PO::NCH, PO::KC);
      ws.pairs(L.w_gate_up, H, I, p0, p1, PH::NCH, PH::KC);
      ws.rows(L.w_down, I, r0, r1, PI::NCH, PI::KC);
    }
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }

  reg_take<CONSUMER_REGS>();
  Consumer<Geo> co{sh, m.slots, m.aslots, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  GridSync gs{p.bar, 0ull, (unsigned)G, sh, p.err};
  const bf16* x_cur = p.x;
  const float* r_cur = p.res_in;
  for (int l = 0; l < p.n_layers; ++l) {
    const LayerDesc& L = p.layers[l];
    AttnTables t = p.t;
    t.k_cache = L.k_cache;
    t.v_cache = L.v_cache;
    t.window = L.window;
    t.num_pages = L.num_pages;
    t.log2ps = L.log2ps;
    attn_half<HT, OT, HD, Geo>(co, gs, m, x_cur, r_cur, p.res_a, L.norm_attn, L.eps_attn, L.b_qkv, p.NQKV, p.qkv, p.attn, p.y,
                               p.B, t, q0, q1, r0, r1, l == 0);
    gs.sync(false);    // the norm that follows reads y and the residual stream that CTA 0 wrote
    ffn_half<HT, IT, Geo>(co, gs, m.xs, p.y, p.res_a, p.res_b, L.norm_ffn, L.eps_ffn, p.act, p.y, p.B, p0, p1, r0, r1, false);
    x_cur = p.y;
    r_cur = p.res_b;
    if (l + 1 < p.n_layers) gs.sync(false);
  }
  __syncthreads();
}

int& fused_with_pdl() {
  static int v = 1;
  return v;
}
int& fused_cooperative() {
  static int v = 1;
  return v;
}

template <class Geo>
constexpr size_t fused_smem_bytes() {
  return (size_t)Geo::NST * Geo::SLOT + (size_t)Geo::AST * Geo::ASLOT + Geo::RED_FLOATS * sizeof(float) + sizeof(Shared);
}

// One CTA per SM. `cooperative`: the CTAs wait for one another, so the launch must fail rather than start
// a part of them.
template <class Geo, class Params>
int launch_fused(void (*kernel)(Params), const Params& p, int n_sm, bool cooperative, cudaStream_t stream,
                 int threads = NTHREADS) {
  constexpr size_t smem = fused_smem_bytes<Geo>();
  static_assert(smem <= 232448, "more shared memory than a CTA can have");
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int& with_pdl = fused_with_pdl();
  for (;;) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_sm);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cooperative && fused_cooperative()) {
      attr[n].id = cudaLaunchAttributeCooperative;
      attr[n].val.cooperative = 1;
      ++n;
    }
    if (with_pdl && osb_pdl_enabled()) {
      attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    e = cudaLaunchKernelEx(&cfg, kernel, p);
    if (e == cudaSuccess) return OSB_OK;
    if (n == 2 && with_pdl) {  // the two attributes may not go together on this driver
      (void)cudaGetLastError();
      with_pdl = 0;
      continue;
    }
    return (int)e;
  }
}

template <int HT, int IT, class Geo>
int launch_ffn(const FfnParams& p, int n_sm, cudaStream_t stream) {
  return launch_fused<Geo>(ffn_decode_fused_kernel<HT, IT, Geo>, p, n_sm, true, stream, NTHREADS_ACT);
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace

// Diagnostics: whether the launches carry the programmatic-dependent-launch attribute (it is dropped when
// the driver refuses it beside the cooperative one), and a switch for the cooperative attribute.
OSB_API int osb_fused_pdl_state() { return fused_with_pdl(); }
OSB_API void osb_fused_set_cooperative(int on) { fused_cooperative() = on; }

// 1 when the fused feed-forward has a build for these sizes.
OSB_API int osb_ffn_decode_fused_supported(int H, int I) {
  return (H == 1536 && I == 8960) || (H == 256 && I == 512) || (H == 384 && I == 1920) || (H == 2048 && I == 256);
}

// y [B,H] = down(silu(gate(h)) * up(h)), h = rmsnorm(res_in + x) * norm_w; res_out = res_in + x (fp32).
// B <= 16, bf16 weights and activations. `act` [B,I] is scratch; `bar` is a zeroed 64-bit counter that belongs
// to these launches alone (between launches it is a multiple of the number of SMs); `err` is the device error flag.
OSB_API int osb_ffn_decode_fused(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w,
                                 float eps, const void* w_gate_up, const void* w_down, void* act, unsigned long long* bar,
                                 int* err, int B, int H, int I, cudaStream_t stream) {
  if (B <= 0) return OSB_OK;
  if (B > 2 * MAX_B || !osb_ffn_decode_fused_supported(H, I)) return OSB_ERR_UNSUPPORTED;
  if ((((uintptr_t)y | (uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w_gate_up |
        (uintptr_t)w_down | (uintptr_t)act) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  FfnParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w;
  p.w_gate_up = (const bf16*)w_gate_up; p.w_down = (const bf16*)w_down; p.act = (bf16*)act; p.y = (bf16*)y;
  p.bar = bar; p.err = err; p.eps = eps; p.B = B; p.H = H; p.I = I;
  const int n_sm = sm_count();
  if (B > MAX_B) {   // 9 to 16 rows: two column tiles, activation tiles of 16 rows, two weight tiles in flight
    typedef Geometry<16, 12, 2, 2, 2> GeoB2;
    typedef Geometry<12, 7, 5, 3, 2> GeoA2;
    typedef Geometry<16, 8, 2, 2, 2> GeoC2;
    if (H == 1536 && I == 8960) return launch_ffn<12, 70, GeoB2>(p, n_sm, stream);
    if (H == 256 && I == 512) return launch_ffn<2, 4, GeoB2>(p, n_sm, stream);
    if (H == 384 && I == 1920) return launch_ffn<3, 15, GeoA2>(p, n_sm, stream);
    return launch_ffn<16, 2, GeoC2>(p, n_sm, stream);
  }
  typedef Geometry<16, 12, 3, 3> GeoB;
  typedef Geometry<12, 7, 7, 4> GeoA;
  if (H == 1536 && I == 8960) return launch_ffn<12, 70, GeoB>(p, n_sm, stream);
  if (H == 256 && I == 512) return launch_ffn<2, 4, GeoB>(p, n_sm, stream);
  if (H == 384 && I == 1920) return launch_ffn<3, 15, GeoA>(p, n_sm, stream);
  return launch_ffn<16, 2, GeoB>(p, n_sm, stream);
}

// 1 when the fused attention half has a build for these sizes (hidden size, heads * head size, head size).
OSB_API int osb_attn_decode_fused_supported(int H, int OD, int hd) {
  return (H == 1536 && OD == 1536 && hd == 128) || (H == 256 && OD == 256 && hd == 64) ||
         (H == 384 && OD == 512 && hd == 128) || (H == 2048 && OD == 256 && hd == 64);
}

// y [B,H] = attention(rmsnorm(res_in + x) * norm_w) Wo^T for a decode step of B <= 8 requests with one new
// token each (row s of x is request s); res_out = res_in + x (fp32). The projections' weights are bf16; q and k
// are rotated by the tables and the new key and value are stored at rope_slot_map, as osb_attn_decode_stream
// does in its fused rotary form; the cache arguments, part_o / part_ml / counters (for nsplits) and the tables
// have the meaning they have there. qkv [B,NQKV] and attn [B, nh*hd] are scratch; bar as for osb_ffn_decode_fused.
OSB_API int osb_attn_decode_fused(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w,
                                  float eps, const void* w_qkv, const void* b_qkv, const void* w_o, void* qkv,
                                  void* attn, unsigned long long* bar, int* err, int B, int H, void* k_cache,
                                  void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                                  const int* seq_lens, const int* decode_index, int nh, int nkv, int hd, int page_size,
                                  int num_pages, float scale, int window, float* part_o, float* part_ml, int* counters,
                                  int nsplits, const float* rope_cos, const float* rope_sin, const int* rope_slot_map,
                                  int rope_rot, cudaStream_t stream) {
  if (B <= 0) return OSB_OK;
  const int OD = nh * hd, NQKV = (nh + 2 * nkv) * hd;
  if (B > MAX_B || nkv <= 0 || nh % nkv != 0 || nh / nkv > 8 || !osb_attn_decode_fused_supported(H, OD, hd))
    return OSB_ERR_UNSUPPORTED;
  if (page_size < 1 || (page_size & (page_size - 1)) || nsplits < 1 || rope_cos == nullptr) return OSB_ERR_UNSUPPORTED;
  if (rope_rot <= 0 || rope_rot > hd || (rope_rot & 1)) return OSB_ERR_BAD_SHAPE;
  // the merging CTA's table of the splits' (max, sum) lives where the warps' outputs were
  if ((size_t)8 * nsplits * 2 > (size_t)NCW * 16 * (hd + 8)) return OSB_ERR_TOO_LARGE;
  if ((((uintptr_t)y | (uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w_qkv |
        (uintptr_t)w_o | (uintptr_t)qkv | (uintptr_t)attn | (uintptr_t)k_cache | (uintptr_t)v_cache |
        (uintptr_t)rope_cos | (uintptr_t)rope_sin | (uintptr_t)part_o) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  int log2ps = 0;
  while ((1 << log2ps) < page_size) ++log2ps;
  AttnHalfParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w;
  p.w_qkv = (const bf16*)w_qkv; p.b_qkv = (const bf16*)b_qkv; p.w_o = (const bf16*)w_o; p.qkv = (bf16*)qkv;
  p.attn = (bf16*)attn; p.y = (bf16*)y; p.bar = bar; p.err = err; p.eps = eps; p.B = B; p.NQKV = NQKV;
  p.t.k_cache = (bf16*)k_cache; p.t.v_cache = (bf16*)v_cache; p.t.block_table = block_table; p.t.cu_q = cu_q;
  p.t.seq_lens = seq_lens; p.t.decode_index = decode_index; p.t.counters = counters; p.t.part_o = part_o; p.t.part_ml = part_ml;
  p.t.rope.cos_t = rope_cos; p.t.rope.sin_t = rope_sin; p.t.rope.slot_map = rope_slot_map; p.t.rope.rot = rope_rot;
  p.t.scale_log2 = scale * 1.4426950408889634f;
  p.t.bt_stride = bt_stride; p.t.nh = nh; p.t.nkv = nkv; p.t.log2ps = log2ps; p.t.num_pages = num_pages;
  p.t.window = window; p.t.nsplits = nsplits;
  typedef Geometry<16, 12, 3, 3> GeoB;
  const int n_sm = sm_count();
  if (H == 1536) return launch_fused<GeoB>(attn_decode_fused_kernel<12, 12, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  if (H == 256) return launch_fused<GeoB>(attn_decode_fused_kernel<2, 2, 64, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  if (H == 384) return launch_fused<GeoB>(attn_decode_fused_kernel<3, 4, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  return launch_fused<GeoB>(attn_decode_fused_kernel<16, 2, 64, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
}

// 1 when decode_layers_fused has a build for these sizes.
OSB_API int osb_decode_layers_fused_supported(int H, int OD, int I, int hd) {
  return (H == 1536 && OD == 1536 && I == 8960 && hd == 128) || (H == 256 && OD == 256 && I == 512 && hd == 64) ||
         (H == 384 && OD == 512 && I == 1920 && hd == 128);
}
OSB_API int osb_decode_layer_desc_bytes() { return (int)sizeof(LayerDesc); }

// A run of n_layers pre-norm layers for a decode step of B <= 8 single-token requests. `layers` is a device
// array of n_layers records of osb_decode_layer_desc_bytes() bytes each, filled by the caller in this order
// (all pointers device pointers): norm_attn, w_qkv, b_qkv (or 0), w_o, norm_ffn, w_gate_up, w_down, k_cache,
// v_cache (8 bytes each), eps_attn, eps_ffn (float), window, num_pages, log2 of the page size, 0 (int). All
// layers share the block table and the slot map of one cache group. On return y [B,H] is the last half's output and the residual stream is in
// res_b (an even number of norms ran). The other arguments as for osb_attn_decode_fused / osb_ffn_decode_fused.
OSB_API int osb_decode_layers_fused(const void* layers, int n_layers, void* y, float* res_a, float* res_b, const void* x,
                                    const float* res_in, void* qkv, void* attn, void* act, unsigned long long* bar,
                                    int* err, int B, int H, int I, const int* block_table, int bt_stride,
                                    const int* slot_map, const int* cu_q, const int* seq_lens,
                                    const int* decode_index, int nh, int nkv, int hd, float scale, float* part_o,
                                    float* part_ml, int* counters, int nsplits, const float* rope_cos,
                                    const float* rope_sin, int rope_rot, cudaStream_t stream) {
  if (B <= 0 || n_layers <= 0) return OSB_OK;
  const int OD = nh * hd, NQKV = (nh + 2 * nkv) * hd;
  if (B > MAX_B || nkv <= 0 || nh % nkv != 0 || nh / nkv > 8 || !osb_decode_layers_fused_supported(H, OD, I, hd))
    return OSB_ERR_UNSUPPORTED;
  if (nsplits < 1 || rope_cos == nullptr || rope_rot <= 0 || rope_rot > hd || (rope_rot & 1)) return OSB_ERR_UNSUPPORTED;
  if ((size_t)8 * nsplits * 2 > (size_t)NCW * 16 * (hd + 8)) return OSB_ERR_TOO_LARGE;
  if ((((uintptr_t)y | (uintptr_t)res_a | (uintptr_t)res_b | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)qkv |
        (uintptr_t)attn | (uintptr_t)act | (uintptr_t)layers | (uintptr_t)rope_cos | (uintptr_t)rope_sin |
        (uintptr_t)part_o) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  LayersParams p;
  p.layers = (const LayerDesc*)layers; p.n_layers = n_layers; p.x = (const bf16*)x; p.res_in = res_in; p.res_a = res_a;
  p.res_b = res_b; p.y = (bf16*)y; p.qkv = (bf16*)qkv; p.attn = (bf16*)attn; p.act = (bf16*)act; p.bar = bar; p.err = err;
  p.B = B; p.NQKV = NQKV;
  p.t.k_cache = nullptr; p.t.v_cache = nullptr; p.t.window = 0; p.t.num_pages = 0; p.t.log2ps = 0;   // per layer
  p.t.cu_q = cu_q; p.t.seq_lens = seq_lens; p.t.decode_index = decode_index; p.t.counters = counters;
  p.t.block_table = block_table; p.t.bt_stride = bt_stride; p.t.part_o = part_o; p.t.part_ml = part_ml;
  p.t.rope.cos_t = rope_cos; p.t.rope.sin_t = rope_sin; p.t.rope.slot_map = slot_map; p.t.rope.rot = rope_rot;
  p.t.scale_log2 = scale * 1.4426950408889634f; p.t.nh = nh; p.t.nkv = nkv; p.t.nsplits = nsplits;
  typedef Geometry<16, 12, 3, 3> GeoB;
  const int n_sm = sm_count();
  if (H == 1536) return launch_fused<GeoB>(decode_layers_fused_kernel<12, 12, 70, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  if (H == 256) return launch_fused<GeoB>(decode_layers_fused_kernel<2, 2, 4, 64, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  return launch_fused<GeoB>(decode_layers_fused_kernel<3, 4, 15, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
}

OSB_API int osb_norm_linear_decode_supported(int H) { return H == 1536 || H == 256 || H == 384 || H == 2048; }

// y [B,N] = (rmsnorm(res_in + x) * norm_w) W^T + bias; res_out = res_in + x (fp32). B <= 16, everything bf16
// but the residual stream. Without norm_w (then no res_in, no res_out): y = x W^T + bias.
OSB_API int osb_norm_linear_decode(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w,
                                   float eps, const void* w, const void* bias, int* err, int B, int N, int H,
                                   cudaStream_t stream) {
  if (B <= 0 || N <= 0) return OSB_OK;
  if (B > 2 * MAX_B || !osb_norm_linear_decode_supported(H)) return OSB_ERR_UNSUPPORTED;
  if ((((uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  if (norm_w == nullptr && (res_in != nullptr || res_out != nullptr)) return OSB_ERR_BAD_SHAPE;
  NormLinearParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w; p.w = (const bf16*)w;
  p.bias = (const bf16*)bias; p.y = (bf16*)y; p.err = err; p.eps = eps; p.B = B; p.N = N;
  // little shared memory: the kernels before and after can be on the SM at the same time
  typedef Geometry<16, 12, 2, 1> GeoS;
  typedef Geometry<12, 7, 4, 3> GeoT;
  typedef Geometry<16, 8, 3, 2> GeoU;
  const int n_sm = sm_count();
  if (B > MAX_B) {   // 9 to 16 rows: two column tiles
    typedef Geometry<16, 12, 2, 1, 2> GeoS2;
    typedef Geometry<12, 7, 4, 2, 2> GeoT2;
    typedef Geometry<16, 8, 2, 2, 2> GeoU2;
    if (H == 1536) return launch_fused<GeoS2>(norm_linear_decode_kernel<12, GeoS2>, p, n_sm, false, stream);
    if (H == 256) return launch_fused<GeoS2>(norm_linear_decode_kernel<2, GeoS2>, p, n_sm, false, stream);
    if (H == 384) return launch_fused<GeoT2>(norm_linear_decode_kernel<3, GeoT2>, p, n_sm, false, stream);
    return launch_fused<GeoU2>(norm_linear_decode_kernel<16, GeoU2>, p, n_sm, false, stream);
  }
  if (H == 1536) return launch_fused<GeoS>(norm_linear_decode_kernel<12, GeoS>, p, n_sm, false, stream);
  if (H == 256) return launch_fused<GeoS>(norm_linear_decode_kernel<2, GeoS>, p, n_sm, false, stream);
  if (H == 384) return launch_fused<GeoT>(norm_linear_decode_kernel<3, GeoT>, p, n_sm, false, stream);
  return launch_fused<GeoU>(norm_linear_decode_kernel<16, GeoU>, p, n_sm, false, stream);
}

#ifdef OSB_FUSED_TIMELINE
OSB_API int osb_fused_timeline(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_fused_timeline, sizeof(long long) * (size_t)n);
}
#endif
