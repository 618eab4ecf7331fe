// Weight-streaming kernels for decode steps of a few rows: one CTA per SM, all sizes taken at run time.
//
// A decode step of a few rows is bound by reading every weight once. One warp per CTA streams the CTA's share
// of a weight matrix through a ring of shared-memory tiles with bulk asynchronous copies (L2 evict-first: the
// bytes are read once per step), stage after stage without a pause; the weights do not depend on the
// activations, so the stream starts before the kernel has waited for the kernel in front of it and runs ahead
// across the point where the CTAs wait for one another. Eight warps consume the tiles with m16n8k16 MMAs:
// weight rows on the M side, 8 batch rows per column tile on the N side (NT column tiles: up to 8 NT rows), the
// K range of a tile split over the warps and summed in a fixed order through shared memory.
//
// The rows of the activation come from one of two places. Resident: all rows whole in shared memory, after an
// RMS norm that every CTA computes for itself (or copied as they are); that needs 8 NT rows of K elements beside
// the ring. Streamed: tiles of the activation beside every weight tile, copied by a second producer warp from
// global memory, for any K; the activation must then be complete in global memory (the output of an earlier
// kernel, or of an earlier stage of this one behind a barrier of all CTAs).
//
// Kernels (K, N, H, I any multiples of 128 / any N):
//   stream_linear_kernel   y = f(x) W^T + b, f = RMS norm of (residual + x) or nothing; optionally W = [gate; up]
//                          and y = silu(gate) * up. No CTA waits for another.
//   stream_ffn_kernel      r = residual + x; h = rmsnorm(r) * w; act = silu(h Wg^T) * (h Wu^T)
//                          -- all CTAs meet --  y = act Wd^T
// Every wait is bounded and reports through the error flag instead of hanging; a CTA that gives up keeps its
// control flow (every barrier is still reached), on data that is no longer meaningful.
// Formulas: omniserve/kernels/fused_ops.py:21-29, 43-57 (add + norm), 111-119 (silu * up);
// omniserve/model/qwen2_llm.py:116-134 (feed-forward), 137-157 (the residual stream).
#include "mma_utils.cuh"
#include "tc_utils.cuh"

namespace {

constexpr int NCW = 8;               // consumer warps
constexpr int NCT = NCW * 32;        // consumer threads
constexpr int W_WARP = NCW;          // the warp that streams the weights
constexpr int A_WARP = NCW + 1;      // the warp that streams activations from global memory
constexpr int NTHREADS = NCT + 64;
constexpr int MAX_ST = 8;            // most tiles in flight per stream (the barrier arrays)
constexpr int NORM_REG_TILES = 16;   // the norm keeps a row in registers up to 16 * 128 = 2,048 elements
constexpr uint32_t GRID_WAIT_LIMIT = 1u << 21;
constexpr size_t MAX_SMEM = 232448;  // dynamic shared memory a CTA can have on sm_100

enum : int { ERR_TILE_WAIT = 131, ERR_SLOT_WAIT = 132, ERR_GRID_WAIT = 133, ERR_DRAIN = 134 };

// How the shared memory is cut: weight tiles of RS rows by at most KTW * 128 elements along K, NST of them in
// flight; activation tiles of 8 NT rows by the same length, AST in flight.
template <int RS_, int KTW_, int NST_, int AST_, int NT_>
struct Geometry {
  static constexpr int RS = RS_, PG = RS_ / 2, KTW = KTW_, NST = NST_, AST = AST_, NT = NT_;
  static constexpr int KC = KTW * NCW * 16;                // elements of K per tile
  // row stride in a tile; = 32 mod 128, so the 8-byte fragment loads of four rows fall on different banks
  static constexpr int SROW = KC * 2 + 32;
  static constexpr int SLOT = RS * SROW, ASLOT = 8 * NT * SROW;
  static constexpr int RED_FLOATS = 2 * NCW * 128 * NT;    // two buffers of every warp's accumulators
  static_assert(NST <= MAX_ST && AST <= MAX_ST && RS % 2 == 0 && RS <= 16, "");
};

struct Shared {
  uint64_t full[MAX_ST], empty[MAX_ST];
  uint64_t afull[MAX_ST], aempty[MAX_ST];
  uint64_t act_ready;      // the activation of the second stage is complete in global memory
  volatile int abort_flag;
};

// bytes of a resident activation row of K elements (= 32 mod 128 for K a multiple of 64)
__host__ __device__ constexpr size_t xs_row_bytes(int K) { return (size_t)K * 2 + 32; }

template <class Geo>
__host__ __device__ constexpr size_t region_a_bytes(int resident_k) {
  const size_t tiles = (size_t)Geo::AST * Geo::ASLOT, rows = resident_k > 0 ? 8 * Geo::NT * xs_row_bytes(resident_k) : 0;
  return tiles > rows ? tiles : rows;
}
template <class Geo>
__host__ __device__ constexpr size_t smem_bytes(int resident_k) {
  return (size_t)Geo::NST * Geo::SLOT + region_a_bytes<Geo>(resident_k) + Geo::RED_FLOATS * sizeof(float) + sizeof(Shared);
}

template <class Geo>
struct Carve {
  uint8_t *slots, *aslots, *xs;
  float* red;
  Shared* sh;
  __device__ __forceinline__ Carve(uint8_t* smem, int resident_k) {
    slots = smem;
    aslots = slots + Geo::NST * Geo::SLOT;
    xs = aslots;   // the resident rows and the activation tiles use the same bytes, at different times
    red = reinterpret_cast<float*>(aslots + region_a_bytes<Geo>(resident_k));
    sh = reinterpret_cast<Shared*>(red + Geo::RED_FLOATS);
  }
};

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(tc::smem_addr(dst)), "l"(src), "r"(bytes), "r"(tc::smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(tc::smem_addr(dst)), "l"(src), "r"(bytes), "r"(tc::smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
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

// A bounded wait on one of the CTA's barriers; the first thread that runs out of patience makes every later
// wait of the CTA return at once.
__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, Shared* sh, int* err, int code) {
  if (!tc::mbar_wait(bar, parity, (volatile int*)&sh->abort_flag) && !sh->abort_flag) {
    sh->abort_flag = 1;
    atomicExch(err, code);
  }
}

// K = kt * 128 elements are cut into pieces of at most KTW * 128: piece ch has `n` k-tiles of 16 per warp.
struct Pieces {
  int kt, nch;
  __device__ __forceinline__ Pieces(int K, int ktw) : kt(K >> 7), nch(((K >> 7) + ktw - 1) / ktw) {}
  __device__ __forceinline__ int n(int ch, int ktw) const { return min(ktw, kt - ch * ktw); }
};

// ------------------------------------------------------------------ a stream of tiles (one warp)
// Used twice: the weights (tiles of RS rows, read once: first out of the L2), and activations that are complete
// in global memory (tiles of B rows).
template <class Geo, bool WEIGHTS>
struct Streamer {
  static constexpr int NST = WEIGHTS ? Geo::NST : Geo::AST, SLOT = WEIGHTS ? Geo::SLOT : Geo::ASLOT;
  static constexpr int SROW = Geo::SROW, KTW = Geo::KTW, KC = Geo::KC;
  Shared* sh;
  uint64_t *full, *empty;
  uint8_t* slots;
  uint32_t idx;
  uint64_t policy;
  int lane;
  int* err;

  __device__ __forceinline__ Streamer(Shared* s, uint8_t* mem, int lane_, int* err_)
      : sh(s), full(WEIGHTS ? s->full : s->afull), empty(WEIGHTS ? s->empty : s->aempty), slots(mem), idx(0u),
        policy(WEIGHTS ? policy_evict_first() : 0ull), lane(lane_), err(err_) {}

  // One tile: lane l < n copies `bytes` from src(l) to row l of the next slot.
  template <class Src>
  __device__ __forceinline__ void tile(int n, uint32_t bytes, Src src) {
    const uint32_t slot = idx % NST, round = idx / NST;
    wait_or_abort(&empty[slot], (round & 1u) ^ 1u, sh, err, ERR_SLOT_WAIT);
    if (lane == 0) tc::mbar_expect_tx(&full[slot], bytes * (uint32_t)n);
    __syncwarp();
    if (lane < n) {
      void* dst = slots + (size_t)slot * SLOT + (size_t)lane * SROW;
      if constexpr (WEIGHTS) bulk_copy(dst, src(lane), bytes, &full[slot], policy);
      else bulk_copy(dst, src(lane), bytes, &full[slot]);
    }
    ++idx;
  }
  // rows [r0, r1) of W [*, K] in groups of RS rows, each group piece after piece along K
  __device__ void rows(const bf16* W, int K, int r0, int r1) {
    const Pieces pc(K, KTW);
    for (int rg = r0; rg < r1; rg += Geo::RS) {
      const int nr = min(Geo::RS, r1 - rg);
      for (int ch = 0; ch < pc.nch; ++ch)
        tile(nr, (uint32_t)pc.n(ch, KTW) * 256u, [&](int l) { return W + (size_t)(rg + l) * K + (size_t)ch * KC; });
    }
  }
  // pairs [p0, p1): row p of W [2I, K] in tile rows 0 .. PG-1 beside row I + p in tile rows PG ..
  __device__ void pairs(const bf16* W, int K, int I, int p0, int p1) {
    constexpr int PG = Geo::PG;
    const Pieces pc(K, KTW);
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      for (int ch = 0; ch < pc.nch; ++ch)
        tile(Geo::RS, (uint32_t)pc.n(ch, KTW) * 256u, [&](int l) {
          // a short last tile repeats its last pair: the rows exist and are not used
          const int q = pg + min(l < PG ? l : l - PG, np - 1);
          return W + (size_t)((l < PG ? 0 : I) + q) * K + (size_t)ch * KC;
        });
    }
  }
  // the activation x [B, K] once for every row group of a stage that has `groups` of them
  __device__ void activation(const bf16* x, int K, int B, int groups) {
    const Pieces pc(K, KTW);
    for (int gidx = 0; gidx < groups; ++gidx)
      for (int ch = 0; ch < pc.nch; ++ch)
        tile(B, (uint32_t)pc.n(ch, KTW) * 256u, [&](int l) { return x + (size_t)l * K + (size_t)ch * KC; });
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
  static constexpr int NST = Geo::NST, SROW = Geo::SROW, RS = Geo::RS, NT = Geo::NT, KTW = Geo::KTW;
  static constexpr int CH = NT == 1 ? 2 : 1;   // with one column tile: two chains of dependent MMAs instead of one
  Shared* sh;
  uint8_t* slots;
  uint8_t* aslots;
  float* red;
  uint32_t idx;    // weight tiles consumed
  uint32_t aidx;   // activation tiles consumed
  uint32_t nred;   // reductions done
  int warp, lane;
  int wk;          // which of the NCW ranges along K of a tile this warp sums: rotated from CTA to CTA
  int* err;

  // This warp's fragments of the activation for one piece of K: rows 8 nt + g of `xp` (rows `xstride` bytes apart,
  // `xp` at the piece's first element). The summation index inside a k-tile is permuted so that one 8-byte load
  // holds both halves of a fragment (the weights are read the same way). FULL: the piece has KTW k-tiles per warp
  // (no test per k-tile: a branch around every load costs more than the load).
  template <bool FULL>
  __device__ __forceinline__ void load_x_n(uint2 (&xv)[NT][KTW], int n, const uint8_t* xp, size_t xstride) const {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* x_p = xp + (size_t)g * xstride + (size_t)(wk * n * 16 + 4 * t) * 2;
#pragma unroll
    for (int j = 0; j < KTW; ++j)
      if (FULL || j < n) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xv[nt][j] = lds64(x_p + (size_t)nt * 8 * xstride + j * 32);
      }
  }
  __device__ __forceinline__ void load_x(uint2 (&xv)[NT][KTW], int n, const uint8_t* xp, size_t xstride) const {
    if (n == KTW) load_x_n<true>(xv, KTW, xp, xstride);
    else load_x_n<false>(xv, n, xp, xstride);
  }

  // acc += (tile rows) x (this warp's K range of the tile) . x. MMA row r < 8 is tile row r, MMA row 8 + r is tile
  // row HI + r (8 for plain rows, PG for pairs); rows past the tile's end read whatever the slot holds and are
  // not stored. The fragment loads of the tile (of half of it with two column tiles) are issued before the first
  // MMA (loads and MMAs are volatile asm statements, kept in program order): the MMAs wait for one round trip to
  // shared memory, not for one each.
  template <int HI, bool FULL>
  __device__ __forceinline__ void mma_tile_n(float (&acc)[NT][CH][4], int n, const uint2 (&xv)[NT][KTW], uint32_t slot) {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* base = slots + (size_t)slot * Geo::SLOT + (size_t)(wk * n * 16 + 4 * t) * 2;
    const uint8_t* lo_p = base + (size_t)g * SROW;
    const uint8_t* hi_p = base + (size_t)min(HI + g, RS - 1) * SROW;
    constexpr int LB = NT == 1 ? KTW : (KTW + 1) / 2;   // k-tiles whose loads are in flight together
#pragma unroll
    for (int j0 = 0; j0 < KTW; j0 += LB) {
      uint2 lo[LB], hi[LB];
#pragma unroll
      for (int u = 0; u < LB; ++u)
        if (j0 + u < KTW && (FULL || j0 + u < n)) {
          lo[u] = lds64(lo_p + (j0 + u) * 32);
          hi[u] = lds64(hi_p + (j0 + u) * 32);
        }
#pragma unroll
      for (int u = 0; u < LB; ++u)
        if (j0 + u < KTW && (FULL || j0 + u < n)) {
          const int j = j0 + u;
          const unsigned a[4] = {lo[u].x, hi[u].x, lo[u].y, hi[u].y};
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[nt][CH == 2 ? (j & 1) : 0], a, xv[nt][j].x, xv[nt][j].y);
        }
    }
  }
  template <int HI>
  __device__ __forceinline__ void mma_tile(float (&acc)[NT][CH][4], int n, const uint2 (&xv)[NT][KTW]) {
    const uint32_t slot = idx % NST, round = idx / NST;
    wait_or_abort(&sh->full[slot], round & 1u, sh, err, ERR_TILE_WAIT);
    if (n == KTW) mma_tile_n<HI, true>(acc, KTW, xv, slot);
    else mma_tile_n<HI, false>(acc, n, xv, slot);
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&sh->empty[slot]);
    ++idx;
  }

  // Sum of the warps' accumulators of all column tiles: thread i < 128 gets, per tile, element (MMA row i / 8,
  // batch row 8 nt + i % 8) in s, and with PAIR (i < 64) the element of MMA row + 8 in s2.
  template <bool PAIR>
  __device__ __forceinline__ void reduce(const float (&acc)[NT][CH][4], float (&s)[NT], float (&s2)[NT]) {
    float* buf = red + (nred & 1u) * (NCW * 128 * NT);
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = CH == 2 ? acc[nt][0][i] + acc[nt][CH - 1][i] : acc[nt][0][i];
      *reinterpret_cast<float2*>(buf + (nt * NCW + warp) * 128 + g * 8 + 2 * t) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2*>(buf + (nt * NCW + warp) * 128 + 64 + g * 8 + 2 * t) = make_float2(c[2], c[3]);
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

  // One group of rows (or pairs) over all pieces of K. RESIDENT: the activation's rows are whole in shared
  // memory at `xs` (rows `xstride` bytes apart); if K is one piece, this warp's fragments of it are already in
  // `xv` (loaded once for all groups). Otherwise a tile of the activation arrives beside every weight tile; its
  // fragments are taken and the tile handed back before the weight tile is waited for.
  template <int HI, bool RESIDENT>
  __device__ __forceinline__ void row_group(float (&acc)[NT][CH][4], const Pieces& pc, const uint8_t* xs, size_t xstride,
                                            uint2 (&xv)[NT][KTW]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < CH; ++c) acc[nt][c][0] = acc[nt][c][1] = acc[nt][c][2] = acc[nt][c][3] = 0.0f;
    for (int ch = 0; ch < pc.nch; ++ch) {
      const int n = pc.n(ch, KTW);
      if constexpr (RESIDENT) {
        if (pc.nch > 1) load_x(xv, n, xs + (size_t)ch * Geo::KC * 2, xstride);
      } else {
        const uint32_t slot = aidx % Geo::AST, round = aidx / Geo::AST;
        wait_or_abort(&sh->afull[slot], round & 1u, sh, err, ERR_TILE_WAIT);
        load_x(xv, n, aslots + (size_t)slot * Geo::ASLOT, SROW);
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&sh->aempty[slot]);
        ++aidx;
      }
      mma_tile<HI>(acc, n, xv);
    }
  }

  // rows [r0, r1) of a projection: epi(row, n, sum) by the thread that holds output (row, batch row n < B)
  template <bool RESIDENT, class Epi>
  __device__ __forceinline__ void rows(int K, int r0, int r1, int B, const uint8_t* xs, size_t xstride, Epi epi) {
    const Pieces pc(K, KTW);
    uint2 xv[NT][KTW];
    if (RESIDENT && pc.nch == 1) load_x(xv, pc.n(0, KTW), xs, xstride);
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float acc[NT][CH][4], s[NT], s2[NT];
      row_group<8, RESIDENT>(acc, pc, xs, xstride, xv);
      reduce<false>(acc, s, s2);
      const int i = warp * 32 + lane, row = i >> 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + (i & 7);
        if (i < 128 && row < nr && n < B) epi(rg + row, n, s[nt]);
      }
    }
  }
  // pairs [p0, p1) of a gated projection: epi(pair, n, gate sum, up sum)
  template <bool RESIDENT, class Epi>
  __device__ __forceinline__ void pairs(int K, int p0, int p1, int B, const uint8_t* xs, size_t xstride, Epi epi) {
    constexpr int PG = Geo::PG;
    const Pieces pc(K, KTW);
    uint2 xv[NT][KTW];
    if (RESIDENT && pc.nch == 1) load_x(xv, pc.n(0, KTW), xs, xstride);
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      float acc[NT][CH][4], s[NT], s2[NT];
      row_group<PG, RESIDENT>(acc, pc, xs, xstride, xv);
      reduce<true>(acc, s, s2);
      const int i = warp * 32 + lane, pair = i >> 3;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + (i & 7);
        if (i < 64 && pair < np && n < B) epi(pg + pair, n, s[nt], s2[nt]);
      }
    }
  }
};

// ------------------------------------------------------------------ all CTAs meet
// Every CTA adds one to a counter that only grows and waits until it reaches the next multiple of the number of
// CTAs. Called by one thread per CTA, between two consumer_sync(): the barrier before orders the other threads'
// stores before the release here. `expected` is the grid size (a test passes more, so that the wait must run out).
struct GridSync {
  unsigned long long* bar;
  unsigned long long target;   // kept by thread 0
  unsigned expected;
  uint32_t limit;
  Shared* sh;
  int* err;
  // after the kernel's wait for the kernel before it: no CTA passes the first barrier before this one arrives,
  // so the counter is less than a grid size past the multiple that the launch started from
  __device__ __forceinline__ void begin() {
    if (threadIdx.x == 0) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(bar) : "memory");
      target = v - v % (unsigned long long)expected;
    }
  }
  __device__ __forceinline__ void arrive(bool for_bulk_copies) {
    if (for_bulk_copies) publish_for_bulk_copies();
    consumer_sync();
    if (threadIdx.x == 0) {
      if (!sh->abort_flag) asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(bar) : "memory");
      target += (unsigned long long)expected;
    }
  }
  __device__ __forceinline__ void wait() {
    if (threadIdx.x == 0 && !sh->abort_flag) {
      bool ok = false;
      for (uint32_t i = 0; i < limit && !ok; ++i) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(bar) : "memory");
        ok = v >= target;
      }
      if (!ok) {
        sh->abort_flag = 1;
        atomicExch(err, ERR_GRID_WAIT);
      }
    }
    consumer_sync();
  }
};

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

// ------------------------------------------------------------------ the resident rows
__device__ __forceinline__ void unpack4(const uint2 v, float (&f)[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// r = residual + x (fp32), h = rmsnorm(r) * w rounded to bf16 into the resident rows (xs, rows of XS bytes):
// consumer warp n does batch rows n, n + 8, ... (rows from B on are zeros). CTA 0 also writes r to res_out.
// `wait_pdl`: this is the kernel's first use of anything the kernel before it wrote; for rows of up to 2,048
// elements the norm's weights are fetched before that wait and the row stays in registers, longer rows are
// read a second time (from the L2). Loads are issued in groups before anything waits for one of them (a lane's
// loads stand in loops of their own, apart from the arithmetic that waits for them): the norm costs a few round
// trips to the L2, not one per 128 elements.
template <int NT>
__device__ __forceinline__ void norm_rows(const bf16* x, const float* res_in, float* res_out, const bf16* norm_w,
                                          float eps, int B, int K, uint8_t* xs, int warp, int lane, bool wait_pdl) {
  const size_t XS = xs_row_bytes(K);
  const int tiles = K >> 7;   // 128 elements: 4 per lane
  const bool write_res = blockIdx.x == 0 && res_out != nullptr;
  if (tiles <= NORM_REG_TILES) {
    uint2 nw[NORM_REG_TILES];
#pragma unroll
    for (int i = 0; i < NORM_REG_TILES; ++i)
      if (i < tiles) nw[i] = *reinterpret_cast<const uint2*>(norm_w + (i * 32 + lane) * 4);
    if (wait_pdl) pdl_wait();
#pragma unroll 1
    for (int nt = 0; nt < NT; ++nt) {
      const int n = nt * 8 + warp;
      uint8_t* xrow = xs + (size_t)n * XS;
      if (n < B) {
        uint2 xr[NORM_REG_TILES];
        float4 rr[NORM_REG_TILES];
#pragma unroll
        for (int i = 0; i < NORM_REG_TILES; ++i)   // nothing but loads here: they are all in flight together
          if (i < tiles) xr[i] = __ldcg(reinterpret_cast<const uint2*>(x + (size_t)n * K + (i * 32 + lane) * 4));
        if (res_in) {
#pragma unroll
          for (int i = 0; i < NORM_REG_TILES; ++i)
            if (i < tiles) rr[i] = __ldcg(reinterpret_cast<const float4*>(res_in + (size_t)n * K + (i * 32 + lane) * 4));
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NORM_REG_TILES; ++i) {   // rr[i] becomes the sum
          if (i < tiles) {
            float v[4];
            unpack4(xr[i], v);
            if (res_in) rr[i] = make_float4(rr[i].x + v[0], rr[i].y + v[1], rr[i].z + v[2], rr[i].w + v[3]);
            else rr[i] = make_float4(v[0], v[1], v[2], v[3]);
            ss += rr[i].x * rr[i].x + rr[i].y * rr[i].y + rr[i].z * rr[i].z + rr[i].w * rr[i].w;
          }
        }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
        for (int i = 0; i < NORM_REG_TILES; ++i) {
          if (i < tiles) {
            const int e = (i * 32 + lane) * 4;
            if (write_res) *reinterpret_cast<float4*>(res_out + (size_t)n * K + e) = rr[i];
            float w[4];
            unpack4(nw[i], w);
            uint2 o;
            o.x = pack_bf16(rr[i].x * rstd * w[0], rr[i].y * rstd * w[1]);
            o.y = pack_bf16(rr[i].z * rstd * w[2], rr[i].w * rstd * w[3]);
            *reinterpret_cast<uint2*>(xrow + e * 2) = o;
          }
        }
      } else {
        for (int i = 0; i < tiles; ++i) *reinterpret_cast<uint2*>(xrow + (i * 32 + lane) * 8) = make_uint2(0u, 0u);
      }
    }
    return;
  }
  // long rows: two passes over the row in groups of eight tiles
  constexpr int GRP = 8;
  if (wait_pdl) pdl_wait();
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + warp;
    uint8_t* xrow = xs + (size_t)n * XS;
    if (n >= B) {
      for (int i = 0; i < tiles; ++i) *reinterpret_cast<uint2*>(xrow + (i * 32 + lane) * 8) = make_uint2(0u, 0u);
      continue;
    }
    float ss = 0.0f, rstd = 0.0f;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
#pragma unroll 1
      for (int i0 = 0; i0 < tiles; i0 += GRP) {
        uint2 xr[GRP], wv[GRP];
        float4 rr[GRP];
#pragma unroll
        for (int u = 0; u < GRP; ++u) xr[u] = __ldcg(reinterpret_cast<const uint2*>(x + (size_t)n * K + (min(i0 + u, tiles - 1) * 32 + lane) * 4));
        if (res_in) {
#pragma unroll
          for (int u = 0; u < GRP; ++u)
            rr[u] = __ldcg(reinterpret_cast<const float4*>(res_in + (size_t)n * K + (min(i0 + u, tiles - 1) * 32 + lane) * 4));
        }
        if (pass == 1) {
#pragma unroll
          for (int u = 0; u < GRP; ++u) wv[u] = *reinterpret_cast<const uint2*>(norm_w + (min(i0 + u, tiles - 1) * 32 + lane) * 4);
        }
#pragma unroll
        for (int u = 0; u < GRP; ++u) {
          if (i0 + u < tiles) {
            const int e = ((i0 + u) * 32 + lane) * 4;
            float r[4];
            unpack4(xr[u], r);
            if (res_in) { r[0] += rr[u].x; r[1] += rr[u].y; r[2] += rr[u].z; r[3] += rr[u].w; }
            if (pass == 0) {
              if (write_res) *reinterpret_cast<float4*>(res_out + (size_t)n * K + e) = make_float4(r[0], r[1], r[2], r[3]);
#pragma unroll
              for (int j = 0; j < 4; ++j) ss += r[j] * r[j];
            } else {
              float w[4];
              unpack4(wv[u], w);
              uint2 o;
              o.x = pack_bf16(r[0] * rstd * w[0], r[1] * rstd * w[1]);
              o.y = pack_bf16(r[2] * rstd * w[2], r[3] * rstd * w[3]);
              *reinterpret_cast<uint2*>(xrow + e * 2) = o;
            }
          }
        }
      }
      if (pass == 0) {
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)K + eps);
      }
    }
  }
}

// the rows of x as they are into the resident rows (no norm in front); loads in groups of eight, as above
template <int NT>
__device__ __forceinline__ void copy_rows(const bf16* x, int B, int K, uint8_t* xs, int warp, int lane) {
  const size_t XS = xs_row_bytes(K);
  const int vecs = K >> 3;   // 16 bytes each; a multiple of 16 (K is a multiple of 128)
  constexpr int GRP = 8;
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + warp;
    uint8_t* xrow = xs + (size_t)n * XS;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)min(n, B - 1) * K);
#pragma unroll 1
    for (int i0 = lane; i0 < vecs; i0 += 32 * GRP) {
      uint4 v[GRP];
#pragma unroll
      for (int u = 0; u < GRP; ++u) v[u] = __ldcg(src + min(i0 + 32 * u, vecs - 1));
#pragma unroll
      for (int u = 0; u < GRP; ++u) {
        const int i = i0 + 32 * u;
        // rows are 32 bytes past a multiple of 128: 16-byte stores stay aligned
        if (i < vecs) *reinterpret_cast<uint4*>(xrow + (size_t)i * 16) = n < B ? v[u] : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return (gate / (1.0f + expf(-gate))) * up; }

// ------------------------------------------------------------------ kernels
struct LinearParams {
  const bf16* x;        // [B, K]
  const float* res_in;  // [B, K] or null
  float* res_out;       // [B, K] or null (with norm_w: res_in + x)
  const bf16* norm_w;   // [K], or null: no norm (then no res_in, no res_out)
  const bf16* w;        // [N, K]; gated: [2 N, K], gate rows first
  const bf16* bias;     // [N] or null (not with gated)
  bf16* y;              // [B, N]
  int* err;
  float eps;
  int B, N, K;
};

// y = f(x) W^T + bias for a few rows; GATED: y = silu(f(x) Wg^T) * (f(x) Wu^T). RESIDENT: f(x) whole in shared memory
// (normalised by every CTA itself while its rows of W are already on their way); otherwise x is streamed in tiles
// and there is no norm. No CTA waits for another.
template <class Geo, bool GATED, bool RESIDENT>
__global__ void __launch_bounds__(NTHREADS, 1) stream_linear_kernel(const __grid_constant__ LinearParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem, RESIDENT ? p.K : 0);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int r0, r1;
  cta_rows(p.N, cta, G, r0, r1);
  constexpr int GROUP = GATED ? Geo::PG : Geo::RS;

  if (warp == W_WARP) {
    // the weights depend on nothing that runs before this kernel: the stream starts at once
    Streamer<Geo, true> ws(sh, m.slots, lane, p.err);
    if (GATED) ws.pairs(p.w, p.K, p.N, r0, r1);
    else ws.rows(p.w, p.K, r0, r1);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  if (warp == A_WARP) {
    if (!RESIDENT) {
      Streamer<Geo, false> as(sh, m.aslots, lane, p.err);
      pdl_wait();   // x is what the kernel before this one wrote
      as.activation(p.x, p.K, p.B, (r1 - r0 + GROUP - 1) / GROUP);
      __syncthreads();
      if (sh->abort_flag) as.drain();
    } else {
      __syncthreads();
    }
    return;
  }
  Consumer<Geo> co{sh, m.slots, m.aslots, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  const size_t XS = xs_row_bytes(p.K);
  if (RESIDENT) {
    if (p.norm_w != nullptr) {
      norm_rows<Geo::NT>(p.x, p.res_in, p.res_out, p.norm_w, p.eps, p.B, p.K, m.xs, warp, lane, true);
    } else {
      pdl_wait();
      copy_rows<Geo::NT>(p.x, p.B, p.K, m.xs, warp, lane);
    }
    consumer_sync();
  } else {
    pdl_wait();
  }
  pdl_trigger();
  if constexpr (GATED) {
    co.template pairs<RESIDENT>(p.K, r0, r1, p.B, m.xs, XS, [&](int pair, int n, float gate, float up) {
      p.y[(size_t)n * p.N + pair] = __float2bfloat16_rn(silu_mul(gate, up));
    });
  } else {
    co.template rows<RESIDENT>(p.K, r0, r1, p.B, m.xs, XS, [&](int row, int n, float s) {
      if (p.bias) s += __bfloat162float(p.bias[row]);
      p.y[(size_t)n * p.N + row] = __float2bfloat16_rn(s);
    });
  }
  __syncthreads();
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
  uint32_t wait_limit;    // polls of the counter before a CTA gives up at the barrier
  unsigned bar_extra;     // arrivals the barrier expects beyond the grid's (0; a test makes the wait run out with 1)
};

// The feed-forward half as one kernel: r = res_in + x; h = rmsnorm(r) * w; act = silu(h Wg^T) * (h Wu^T) -- all CTAs
// meet -- y = act Wd^T. The rows of Wd are on their way into shared memory while the CTAs wait for one another.
template <class Geo>
__global__ void __launch_bounds__(NTHREADS, 1) stream_ffn_kernel(const __grid_constant__ FfnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const Carve<Geo> m(smem, p.H);
  Shared* sh = m.sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int p0, p1, r0, r1;
  cta_rows(p.I, cta, G, p0, p1);
  cta_rows(p.H, cta, G, r0, r1);

  if (warp == W_WARP) {
    Streamer<Geo, true> ws(sh, m.slots, lane, p.err);
    ws.pairs(p.w_gate_up, p.H, p.I, p0, p1);
    ws.rows(p.w_down, p.I, r0, r1);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  if (warp == A_WARP) {
    Streamer<Geo, false> as(sh, m.aslots, lane, p.err);
    wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
    as.activation(p.act, p.I, p.B, (r1 - r0 + Geo::RS - 1) / Geo::RS);
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  Consumer<Geo> co{sh, m.slots, m.aslots, m.red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  GridSync gs{p.bar, 0ull, (unsigned)G + p.bar_extra, p.wait_limit, sh, p.err};
  norm_rows<Geo::NT>(p.x, p.res_in, p.res_out, p.norm_w, p.eps, p.B, p.H, m.xs, warp, lane, true);
  consumer_sync();
  gs.begin();
  co.template pairs<true>(p.H, p0, p1, p.B, m.xs, xs_row_bytes(p.H), [&](int pair, int n, float gate, float up) {
    p.act[(size_t)n * p.I + pair] = __float2bfloat16_rn(silu_mul(gate, up));
  });
  // also: every warp is done with the resident rows, whose memory the activation tiles use next
  gs.arrive(true);
  gs.wait();
  pdl_trigger();
  if (warp == 0 && lane == 0) tc::mbar_arrive(&sh->act_ready);
  co.template rows<false>(p.I, r0, r1, p.B, nullptr, 0, [&](int row, int n, float s) {
    p.y[(size_t)n * p.H + row] = __float2bfloat16_rn(s);
  });
  __syncthreads();
}

// ------------------------------------------------------------------ host
int& stream_with_pdl() {
  static int v = 1;
  return v;
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

// One CTA per SM. `cooperative`: the CTAs wait for one another, so the launch must fail rather than start a part
// of them.
template <class Params>
int launch_stream(void (*kernel)(Params), const Params& p, size_t smem, bool cooperative, cudaStream_t stream) {
  if (smem > MAX_SMEM) return OSB_ERR_TOO_LARGE;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int& with_pdl = stream_with_pdl();
  for (;;) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cooperative) {
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

// Geometries. Tiles of 16 rows by 1,536 elements (3 KB a row) stream best; little shared memory for the plain
// projection, so that the kernels before and after it can be on the SM at the same time; a shorter tile where
// the resident rows of a wide model need the room.
typedef Geometry<16, 12, 2, 1, 1> LinS;     // projection, rows resident, up to 8 rows
typedef Geometry<16, 12, 2, 1, 2> LinS2;    //   9 to 16 rows
typedef Geometry<16, 8, 2, 1, 1> LinW;      //   wide rows (K up to 8,192 at 8 rows)
typedef Geometry<16, 8, 2, 1, 2> LinW2;
typedef Geometry<16, 12, 2, 2, 1> LinT;     // projection, rows streamed in tiles (any K)
typedef Geometry<16, 12, 2, 2, 2> LinT2;
typedef Geometry<16, 12, 3, 3, 1> FfnB;     // feed-forward half, up to 8 rows
typedef Geometry<16, 12, 2, 2, 2> FfnB2;    //   9 to 16 rows
typedef Geometry<16, 6, 3, 2, 1> FfnW;      //   wide rows (H up to 8,192 at 8 rows)
typedef Geometry<16, 8, 2, 2, 2> FfnW2;

template <class Geo, bool GATED, bool RESIDENT>
int launch_linear(const LinearParams& p, cudaStream_t stream) {
  return launch_stream(stream_linear_kernel<Geo, GATED, RESIDENT>, p, smem_bytes<Geo>(RESIDENT ? p.K : 0), false, stream);
}

// which form a projection of B rows over K elements takes: 0 none, 1 rows resident (long tiles), 2 rows resident
// (short tiles: the rows of a wide model need the room), 3 rows streamed. Without a norm, streamed rows beside long
// tiles are faster than resident rows beside short tiles (measured at K = 8,960: 7.7 against 10.1 us).
int linear_form(int B, int K, bool needs_norm) {
  if (B <= 0 || B > 16 || K <= 0 || (K & 127)) return 0;
  const bool two = B > 8;
  if ((two ? smem_bytes<LinS2>(K) : smem_bytes<LinS>(K)) <= MAX_SMEM) return 1;
  if (!needs_norm) return 3;
  if ((two ? smem_bytes<LinW2>(K) : smem_bytes<LinW>(K)) <= MAX_SMEM) return 2;
  return 0;
}

int ffn_form(int B, int H, int I) {
  if (B <= 0 || B > 16 || H <= 0 || I <= 0 || (H & 127) || (I & 127)) return 0;
  if (B <= 8) {
    if (smem_bytes<FfnB>(H) <= MAX_SMEM) return 1;
    if (smem_bytes<FfnW>(H) <= MAX_SMEM) return 2;
  } else {
    if (smem_bytes<FfnB2>(H) <= MAX_SMEM) return 1;
    if (smem_bytes<FfnW2>(H) <= MAX_SMEM) return 2;
  }
  return 0;
}

}  // namespace

// 1 when osb_stream_linear takes B rows over K elements (with_norm: with the RMS norm in front). The rule: B <= 16,
// K a multiple of 128 and, with a norm, 8 (or 16) rows of K elements fit in shared memory beside the tiles.
OSB_API int osb_stream_linear_supported(int B, int K, int with_norm) { return linear_form(B, K, with_norm != 0) != 0; }

// y [B,N] = (rmsnorm(res_in + x) * norm_w) W^T + bias; res_out = res_in + x (fp32). B <= 16, everything bf16 but
// the residual stream. Without norm_w (then no res_in, no res_out): y = x W^T + bias. gated != 0: W is [2N, K] with
// the gate rows first, no bias, and y [B,N] = silu(h Wg^T) * (h Wu^T).
OSB_API int osb_stream_linear(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w, float eps,
                              const void* w, const void* bias, int* err, int B, int N, int K, int gated,
                              cudaStream_t stream) {
  if (B <= 0 || N <= 0) return OSB_OK;
  const int form = linear_form(B, K, norm_w != nullptr);
  if (form == 0) return OSB_ERR_UNSUPPORTED;
  if ((((uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  if (norm_w == nullptr && (res_in != nullptr || res_out != nullptr)) return OSB_ERR_BAD_SHAPE;
  if (gated && bias != nullptr) return OSB_ERR_BAD_SHAPE;
  LinearParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w; p.w = (const bf16*)w;
  p.bias = (const bf16*)bias; p.y = (bf16*)y; p.err = err; p.eps = eps; p.B = B; p.N = N; p.K = K;
  const bool two = B > 8;
#define OSB_LIN(G1, G2, RES)                                                                          \
  return gated ? (two ? launch_linear<G2, true, RES>(p, stream) : launch_linear<G1, true, RES>(p, stream)) \
               : (two ? launch_linear<G2, false, RES>(p, stream) : launch_linear<G1, false, RES>(p, stream))
  if (form == 1) { OSB_LIN(LinS, LinS2, true); }
  if (form == 2) { OSB_LIN(LinW, LinW2, true); }
  OSB_LIN(LinT, LinT2, false);
#undef OSB_LIN
}

// 1 when osb_stream_ffn takes these sizes: B <= 16, H and I multiples of 128, 8 (or 16) rows of H elements fit in
// shared memory beside the tiles.
OSB_API int osb_stream_ffn_supported(int B, int H, int I) { return ffn_form(B, H, I) != 0; }

// y [B,H] = down(silu(gate(h)) * up(h)), h = rmsnorm(res_in + x) * norm_w; res_out = res_in + x (fp32).
// bf16 weights and activations. `act` [B,I] is scratch; `bar` is a zeroed 64-bit counter that belongs to these
// launches alone (between launches it is a multiple of the number of SMs); `err` is the device error flag.
// wait_limit / bar_extra: 0 / 0 but in the test of the barrier's give-up path (see FfnParams).
OSB_API int osb_stream_ffn(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w, float eps,
                           const void* w_gate_up, const void* w_down, void* act, unsigned long long* bar, int* err,
                           int B, int H, int I, unsigned wait_limit, unsigned bar_extra, cudaStream_t stream) {
  if (B <= 0) return OSB_OK;
  const int form = ffn_form(B, H, I);
  if (form == 0) return OSB_ERR_UNSUPPORTED;
  if ((((uintptr_t)y | (uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w_gate_up |
        (uintptr_t)w_down | (uintptr_t)act) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  FfnParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w;
  p.w_gate_up = (const bf16*)w_gate_up; p.w_down = (const bf16*)w_down; p.act = (bf16*)act; p.y = (bf16*)y;
  p.bar = bar; p.err = err; p.eps = eps; p.B = B; p.H = H; p.I = I;
  p.wait_limit = wait_limit ? wait_limit : GRID_WAIT_LIMIT;
  p.bar_extra = bar_extra;
  if (B > 8) {
    if (form == 1) return launch_stream(stream_ffn_kernel<FfnB2>, p, smem_bytes<FfnB2>(H), true, stream);
    return launch_stream(stream_ffn_kernel<FfnW2>, p, smem_bytes<FfnW2>(H), true, stream);
  }
  if (form == 1) return launch_stream(stream_ffn_kernel<FfnB>, p, smem_bytes<FfnB>(H), true, stream);
  return launch_stream(stream_ffn_kernel<FfnW>, p, smem_bytes<FfnW>(H), true, stream);
}
