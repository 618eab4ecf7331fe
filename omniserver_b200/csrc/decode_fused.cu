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
template <int RS_, int MAX_KTW_, int NST_, int AST_>
struct Geometry {
  static constexpr int RS = RS_, PG = RS_ / 2, MAX_KTW = MAX_KTW_, NST = NST_, AST = AST_;
  static constexpr int MAX_KC = MAX_KTW * NCW * 16;
  // row stride in a tile; = 32 mod 128, so the 8-byte fragment loads of four rows fall on different banks
  static constexpr int SROW = MAX_KC * 2 + 32;
  static constexpr int SLOT = RS * SROW, ASLOT = 8 * SROW;
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

template <int HT, int IT, class Geo>
__global__ void __launch_bounds__(NTHREADS_ACT, 1) ffn_decode_fused_kernel(const __grid_constant__ FfnParams p) {
  constexpr int H = HT * NCW * 16, I = IT * NCW * 16;
  constexpr int NSTAGE = Geo::NST, ASTAGE = Geo::AST, RS = Geo::RS, PG = Geo::PG, MAX_KTW = Geo::MAX_KTW;
  constexpr int SLOT_BYTES = Geo::SLOT, ASLOT_BYTES = Geo::ASLOT;
  typedef Streamer<Geo::NST, Geo::SLOT, Geo::SROW, Geo::RS, true> WeightStream;
  typedef Streamer<Geo::AST, Geo::ASLOT, Geo::SROW, Geo::RS, false> ActStream;
  constexpr int KTW_H = largest_divisor_le(HT, MAX_KTW), NCH_H = HT / KTW_H, KC_H = KTW_H * NCW * 16;
  constexpr int KTW_I = largest_divisor_le(IT, MAX_KTW), NCH_I = IT / KTW_I, KC_I = KTW_I * NCW * 16;
  constexpr int XS = H * 2 + 32;  // row stride of the normalised rows in shared memory
  static_assert(MAX_B * XS <= ASTAGE * ASLOT_BYTES, "the normalised rows share the activation tiles' memory");

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* slots = smem;
  uint8_t* aslots = slots + NSTAGE * SLOT_BYTES;
  uint8_t* xs = aslots;  // used before the first activation tile is asked for
  float* red = reinterpret_cast<float*>(aslots + ASTAGE * ASLOT_BYTES);
  Shared* sh = reinterpret_cast<Shared*>(red + 2 * NCW * 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);

  int p0, p1, r0, r1;
  cta_rows(I, cta, G, p0, p1);
  cta_rows(H, cta, G, r0, r1);

  if (warp == W_WARP) {
    // the weights depend on nothing that runs before this kernel: the stream starts at once
    WeightStream ws{sh, sh->full, sh->empty, slots, 0u, policy_evict_first(), lane, p.err};
    FTL(10);
    ws.pairs(p.w_gate_up, H, I, p0, p1, NCH_H, KC_H);
    FTL(11);
    ws.rows(p.w_down, I, r0, r1, NCH_I, KC_I);
    FTL(12);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  if (warp == A_WARP) {
    ActStream as{sh, sh->afull, sh->aempty, aslots, 0u, 0ull, lane, p.err};
    wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
    as.activation(p.act, I, p.B, (r1 - r0 + RS - 1) / RS, NCH_I, KC_I);
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  Consumer<Geo> co{sh, slots, aslots, red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  unsigned long long target = 0;
  FTL(0);
  // the norm's weights do not depend on the kernel before: fetch them while it finishes
  uint2 nw[HT];
#pragma unroll
  for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(p.norm_w + (i * 32 + lane) * 4);
  pdl_wait();
  FTL(1);
  if (threadIdx.x == 0) {
    // no CTA passes the first barrier before this one arrives: the counter is less than a grid size past
    // the multiple that the launch started from
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.bar) : "memory");
    target = v - v % (unsigned long long)G + (unsigned long long)G;
  }

  norm_rows<HT>(p.x, p.res_in, cta == 0 ? p.res_out : nullptr, nw, p.eps, p.B, xs, warp, lane);
  consumer_sync();
  FTL(2);

  // ---- act = silu(h Wg^T) * (h Wu^T)
  {
    uint32_t xf[HT][2];
    load_local_x<HT, KTW_H, NCH_H>(xf, xs, co.wk, lane);
    for (int pg = p0; pg < p1; pg += PG) {
      const int np = min(PG, p1 - pg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      co.template row_group_local<KTW_H, NCH_H, PG>(c, xf);
      if (pg == p0) FTL(3);
      float up;
      const float gate = co.reduce(c, &up);
      const int i = warp * 32 + lane;
      const int pair = i >> 3, n = i & 7;
      if (i < 64 && pair < np && n < p.B)
        p.act[(size_t)n * I + pg + pair] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
    }
  }
  FTL(4);
  publish_for_bulk_copies();
  consumer_sync();   // also: every warp has its fragments out of xs, whose memory the activation tiles use next
  FTL(5);
  if (threadIdx.x == 0) grid_barrier(p.bar, target, sh, p.err);
  consumer_sync();
  FTL(6);
  pdl_trigger();
  co.act_begin();

  // ---- y = act Wd^T
  for (int rg = r0; rg < r1; rg += RS) {
    const int nr = min(RS, r1 - rg);
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    FTL(7);
    co.template row_group_streamed<KTW_I, NCH_I, 8>(c);
    FTL(8);
    const float s = co.reduce(c, nullptr);
    const int i = warp * 32 + lane;
    const int row = i >> 3, n = i & 7;
    if (i < 128 && row < nr && n < p.B) p.y[(size_t)n * H + rg + row] = __float2bfloat16_rn(s);
  }
  FTL(9);
  __syncthreads();
}


struct NormLinearParams {
  const bf16* x;        // [B, H] branch output of the part before
  const float* res_in;  // [B, H] or null
  float* res_out;       // [B, H]
  const bf16* norm_w;   // [H]
  const bf16* w;        // [N, H]
  const bf16* bias;     // [N] or null
  bf16* y;              // [B, N]
  int* err;
  float eps;
  int B, N;
};

// y = (rmsnorm(res_in + x) * norm_w) W^T + bias for a few rows: every CTA normalises the rows itself while
// its rows of W are already on their way; no CTA waits for another.
template <int HT, class Geo>
__global__ void __launch_bounds__(NTHREADS, 1) norm_linear_decode_kernel(const __grid_constant__ NormLinearParams p) {
  constexpr int H = HT * NCW * 16;
  constexpr int KTW = largest_divisor_le(HT, Geo::MAX_KTW), NCH = HT / KTW, KC = KTW * NCW * 16;
  constexpr int RS = Geo::RS;
  typedef Streamer<Geo::NST, Geo::SLOT, Geo::SROW, Geo::RS, true> WeightStream;
  typedef Streamer<Geo::AST, Geo::ASLOT, Geo::SROW, Geo::RS, false> ActStream;
  static_assert(MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows use the activation tiles' memory");

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* slots = smem;
  uint8_t* xs = slots + Geo::NST * Geo::SLOT;
  float* red = reinterpret_cast<float*>(xs + Geo::AST * Geo::ASLOT);
  Shared* sh = reinterpret_cast<Shared*>(red + 2 * NCW * 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);
  int r0, r1;
  cta_rows(p.N, cta, G, r0, r1);

  if (warp == W_WARP) {
    WeightStream ws{sh, sh->full, sh->empty, slots, 0u, policy_evict_first(), lane, p.err};
    ws.rows(p.w, H, r0, r1, NCH, KC);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }
  Consumer<Geo> co{sh, slots, xs, red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  uint32_t xf[HT][2];
  if (p.norm_w != nullptr) {
    uint2 nw[HT];
#pragma unroll
    for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(p.norm_w + (i * 32 + lane) * 4);
    pdl_wait();
    norm_rows<HT>(p.x, p.res_in, cta == 0 ? p.res_out : nullptr, nw, p.eps, p.B, xs, warp, lane);
    consumer_sync();
    load_local_x<HT, KTW, NCH>(xf, xs, co.wk, lane);
  } else {
    // no norm in front: the rows' fragments come straight from global memory
    pdl_wait();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
      for (int j = 0; j < KTW; ++j) {
        const int k0 = ch * KC + (co.wk * KTW + j) * 16 + 4 * t;
        uint2 v = make_uint2(0u, 0u);
        if (g < p.B) v = __ldcg(reinterpret_cast<const uint2*>(p.x + (size_t)g * H + k0));
        xf[ch * KTW + j][0] = v.x;
        xf[ch * KTW + j][1] = v.y;
      }
  }
  pdl_trigger();
  for (int rg = r0; rg < r1; rg += RS) {
    const int nr = min(RS, r1 - rg);
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    co.template row_group_local<KTW, NCH, 8>(c, xf);
    float s = co.reduce(c, nullptr);
    const int i = warp * 32 + lane;
    const int row = i >> 3, n = i & 7;
    if (i < 128 && row < nr && n < p.B) {
      if (p.bias) s += __bfloat162float(p.bias[rg + row]);
      p.y[(size_t)n * p.N + rg + row] = __float2bfloat16_rn(s);
    }
  }
  __syncthreads();
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
  // the cache and the step's tables, as osb_attn_decode_stream takes them
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

// The attention half of a layer for a decode step of up to 8 requests:
//   r = residual + x; h = rmsnorm(r) * w; qkv = h Wqkv^T + b     (rows of Wqkv split over the CTAs)
//   -- grid barrier --
//   rotary encoding, the new key and value into the cache, attention over the cache: one
//   (request, kv head, split of the keys) per CTA and turn, as attn_decode_stream_kernel does it; the CTA
//   that finishes a (request, kv head) last merges its splits
//   -- grid barrier --
//   y = attn Wo^T                                                 (rows of Wo split over the CTAs)
// The rows of Wo are on their way into shared memory while the attention runs.
// Formulas: omniserve/model/qwen2_llm.py:75-113.
template <int HT, int OT, int HD, class Geo>
__global__ void __launch_bounds__(NTHREADS_WIDE, 1) attn_decode_fused_kernel(const __grid_constant__ AttnHalfParams p) {
  constexpr int H = HT * NCW * 16, OD = OT * NCW * 16;
  constexpr int RS = Geo::RS, MAX_KTW = Geo::MAX_KTW;
  typedef Streamer<Geo::NST, Geo::SLOT, Geo::SROW, Geo::RS, true> WeightStream;
  typedef Streamer<Geo::AST, Geo::ASLOT, Geo::SROW, Geo::RS, false> ActStream;
  constexpr int KTW_H = largest_divisor_le(HT, MAX_KTW), NCH_H = HT / KTW_H, KC_H = KTW_H * NCW * 16;
  constexpr int KTW_O = largest_divisor_le(OT, MAX_KTW), NCH_O = OT / KTW_O, KC_O = KTW_O * NCW * 16;
  static_assert(MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows share the activation tiles' memory");
  // the attention's q rows, per-warp (max, sum) and outputs use the activation tiles and the reduction buffers
  static_assert(16 * (HD + 8) * 2 + NCW * 16 * 2 * 4 + 16 * 2 * 4 + NCW * 16 * (HD + 8) * 4 <=
                    Geo::AST * Geo::ASLOT + 2 * NCW * 128 * 4, "the attention's scratch does not fit");

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* slots = smem;
  uint8_t* aslots = slots + Geo::NST * Geo::SLOT;
  uint8_t* xs = aslots;
  float* red = reinterpret_cast<float*>(aslots + Geo::AST * Geo::ASLOT);
  Shared* sh = reinterpret_cast<Shared*>(red + 2 * NCW * 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  init_shared<Geo>(sh);

  int q0, q1, r0, r1;
  cta_rows(p.NQKV, cta, G, q0, q1);
  cta_rows(H, cta, G, r0, r1);

  if (warp >= W_WARP) reg_give<PRODUCER_REGS>();   // all four warps of the last warp group, at one place
  if (warp > A_WARP) return;
  if (warp == A_WARP) {
    ActStream as{sh, sh->afull, sh->aempty, aslots, 0u, 0ull, lane, p.err};
    wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
    as.activation(p.attn, OD, p.B, (r1 - r0 + RS - 1) / RS, NCH_O, KC_O);
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  if (warp == W_WARP) {
    WeightStream ws{sh, sh->full, sh->empty, slots, 0u, policy_evict_first(), lane, p.err};
    FTL(10);
    ws.rows(p.w_qkv, H, q0, q1, NCH_H, KC_H);
    FTL(11);
    ws.rows(p.w_o, OD, r0, r1, NCH_O, KC_O);
    FTL(12);
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }

  reg_take<CONSUMER_REGS>();
  Consumer<Geo> co{sh, slots, aslots, red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  unsigned long long target = 0;
  uint2 nw[HT];
#pragma unroll
  for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(p.norm_w + (i * 32 + lane) * 4);
  FTL(0);
  // this CTA's first (request, kv head, split): its old keys and values depend on nothing in this step
  const int grp = p.nh / p.nkv;
  const int ny = p.nkv * ((grp + 7) >> 3);
  const int units = p.B * ny * p.nsplits;
  if (cta < units) {
    const int rest = cta / p.nsplits;
    attn_stream::attn_stream_prefetch<HD>(cta % p.nsplits, rest % ny, rest / ny, p.k_cache, p.v_cache, p.block_table,
                                          p.bt_stride, p.seq_lens, p.nh, p.nkv, p.log2ps, p.num_pages, p.window,
                                          p.nsplits);
  }
  pdl_wait();
  FTL(1);
  if (threadIdx.x == 0) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.bar) : "memory");
    target = v - v % (unsigned long long)G + (unsigned long long)G;
  }
  norm_rows<HT>(p.x, p.res_in, cta == 0 ? p.res_out : nullptr, nw, p.eps, p.B, xs, warp, lane);
  consumer_sync();
  FTL(2);

  // ---- qkv = h Wqkv^T + b
  {
    uint32_t xf[HT][2];
    load_local_x<HT, KTW_H, NCH_H>(xf, xs, co.wk, lane);
    for (int rg = q0; rg < q1; rg += RS) {
      const int nr = min(RS, q1 - rg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      co.template row_group_local<KTW_H, NCH_H, 8>(c, xf);
      float s = co.reduce(c, nullptr);
      const int i = warp * 32 + lane;
      const int row = i >> 3, n = i & 7;
      if (i < 128 && row < nr && n < p.B) {
        if (p.b_qkv) s += __bfloat162float(p.b_qkv[rg + row]);
        p.qkv[(size_t)n * p.NQKV + rg + row] = __float2bfloat16_rn(s);
      }
    }
  }
  FTL(3);
  consumer_sync();
  if (threadIdx.x == 0) grid_arrive(p.bar, sh);
  // the first unit looks up its pages and starts its first loads before it waits for the other CTAs' q, k, v
  bool waited = false;
  auto wait_qkv = [&] {
    if (!waited) {
      if (threadIdx.x == 0) grid_wait(p.bar, target, sh, p.err);
      consumer_sync();
      waited = true;
      FTL(4);
    }
  };

  // ---- attention: units (request, kv head, split), one per CTA and turn
  {
    for (int u = cta; u < units; u += G) {
      const int split = u % p.nsplits, rest = u / p.nsplits;
      const int by = rest % ny, s = rest / ny;
      attn_stream::attn_stream_unit<HD, false, true>(
          wait_qkv, split, by, s, ny, aslots, &sh->s_last, p.attn, p.part_o, p.part_ml, p.qkv, p.NQKV, p.k_cache, p.v_cache,
          p.block_table, p.bt_stride, p.cu_q, p.seq_lens, p.decode_index, p.counters, p.nh, p.nkv, p.log2ps,
          p.num_pages, p.scale_log2, p.window, 0, p.nsplits, p.rope);
      wait_qkv();        // a unit that has nothing to do returns before it waits
      consumer_sync();   // the scratch in shared memory is used again by the next unit and by the tiles after it
    }
    wait_qkv();
  }
  FTL(5);
  publish_for_bulk_copies();
  consumer_sync();
  if (threadIdx.x == 0) grid_barrier(p.bar, target + (unsigned long long)G, sh, p.err);
  consumer_sync();
  FTL(6);
  pdl_trigger();

  // ---- y = attn Wo^T
  co.act_begin();
  for (int rg = r0; rg < r1; rg += RS) {
    const int nr = min(RS, r1 - rg);
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    co.template row_group_streamed<KTW_O, NCH_O, 8>(c);
    const float s = co.reduce(c, nullptr);
    const int i = warp * 32 + lane;
    const int row = i >> 3, n = i & 7;
    if (i < 128 && row < nr && n < p.B) p.y[(size_t)n * H + rg + row] = __float2bfloat16_rn(s);
  }
  FTL(9);
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
  const int *cu_q, *seq_lens, *decode_index;
  const int *block_table, *slot_map;   // of the one cache group that all these layers belong to
  int* counters;
  float *part_o, *part_ml;
  const float *rope_cos, *rope_sin;
  float scale_log2;
  int bt_stride, rope_rot, nh, nkv, nsplits;
};

// A run of pre-norm layers (attention half, feed-forward half) for a decode step of up to 8 requests as ONE
// kernel: the stages of attn_decode_fused_kernel and ffn_decode_fused_kernel layer after layer, five grid
// barriers per layer, with the weights of all layers as one uninterrupted stream through shared memory.
// The residual stream alternates between two buffers (CTA 0 writes the sum that every CTA computes), the
// halves hand their output on in y.
template <int HT, int OT, int IT, int HD, class Geo>
__global__ void __launch_bounds__(NTHREADS_WIDE, 1) decode_layers_fused_kernel(const __grid_constant__ LayersParams p) {
  constexpr int H = HT * NCW * 16, OD = OT * NCW * 16, I = IT * NCW * 16;
  constexpr int RS = Geo::RS, PG = Geo::PG, MAX_KTW = Geo::MAX_KTW;
  typedef Streamer<Geo::NST, Geo::SLOT, Geo::SROW, Geo::RS, true> WeightStream;
  typedef Streamer<Geo::AST, Geo::ASLOT, Geo::SROW, Geo::RS, false> ActStream;
  constexpr int KTW_H = largest_divisor_le(HT, MAX_KTW), NCH_H = HT / KTW_H, KC_H = KTW_H * NCW * 16;
  constexpr int KTW_O = largest_divisor_le(OT, MAX_KTW), NCH_O = OT / KTW_O, KC_O = KTW_O * NCW * 16;
  constexpr int KTW_I = largest_divisor_le(IT, MAX_KTW), NCH_I = IT / KTW_I, KC_I = KTW_I * NCW * 16;
  static_assert(MAX_B * (H * 2 + 32) <= Geo::AST * Geo::ASLOT, "the normalised rows share the activation tiles' memory");
  static_assert(16 * (HD + 8) * 2 + NCW * 16 * 2 * 4 + 16 * 2 * 4 + NCW * 16 * (HD + 8) * 4 <=
                    Geo::AST * Geo::ASLOT + 2 * NCW * 128 * 4, "the attention's scratch does not fit");

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* slots = smem;
  uint8_t* aslots = slots + Geo::NST * Geo::SLOT;
  uint8_t* xs = aslots;
  float* red = reinterpret_cast<float*>(aslots + Geo::AST * Geo::ASLOT);
  Shared* sh = reinterpret_cast<Shared*>(red + 2 * NCW * 128);
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
    ActStream as{sh, sh->afull, sh->aempty, aslots, 0u, 0ull, lane, p.err};
    const int groups = (r1 - r0 + RS - 1) / RS;
    for (int l = 0; l < p.n_layers; ++l) {
      wait_or_abort(&sh->act_ready, 0u, sh, p.err, ERR_GRID_WAIT);
      as.activation(p.attn, OD, p.B, groups, NCH_O, KC_O);
      wait_or_abort(&sh->act_ready, 1u, sh, p.err, ERR_GRID_WAIT);
      as.activation(p.act, I, p.B, groups, NCH_I, KC_I);
    }
    __syncthreads();
    if (sh->abort_flag) as.drain();
    return;
  }
  if (warp == W_WARP) {
    WeightStream ws{sh, sh->full, sh->empty, slots, 0u, policy_evict_first(), lane, p.err};
    for (int l = 0; l < p.n_layers; ++l) {
      const LayerDesc& L = p.layers[l];
      ws.rows(L.w_qkv, H, q0, q1, NCH_H, KC_H);
      ws.rows(L.w_o, OD, r0, r1, NCH_O, KC_O);
      ws.pairs(L.w_gate_up, H, I, p0, p1, NCH_H, KC_H);
      ws.rows(L.w_down, I, r0, r1, NCH_I, KC_I);
    }
    __syncthreads();
    if (sh->abort_flag) ws.drain();
    return;
  }

  reg_take<CONSUMER_REGS>();
  Consumer<Geo> co{sh, slots, aslots, red, 0u, 0u, 0u, warp, lane, (warp + cta) & (NCW - 1), p.err};
  unsigned long long target = 0;
  const int grp = p.nh / p.nkv;
  const int ny = p.nkv * ((grp + 7) >> 3);
  const int units = p.B * ny * p.nsplits;
  const bf16* x_cur = p.x;
  const float* r_cur = p.res_in;
  int turn = 0;   // norms so far: the next sum goes to res_a when even

  for (int l = 0; l < p.n_layers; ++l) {
    const LayerDesc& L = p.layers[l];
    if (l == 1) FTL(0);
    // ================= the attention half
    {
      uint2 nw[HT];
#pragma unroll
      for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(L.norm_attn + (i * 32 + lane) * 4);
      if (l == 0) {
        pdl_wait();
        if (threadIdx.x == 0) {
          unsigned long long v;
          asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.bar) : "memory");
          target = v - v % (unsigned long long)G;
        }
      }
      float* r_next = (turn & 1) ? p.res_b : p.res_a;
      norm_rows<HT>(x_cur, r_cur, cta == 0 ? r_next : nullptr, nw, L.eps_attn, p.B, xs, warp, lane);
      r_cur = r_next;
      ++turn;
      consumer_sync();
      if (l == 1) FTL(1);
      uint32_t xf[HT][2];
      load_local_x<HT, KTW_H, NCH_H>(xf, xs, co.wk, lane);
      for (int rg = q0; rg < q1; rg += RS) {
        const int nr = min(RS, q1 - rg);
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        co.template row_group_local<KTW_H, NCH_H, 8>(c, xf);
        float s = co.reduce(c, nullptr);
        const int i = warp * 32 + lane;
        const int row = i >> 3, n = i & 7;
        if (i < 128 && row < nr && n < p.B) {
          if (L.b_qkv) s += __bfloat162float(L.b_qkv[rg + row]);
          p.qkv[(size_t)n * p.NQKV + rg + row] = __float2bfloat16_rn(s);
        }
      }
    }
    if (l == 1) FTL(2);
    consumer_sync();
    if (threadIdx.x == 0) {
      grid_arrive(p.bar, sh);
      target += (unsigned long long)G;
    }
    {
      bool waited = false;
      auto wait_qkv = [&] {
        if (!waited) {
          if (threadIdx.x == 0) grid_wait(p.bar, target, sh, p.err);
          consumer_sync();
          waited = true;
          if (l == 1) FTL(3);
        }
      };
      attn_stream::FusedRope fr{p.rope_cos, p.rope_sin, p.slot_map, p.rope_rot};
      for (int u = cta; u < units; u += G) {
        const int split = u % p.nsplits, rest = u / p.nsplits;
        attn_stream::attn_stream_unit<HD, false, true>(
            wait_qkv, split, rest % ny, rest / ny, ny, aslots, &sh->s_last, p.attn, p.part_o, p.part_ml, p.qkv, p.NQKV,
            L.k_cache, L.v_cache, p.block_table, p.bt_stride, p.cu_q, p.seq_lens, p.decode_index, p.counters, p.nh, p.nkv,
            L.log2ps, L.num_pages, p.scale_log2, L.window, 0, p.nsplits, fr);
        wait_qkv();
        consumer_sync();
      }
      wait_qkv();
    }
    if (l == 1) FTL(4);
    publish_for_bulk_copies();
    consumer_sync();
    if (threadIdx.x == 0) {
      target += (unsigned long long)G;
      grid_barrier(p.bar, target, sh, p.err);
    }
    consumer_sync();
    if (l == 1) FTL(5);
    if (l == 0) pdl_trigger();
    co.act_begin();
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      co.template row_group_streamed<KTW_O, NCH_O, 8>(c);
      const float s = co.reduce(c, nullptr);
      const int i = warp * 32 + lane;
      const int row = i >> 3, n = i & 7;
      if (i < 128 && row < nr && n < p.B) p.y[(size_t)n * H + rg + row] = __float2bfloat16_rn(s);
    }
    if (l == 1) FTL(6);
    consumer_sync();
    if (threadIdx.x == 0) {
      target += (unsigned long long)G;
      grid_barrier(p.bar, target, sh, p.err);
    }
    consumer_sync();
    if (l == 1) FTL(7);

    // ================= the feed-forward half
    {
      uint2 nw[HT];
#pragma unroll
      for (int i = 0; i < HT; ++i) nw[i] = *reinterpret_cast<const uint2*>(L.norm_ffn + (i * 32 + lane) * 4);
      float* r_next = (turn & 1) ? p.res_b : p.res_a;
      norm_rows<HT>(p.y, r_cur, cta == 0 ? r_next : nullptr, nw, L.eps_ffn, p.B, xs, warp, lane);
      r_cur = r_next;
      ++turn;
      consumer_sync();
      uint32_t xf[HT][2];
      load_local_x<HT, KTW_H, NCH_H>(xf, xs, co.wk, lane);
      for (int pg = p0; pg < p1; pg += PG) {
        const int np = min(PG, p1 - pg);
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        co.template row_group_local<KTW_H, NCH_H, PG>(c, xf);
        float up;
        const float gate = co.reduce(c, &up);
        const int i = warp * 32 + lane;
        const int pair = i >> 3, n = i & 7;
        if (i < 64 && pair < np && n < p.B)
          p.act[(size_t)n * I + pg + pair] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
      }
    }
    if (l == 1) FTL(8);
    publish_for_bulk_copies();
    consumer_sync();
    if (threadIdx.x == 0) {
      target += (unsigned long long)G;
      grid_barrier(p.bar, target, sh, p.err);
    }
    consumer_sync();
    if (l == 1) FTL(9);
    co.act_begin();
    for (int rg = r0; rg < r1; rg += RS) {
      const int nr = min(RS, r1 - rg);
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      co.template row_group_streamed<KTW_I, NCH_I, 8>(c);
      const float s = co.reduce(c, nullptr);
      const int i = warp * 32 + lane;
      const int row = i >> 3, n = i & 7;
      if (i < 128 && row < nr && n < p.B) p.y[(size_t)n * H + rg + row] = __float2bfloat16_rn(s);
    }
    if (l == 1) FTL(10);
    x_cur = p.y;
    if (l + 1 < p.n_layers) {   // the next layer's norm reads y and the residual stream that CTA 0 wrote
      consumer_sync();
      if (threadIdx.x == 0) {
        target += (unsigned long long)G;
        grid_barrier(p.bar, target, sh, p.err);
      }
      consumer_sync();
      if (l == 1) FTL(11);
    }
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
  return (size_t)Geo::NST * Geo::SLOT + (size_t)Geo::AST * Geo::ASLOT + 2 * NCW * 128 * sizeof(float) + sizeof(Shared);
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
// B <= 8, bf16 weights and activations. `act` [B,I] is scratch; `bar` is a zeroed 64-bit counter that belongs
// to these launches alone (between launches it is a multiple of the number of SMs); `err` is the device error flag.
OSB_API int osb_ffn_decode_fused(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w,
                                 float eps, const void* w_gate_up, const void* w_down, void* act, unsigned long long* bar,
                                 int* err, int B, int H, int I, cudaStream_t stream) {
  if (B <= 0) return OSB_OK;
  if (B > MAX_B || !osb_ffn_decode_fused_supported(H, I)) return OSB_ERR_UNSUPPORTED;
  if ((((uintptr_t)y | (uintptr_t)res_out | (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)norm_w | (uintptr_t)w_gate_up |
        (uintptr_t)w_down | (uintptr_t)act) & 15) != 0)
    return OSB_ERR_BAD_SHAPE;
  FfnParams p;
  p.x = (const bf16*)x; p.res_in = res_in; p.res_out = res_out; p.norm_w = (const bf16*)norm_w;
  p.w_gate_up = (const bf16*)w_gate_up; p.w_down = (const bf16*)w_down; p.act = (bf16*)act; p.y = (bf16*)y;
  p.bar = bar; p.err = err; p.eps = eps; p.B = B; p.H = H; p.I = I;
  const int n_sm = sm_count();
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
  p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.block_table = block_table; p.cu_q = cu_q;
  p.seq_lens = seq_lens; p.decode_index = decode_index; p.counters = counters; p.part_o = part_o; p.part_ml = part_ml;
  p.rope.cos_t = rope_cos; p.rope.sin_t = rope_sin; p.rope.slot_map = rope_slot_map; p.rope.rot = rope_rot;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.bt_stride = bt_stride; p.nh = nh; p.nkv = nkv; p.log2ps = log2ps; p.num_pages = num_pages;
  p.window = window; p.nsplits = nsplits;
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
  p.B = B; p.NQKV = NQKV; p.cu_q = cu_q; p.seq_lens = seq_lens; p.decode_index = decode_index; p.counters = counters;
  p.block_table = block_table; p.bt_stride = bt_stride; p.slot_map = slot_map;
  p.part_o = part_o; p.part_ml = part_ml; p.rope_cos = rope_cos; p.rope_sin = rope_sin;
  p.scale_log2 = scale * 1.4426950408889634f; p.rope_rot = rope_rot; p.nh = nh; p.nkv = nkv; p.nsplits = nsplits;
  typedef Geometry<16, 12, 3, 3> GeoB;
  const int n_sm = sm_count();
  if (H == 1536) return launch_fused<GeoB>(decode_layers_fused_kernel<12, 12, 70, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  if (H == 256) return launch_fused<GeoB>(decode_layers_fused_kernel<2, 2, 4, 64, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
  return launch_fused<GeoB>(decode_layers_fused_kernel<3, 4, 15, 128, GeoB>, p, n_sm, true, stream, NTHREADS_WIDE);
}

OSB_API int osb_norm_linear_decode_supported(int H) { return H == 1536 || H == 256 || H == 384 || H == 2048; }

// y [B,N] = (rmsnorm(res_in + x) * norm_w) W^T + bias; res_out = res_in + x (fp32). B <= 8, everything bf16
// but the residual stream. Without norm_w (then no res_in, no res_out): y = x W^T + bias.
OSB_API int osb_norm_linear_decode(void* y, float* res_out, const void* x, const float* res_in, const void* norm_w,
                                   float eps, const void* w, const void* bias, int* err, int B, int N, int H,
                                   cudaStream_t stream) {
  if (B <= 0 || N <= 0) return OSB_OK;
  if (B > MAX_B || !osb_norm_linear_decode_supported(H)) return OSB_ERR_UNSUPPORTED;
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
