// y[M,N] = x[M,K] * W[N,K]^T (+ bias), or silu(x Wg^T) * (x Wu^T), for a few rows of x (17 to 128: decode steps of
// many requests, short prompt portions), bf16, on tcgen05 with the operands the other way round: 128 rows of W are
// the M side of the MMA and the rows of x its N side (32, 64 or 128 accumulator columns). No row of a 128-row MMA
// tile is padding then, and W, the only large operand, is streamed once by TMA through a ring of shared-memory
// stages; the few rows of x come along from the L2. Where three stages fit in half of an SM's shared memory the ring
// is that shallow, so that two CTAs share an SM and one streams while the other sets up, exchanges or stores.
//
// One CTA owns a tile of output features over a part of K: 128 rows of W (FORM 0); with the activation 128 gate rows
// and the 128 matching up rows in two accumulators (FORM 1), or, where that would leave half of the SMs idle, 64 gate
// rows and 64 up rows as the two halves of one accumulator (FORM 2). When the tiles alone would still leave SMs idle,
// K is cut into up to 8 parts that run as the CTAs of a thread-block cluster. Every CTA writes its fp32 accumulators
// to its own shared memory; after a barrier (of the cluster, if there is one) CTA r takes its share of the rows of x,
// adds the parts in their order straight out of the others' shared memory, applies bias or activation and stores
// four features at a time.
//
// Warp 0 drives TMA (one lane), warp 1 allocates TMEM and issues the MMAs (one lane), warps 2-5 are the epilogue
// (thread = TMEM lane). The first weight tiles are asked for before the wait on the kernel in front (programmatic
// dependent launch): they do not depend on it.
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records an error code in *err, stops issuing
// work, waits (bounded) for the copies it already started, still meets its cluster at both barriers, frees its
// TMEM and returns.
#include "tc_utils.cuh"

namespace {
using namespace tc;

constexpr int WM = 128;           // rows of W per tile: the M side of the MMA
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp 0: TMA, warp 1: TMEM and MMA, warps 2..5: epilogue
constexpr int SMEM_DEEP = 220 * 1024;     // a ring that takes the SM's shared memory for one CTA
constexpr int SMEM_SHALLOW = 108 * 1024;  // one that leaves room for a second CTA on the SM: while one CTA sets up,
                                          // exchanges partial sums or stores, the other streams
constexpr int MAX_STAGES = 10;
constexpr int MAX_SPLITS = 8;     // the portable cluster size

enum { FORM_PLAIN = 0, FORM_GATED_TWO = 1, FORM_GATED_HALVES = 2 };

template <int XR, int FORM>
struct Shape {
  static constexpr int W_TILE = WM * BK * 2;
  static constexpr int W_BYTES = W_TILE * (FORM == FORM_GATED_TWO ? 2 : 1);
  static constexpr int X_BYTES = XR * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  // two CTAs per SM where that leaves each at least three stages and room for its partial sums
  static constexpr bool SHALLOW = FORM != FORM_GATED_TWO && XR <= 64;
  static constexpr int BUDGET = SHALLOW ? SMEM_SHALLOW : SMEM_DEEP;
  static constexpr int STAGES = BUDGET / STAGE_BYTES < MAX_STAGES ? BUDGET / STAGE_BYTES : MAX_STAGES;
  static constexpr int ACC_COLS = XR * (FORM == FORM_GATED_TWO ? 2 : 1);
  static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : 256;
  static constexpr int FEATS = FORM == FORM_GATED_HALVES ? WM / 2 : WM;   // output features per tile
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
  static_assert((size_t)ACC_COLS * WM * 4 <= (size_t)STAGES * STAGE_BYTES, "the partial sums reuse the ring");
  static_assert(XR % 32 == 0 && XR <= 128, "rows of x per tile");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared-memory window, of this CTA's shared address `a` in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t a, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ float silu_mul_bf16(float gate, float up) {
  // gate and up are rounded to bf16 before the activation, as where the product and the activation are two kernels
  const float g = __bfloat162float(__float2bfloat16_rn(gate));
  const float u = __bfloat162float(__float2bfloat16_rn(up));
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <int XR, int FORM>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_fewrows_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, bf16* __restrict__ y,
    const void* __restrict__ bias, int bias_is_f32, int M, int n_out, int K, int up_row0, int splits, int vec_ok,
    int* __restrict__ err, uint32_t wait_limit, uint32_t tx_extra) {
  // n_out: output features (rows of W, or of each half of it with the activation); up_row0: the row of W where the up
  // half begins; vec_ok: y may be stored 8 bytes at a time; wait_limit: try_wait calls before a wait gives up;
  // tx_extra: bytes that the producer announces beyond what it copies (0; the test of the give-up path passes 16, so
  // that no stage ever becomes full)
  using G = Shape<XR, FORM>;
  constexpr int STAGES = G::STAGES, FEATS = G::FEATS;
  constexpr bool GATED = FORM != FORM_PLAIN;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = splits > 1 ? (int)cluster_ctarank() : 0;
  const int n0 = (int)(blockIdx.x / (unsigned)splits) * FEATS;
  const int num_kb = (K + BK - 1) / BK;
  const int kb0 = (int)((long long)num_kb * rank / splits);
  const int nkb = (int)((long long)num_kb * (rank + 1) / splits) - kb0;
  const int pre = nkb < STAGES ? nkb : STAGES;   // stages whose weight tiles are asked for before the wait below
  volatile int* vabort = &abort_flag;

  auto load_w = [&](int s, int kb) {
    unsigned char* dst = ring + (size_t)s * G::STAGE_BYTES;
    tma_load_2d(dst, &map_w, &full_bar[s], kb * BK, n0);   // FORM_GATED_HALVES: a box of 64 rows, else of 128
    if (FORM == FORM_GATED_TWO) tma_load_2d(dst + G::W_TILE, &map_w, &full_bar[s], kb * BK, up_row0 + n0);
    if (FORM == FORM_GATED_HALVES) tma_load_2d(dst + G::W_TILE / 2, &map_w, &full_bar[s], kb * BK, up_row0 + n0);
  };
  auto load_x = [&](int s, int kb) {
    tma_load_2d(ring + (size_t)s * G::STAGE_BYTES + G::W_BYTES, &map_x, &full_bar[s], kb * BK, 0);
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init_fence();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full_bar[i], (uint32_t)G::STAGE_BYTES + tx_extra);
      load_w(i, kb0 + i);
    }
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, (uint32_t)G::TMEM_COLS);
  // x (and whatever shares y's memory) belongs to the kernel in front until here
  pdl_wait();
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  float* part = reinterpret_cast<float*>(ring);   // [accumulator column][TMEM lane] fp32, in the ring once it is drained

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < pre; ++i) load_x(i, kb0 + i);
      int issued = pre;
      for (; issued < nkb && !*vabort; ++issued) {
        const int s = issued % STAGES;
        const uint32_t ph = (uint32_t)(issued / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, vabort, wait_limit)) {
          if (!*vabort) atomicExch(err, 151);
          *vabort = 1;
          break;
        }
        mbar_expect_tx(&full_bar[s], (uint32_t)G::STAGE_BYTES + tx_extra);
        load_w(s, kb0 + issued);
        load_x(s, kb0 + issued);
      }
      pdl_trigger();
      if (*vabort) {
        // copies already started still write into this CTA's shared memory: wait for them (bounded)
        for (int i = max(0, issued - STAGES); i < issued; ++i) {
          const int s = i % STAGES;
          const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
          for (uint32_t w = 0; w < wait_limit && !mbar_try_wait(&full_bar[s], ph); ++w) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nkb > 0) {
      constexpr uint32_t idesc = make_idesc(WM, XR);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, vabort, wait_limit)) {
          if (!*vabort) atomicExch(err, 152);
          *vabort = 1;
          break;
        }
        fence_after();
        const unsigned char* src = ring + (size_t)s * G::STAGE_BYTES;
        const uint64_t wdesc = desc_kmajor(src);
        const uint64_t udesc = desc_kmajor(src + G::W_TILE);
        const uint64_t xdesc = desc_kmajor(src + G::W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing 16 elements (32 bytes) along K inside the swizzled row: +2 in the address field
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tmem_base, wdesc + (uint64_t)(k * 2), xdesc + (uint64_t)(k * 2), idesc, acc);
          if (FORM == FORM_GATED_TWO)
            umma_bf16(tmem_base + (uint32_t)XR, udesc + (uint64_t)(k * 2), xdesc + (uint64_t)(k * 2), idesc, acc);
        }
        umma_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
      }
      umma_commit(&acc_full);  // fires when every MMA issued so far has completed (also on the abort path)
    }
  } else {
    // ------------------------------------------------------------------ accumulators to shared memory: warps 2..5,
    // one TMEM lane quarter each
    const int q = warp & 3;
    const int tl = q * 32 + lane;   // this thread's TMEM lane
    bool ok = true;
    if (nkb > 0) {
      ok = mbar_wait(&acc_full, 0u, vabort, wait_limit);
      if (!ok && lane == 0) {
        if (!*vabort) atomicExch(err, 153);
        *vabort = 1;
      }
      ok = ok && !*vabort;
    }
    ok = __all_sync(0xffffffffu, ok);
    fence_after();
    // every copy into the ring has landed and every MMA has read it
    const uint32_t tmem_acc = tmem_base + ((uint32_t)(q * 32) << 16);
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < XR && c0 < M; c0 += 32) {
#pragma unroll
        for (int h = 0; h < (FORM == FORM_GATED_TWO ? 2 : 1); ++h) {
          uint32_t r[32];
          if (nkb > 0) {
            tmem_ld32(tmem_acc + (uint32_t)(h * XR + c0), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(h * XR + c0 + j) * WM + tl] = __uint_as_float(r[j]);
        }
      }
    }
  }
  __syncwarp();
  // every part's partial sums are in its shared memory
  if (splits > 1) cluster_sync_all();
  else __syncthreads();
  if (warp >= 2 && !*vabort) {
    // ------------------------------------------------------------------ sum over the parts, epilogue, store
    constexpr int GROUPS = FEATS / 4;   // a thread takes four neighbouring features of one row of x at a time
    const int t = threadIdx.x - 64;
    const int f = (t % GROUPS) * 4;
    const int n = n0 + f;
    const int m_lo = (int)((long long)M * rank / splits), m_hi = (int)((long long)M * (rank + 1) / splits);
    float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (!GATED && bias) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < n_out) b[j] = bias_is_f32 ? ((const float*)bias)[n + j] : __bfloat162float(((const bf16*)bias)[n + j]);
    }
    uint32_t peer[MAX_SPLITS];
    if (splits > 1) {
      const uint32_t own = smem_addr(ring);
#pragma unroll
      for (int p = 0; p < MAX_SPLITS; ++p) peer[p] = map_to_cta(own, (uint32_t)(p < splits ? p : 0));
    }
    for (int m = m_lo + t / GROUPS; m < m_hi; m += 128 / GROUPS) {
      // where this row's gate (or only) and up sums of the four features lie in a CTA's partial sums
      const int at_g = m * WM + f;
      const int at_u = FORM == FORM_GATED_TWO ? (XR + m) * WM + f : m * WM + WM / 2 + f;
      float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f), u = g;
      if (splits > 1) {
#pragma unroll
        for (int p = 0; p < MAX_SPLITS; ++p) {   // always in the order of the parts
          if (p < splits) {
            const float4 a = ld_cluster_f32x4(peer[p] + (uint32_t)at_g * 4u);
            g.x += a.x, g.y += a.y, g.z += a.z, g.w += a.w;
            if (GATED) {
              const float4 c = ld_cluster_f32x4(peer[p] + (uint32_t)at_u * 4u);
              u.x += c.x, u.y += c.y, u.z += c.z, u.w += c.w;
            }
          }
        }
      } else {
        g = *reinterpret_cast<const float4*>(part + at_g);
        if (GATED) u = *reinterpret_cast<const float4*>(part + at_u);
      }
      float v[4];
      if (GATED) {
        v[0] = silu_mul_bf16(g.x, u.x), v[1] = silu_mul_bf16(g.y, u.y), v[2] = silu_mul_bf16(g.z, u.z), v[3] = silu_mul_bf16(g.w, u.w);
      } else {
        v[0] = g.x + b[0], v[1] = g.y + b[1], v[2] = g.z + b[2], v[3] = g.w + b[3];
      }
      bf16* yp = y + (size_t)m * n_out + n;
      if (vec_ok && n + 4 <= n_out) {
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(yp) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < n_out) yp[j] = __float2bfloat16_rn(v[j]);
      }
    }
  }
  __syncwarp();
  if (splits > 1) cluster_sync_all();   // nobody's shared memory goes away while another CTA still reads it
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, (uint32_t)G::TMEM_COLS);
  }
}

// A [rows, K] bf16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 elements.
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  return tc::make_map_bf16(map, base, 2, dims, strides, box);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// How many clusters of s CTAs of this kernel the device holds at once, with the deep ring (one CTA per SM) or the
// shallow one (two); asked for once per size. (All forms with the same ring take the same share of an SM.)
int active_clusters(bool shallow, int s) {
  static int cache[2][MAX_SPLITS + 1] = {{0}};
  static bool asked[2][MAX_SPLITS + 1] = {{false}};
  if (s <= 1) return sm_count() * (shallow ? 2 : 1);
  if (s > MAX_SPLITS) return 0;
  if (!asked[shallow][s]) {
    using GS = Shape<64, FORM_PLAIN>;
    using GD = Shape<128, FORM_PLAIN>;
    static_assert(GS::SHALLOW && !GD::SHALLOW, "one form of each kind to ask with");
    void (*k)(CUtensorMap, CUtensorMap, bf16*, const void*, int, int, int, int, int, int, int, int*, uint32_t, uint32_t) =
        shallow ? gemm_fewrows_kernel<64, FORM_PLAIN> : gemm_fewrows_kernel<128, FORM_PLAIN>;
    const size_t smem = shallow ? GS::SMEM : GD::SMEM;
    int n = 0;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * s * sm_count());
      cfg.blockDim = dim3(NUM_THREADS);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = (unsigned)s;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, k, &cfg) != cudaSuccess) n = 0;
    }
    (void)cudaGetLastError();
    cache[shallow][s] = n;
    asked[shallow][s] = true;
  }
  return cache[shallow][s];
}

// Estimated time (in microseconds, roughly) of `tiles` tiles whose stages hold stage_bytes (x_bytes of them rows of x),
// K of num_kb blocks cut into s parts that all run at once: an SM takes in about 75 KB per microsecond for the CTAs it
// holds, all SMs together no more than the memory delivers W; used to choose between the two forms with the activation.
float cost(int tiles, int num_kb, int stage_bytes, int x_bytes, int s) {
  const int ctas = tiles * s;
  const int share = (ctas + sm_count() - 1) / sm_count();   // CTAs that an SM's intake is divided among
  const float per_cta = (float)((num_kb + s - 1) / s) * (float)stage_bytes / 75e3f * (float)share;
  const float memory = (float)tiles * (float)num_kb * (float)(stage_bytes - x_bytes) / 6.0e6f;   // W once
  return (per_cta > memory ? per_cta : memory) + 2.0f + (s > 1 ? 1.0f : 0.0f);
}

// Parts of K. Measured: a CTA alone on its SM takes in W no faster when it has the SM's whole shared memory for its
// ring, SMs without a CTA take in nothing, and parts of 16 blocks of K or more are long enough that clusters which
// have to wait for a place cost less than idle SMs. So: as many parts as give every SM up to two CTAs while a part
// keeps 16 blocks; else as many as still run at once while a part keeps three; one part where not even the tiles
// alone run at once.
int pick_splits(int tiles, int num_kb, int stage_bytes, int x_bytes, bool shallow, float* its_cost) {
  int best = 1;
  for (int s = MAX_SPLITS; s > 1 && best == 1; --s)
    if (num_kb >= 16 * s && tiles * s <= active_clusters(shallow, 1) && active_clusters(shallow, s) > 0) best = s;
  for (int s = MAX_SPLITS; s > 1 && best == 1; --s)
    if (num_kb >= 3 * s && tiles <= active_clusters(shallow, s)) best = s;
  if (its_cost) *its_cost = cost(tiles, num_kb, stage_bytes, x_bytes, best);
  return best;
}

template <int XR, int FORM>
int launch(const void* w, const CUtensorMap& mx, void* y, const void* bias, int bf, int M, int N, int n_out, int K,
           int splits, int* err, uint32_t wait_limit, uint32_t tx_extra, cudaStream_t stream) {
  using G = Shape<XR, FORM>;
  auto k = gemm_fewrows_kernel<XR, FORM>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
  if (e != cudaSuccess) return (int)e;
  CUtensorMap mw;
  int rc = make_map(&mw, w, N, K, FORM == FORM_GATED_HALVES ? WM / 2 : WM);
  if (rc) return rc;
  const int tiles = (n_out + G::FEATS - 1) / G::FEATS;
  const int num_kb = (K + BK - 1) / BK;
  if (splits == 0) splits = pick_splits(tiles, num_kb, G::STAGE_BYTES, G::X_BYTES, G::SHALLOW, nullptr);
  while (splits > 1 && (splits > num_kb || active_clusters(G::SHALLOW, splits) <= 0)) --splits;
  const int vec_ok = (n_out % 4 == 0) && (((uintptr_t)y & 7) == 0);
  rc = osb_launch_cluster(k, dim3(tiles * splits), dim3(NUM_THREADS), G::SMEM, stream, splits, mw, mx, (bf16*)y, bias, bf,
                          M, n_out, K, n_out, splits, vec_ok, err, wait_limit, tx_extra);
  return rc ? rc : osb_last_error();
}

// With the activation: two accumulators per CTA unless one accumulator of half as many features is estimated faster.
template <int XR>
bool halves_are_faster(int n_out, int K) {
  const int num_kb = (K + BK - 1) / BK;
  float two = 0.0f, halves = 0.0f;
  using G2 = Shape<XR, FORM_GATED_TWO>;
  using GH = Shape<XR, FORM_GATED_HALVES>;
  pick_splits((n_out + WM - 1) / WM, num_kb, G2::STAGE_BYTES, G2::X_BYTES, G2::SHALLOW, &two);
  pick_splits((n_out + WM / 2 - 1) / (WM / 2), num_kb, GH::STAGE_BYTES, GH::X_BYTES, GH::SHALLOW, &halves);
  return halves < two - 0.05f;
}
}  // namespace

// mode 0: y[M,N] = x W^T (+ bias); mode 1: w is [2I, K] with the gate rows first, N = 2I, y [M, I], no bias. y bf16,
// 1 <= M <= 128, K % 8 == 0, x and w 16-byte aligned (TMA); other shapes are refused with OSB_ERR_UNSUPPORTED.
// splits: parts of K (1 to 8; 0: chosen from the shape). form: with mode 1, 1 = two accumulators of 128 features,
// 2 = one of 64 gate and 64 up rows, 0 = chosen from the shape. *err receives 151..153 if a wait inside the kernel
// ran out (the kernel then returns early). wait_limit / tx_extra: 0 / 0 but in the test of the give-up path.
OSB_API int osb_gemm_fewrows_tc(void* y, const void* x, const void* w, const void* bias, int bias_dtype, int M, int N,
                                int K, int mode, int splits, int form, int* err, unsigned wait_limit, unsigned tx_extra,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (wait_limit == 0) wait_limit = WAIT_LIMIT;
  if (M > 128 || K <= 0 || (K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return OSB_ERR_UNSUPPORTED;
  if (mode != 0 && mode != 1) return OSB_ERR_BAD_SHAPE;
  if (mode == 1 && ((N & 1) || bias)) return OSB_ERR_BAD_SHAPE;
  if (splits < 0 || splits > MAX_SPLITS || form < 0 || form > 2) return OSB_ERR_BAD_SHAPE;
  const int n_out = mode == 1 ? N / 2 : N;
  const int xr = M <= 32 ? 32 : M <= 64 ? 64 : 128;
  CUtensorMap mx;
  const int rc = make_map(&mx, x, M, K, xr);
  if (rc) return rc;
  const int bf = bias_dtype == OSB_F32;
#define OSB_FEWROWS(XR, F) \
  return launch<XR, F>(w, mx, y, bias, bf, M, N, n_out, K, splits, err, wait_limit, tx_extra, stream)
#define OSB_FEWROWS_XR(XR)                                                          \
  if (mode == 1) {                                                                  \
    if (form == 2 || (form == 0 && halves_are_faster<XR>(n_out, K))) OSB_FEWROWS(XR, FORM_GATED_HALVES); \
    OSB_FEWROWS(XR, FORM_GATED_TWO);                                                \
  }                                                                                 \
  OSB_FEWROWS(XR, FORM_PLAIN)
  if (xr == 32) { OSB_FEWROWS_XR(32); }
  if (xr == 64) { OSB_FEWROWS_XR(64); }
  OSB_FEWROWS_XR(128);
#undef OSB_FEWROWS_XR
#undef OSB_FEWROWS
}

namespace {
template <int XR>
int plan(int n_out, int K, int mode) {
  const int num_kb = (K + BK - 1) / BK;
  using GP = Shape<XR, FORM_PLAIN>;
  using G2 = Shape<XR, FORM_GATED_TWO>;
  using GH = Shape<XR, FORM_GATED_HALVES>;
  if (mode != 1) return pick_splits((n_out + WM - 1) / WM, num_kb, GP::STAGE_BYTES, GP::X_BYTES, GP::SHALLOW, nullptr);
  if (halves_are_faster<XR>(n_out, K))
    return 100 + pick_splits((n_out + WM / 2 - 1) / (WM / 2), num_kb, GH::STAGE_BYTES, GH::X_BYTES, GH::SHALLOW, nullptr);
  return pick_splits((n_out + WM - 1) / WM, num_kb, G2::STAGE_BYTES, G2::X_BYTES, G2::SHALLOW, nullptr);
}
}  // namespace

// What splits = 0 and form = 0 choose for M rows of this shape: parts of K, and 100 more with the halves form.
OSB_API int osb_gemm_fewrows_tc_plan(int M, int N, int K, int mode) {
  const int n_out = mode == 1 ? N / 2 : N;
  return M <= 32 ? plan<32>(n_out, K, mode) : M <= 64 ? plan<64>(n_out, K, mode) : plan<128>(n_out, K, mode);
}

// Asks the device once how many clusters of each size it holds (the answers are kept), so that no launch has to ask
// while a CUDA graph is being captured.
OSB_API int osb_gemm_fewrows_tc_prepare() {
  for (int shallow = 0; shallow < 2; ++shallow)
    for (int s = 2; s <= MAX_SPLITS; ++s) (void)active_clusters(shallow != 0, s);
  return OSB_OK;
}
