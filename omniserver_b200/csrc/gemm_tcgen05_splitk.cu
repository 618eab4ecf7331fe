// y[M,N] = x[M,K] * W[N,K]^T (+ bias) for a few dozen rows (17 to 128: decode steps of many requests, the short
// portions of mixed steps), bf16 operands, on the tcgen05 tensor cores with the K range of a tile cut over the CTAs of
// a thread-block cluster.
//
// With so few rows the product is bound by reading W once, and a projection has too few 128-row tiles of W to give
// every SM one (the o projection of the 2B model: 12). So the CTAs of a cluster (1, 2, 4 or 8, chosen so that the grid
// comes close to the number of SMs) take equal parts of K for the same tile: each streams its slice of x and of the
// W tile with TMA into a ring of shared-memory stages, accumulates a partial 128 x BN tile in tensor memory
// (tcgen05.mma issued by one thread), writes it as fp32 into its own shared memory, and after a cluster barrier
// every CTA sums a share of the rows over all CTAs' partial tiles through distributed shared memory, in rank order
// (the sum does not depend on timing), adds the bias and stores the rows. Nothing goes through global memory but the
// operands and the result.
//
// Warp 0 drives TMA (one lane), warp 1 allocates tensor memory and issues the MMAs (one lane), warps 2-5 read the
// accumulator (32 lanes of tensor memory = 32 rows each). Every mbarrier wait is bounded; a CTA that gives up records
// an error code, skips its work and still takes part in both cluster barriers.
#include <cooperative_groups.h>

#include "tc_utils.cuh"

namespace cg = cooperative_groups;

namespace {
using namespace tc;

constexpr int BM = 128;          // rows of x per tile (rows from M on are read as zeros by TMA)
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192; // 6 warps: TMA, MMA, 4 epilogue

enum : int { ERR_SK_PRODUCER = 151, ERR_SK_MMA = 152, ERR_SK_EPILOGUE = 153 };

template <int BN, int STAGES>
struct SplitK {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int PSTRIDE = BN + 4;                       // floats per row of the partial tile (keeps 16-byte stores apart)
  static constexpr int PART_BYTES = BM * PSTRIDE * 4;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  // the partial tile is written when the ring is no longer read: they use the same bytes
  static constexpr int SMEM_BYTES = (RING_BYTES > PART_BYTES ? RING_BYTES : PART_BYTES) + 1024;
  static constexpr int TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_splitk_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ y,
    int y_is_f32, const void* __restrict__ bias, int bias_is_f32, int M, int N, int K, int cs, int* __restrict__ err,
    uint32_t wait_limit) {
  typedef SplitK<BN, STAGES> G;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* part = reinterpret_cast<float*>(tiles);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / cs, rank = blockIdx.x - tile * cs;
  const int n0 = tile * BN;
  const int num_kb = (K + BK - 1) / BK;
  const int kb0 = (int)((long long)num_kb * rank / cs), kb1 = (int)((long long)num_kb * (rank + 1) / cs);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, (uint32_t)G::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* vabort = &abort_flag;
  // everything above overlaps the end of the kernel in front (programmatic dependent launch); x is its output, and
  // y may be memory it still reads
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++issued) {
        const int s = issued % STAGES;
        const uint32_t ph = (uint32_t)(issued / STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, vabort, wait_limit)) {
          if (!*vabort) atomicExch(err, ERR_SK_PRODUCER);
          *vabort = 1;
          break;
        }
        unsigned char* a_dst = tiles + (size_t)s * G::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], G::STAGE_BYTES);
        tma_load_2d(a_dst, &map_a, &full_bar[s], kb * BK, 0);
        tma_load_2d(a_dst + G::A_BYTES, &map_b, &full_bar[s], kb * BK, n0);
      }
      if (*vabort) {
        // copies already started still write into this CTA's shared memory: wait for them (bounded)
        for (int i = max(0, issued - STAGES); i < issued; ++i) {
          const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
          for (uint32_t w = 0; w < wait_limit && !mbar_try_wait(&full_bar[i % STAGES], ph); ++w) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int consumed = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb, ++consumed) {
        const int s = consumed % STAGES;
        const uint32_t ph = (uint32_t)(consumed / STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, vabort, wait_limit)) {
          if (!*vabort) atomicExch(err, ERR_SK_MMA);
          *vabort = 1;
          ok = false;
          break;
        }
        fence_after();
        const unsigned char* a_src = tiles + (size_t)s * G::STAGE_BYTES;
        const uint64_t adesc = desc_kmajor(a_src);
        const uint64_t bdesc = desc_kmajor(a_src + G::A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&acc_full);   // fires when every MMA issued so far has completed (also on the give-up path)
    }
  } else {
    // the accumulator (this CTA's part of K) into shared memory as fp32, the rows that exist
    const int q = warp & 3;                  // the quarter of tensor memory's lanes this warp may read
    const int row = q * 32 + lane;
    bool ok = mbar_wait(&acc_full, 0u, vabort, wait_limit);
    if (!ok && lane == 0) {
      if (!*vabort) atomicExch(err, ERR_SK_EPILOGUE);
      *vabort = 1;
    }
    ok = __all_sync(0xffffffffu, ok && !*vabort);
    if (ok && kb1 > kb0) {
      fence_after();
      const uint32_t tmem_acc = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + (uint32_t)c0, r);
        tmem_ld_wait();
        if (row < M) {
          float* dst = part + (size_t)row * G::PSTRIDE + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                              __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
    } else if (row < M) {
      // nothing accumulated (an empty part of K, or the CTA gave up): the partial tile is zeros
      for (int c = 0; c < BN; c += 4) *reinterpret_cast<float4*>(part + (size_t)row * G::PSTRIDE + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  fence_before();
  __syncthreads();
  pdl_trigger();

  // every CTA of the cluster sums its share of the rows over all partial tiles, in rank order
  cg::cluster_group cluster = cg::this_cluster();
  if (cs > 1) cluster.sync();
  {
    const int ncols = N - n0 < BN ? N - n0 : BN;
    constexpr int C4 = BN / 4;
    for (int i = threadIdx.x; i < ((M - rank + cs - 1) / cs) * C4; i += NUM_THREADS) {
      const int row = rank + (i / C4) * cs, c = (i % C4) * 4;
      if (c >= ncols) continue;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < cs; ++r) {
        const float* src = cs > 1 ? cluster.map_shared_rank(part, r) : part;
        const float4 v = *reinterpret_cast<const float4*>(src + (size_t)row * G::PSTRIDE + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float o[4] = {acc.x, acc.y, acc.z, acc.w};
      const size_t off = (size_t)row * N + n0 + c;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (c + j >= ncols) break;
        float v = o[j];
        if (bias) v += bias_is_f32 ? ((const float*)bias)[n0 + c + j] : __bfloat162float(((const bf16*)bias)[n0 + c + j]);
        if (y_is_f32) ((float*)y)[off + j] = v;
        else ((bf16*)y)[off + j] = __float2bfloat16_rn(v);
      }
    }
  }
  if (cs > 1) cluster.sync();   // nobody's shared memory goes away while another CTA still reads it
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, (uint32_t)G::TMEM_COLS);
  }
}

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

// The tile width and the cluster size for a projection of N rows of W over K: the pair that puts the most CTAs on the
// GPU without exceeding its SMs (a cluster's CTAs run at the same time), wider tiles on a tie; a CTA keeps at least two
// k-blocks. (0, 0): the projection has more tiles than the GPU has SMs (the caller uses another kernel).
void plan(int N, int K, int* bn_out, int* cs_out) {
  const int widths[3] = {128, 96, 64};
  const int num_kb = (K + BK - 1) / BK;
  int best = 0;
  *bn_out = *cs_out = 0;
  for (int wi = 0; wi < 3; ++wi) {
    const int bn = widths[wi], tiles = (N + bn - 1) / bn;
    for (int cs = 8; cs >= 1; cs >>= 1) {
      if (tiles * cs > sm_count() || (cs > 1 && num_kb / cs < 2)) continue;
      if (tiles * cs > best) {
        best = tiles * cs;
        *bn_out = bn;
        *cs_out = cs;
      }
      break;
    }
  }
}

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* y, int yf, const void* bias, int bf, int M, int N, int K,
           int cs, int* err, uint32_t wait_limit, cudaStream_t stream) {
  typedef SplitK<BN, STAGES> G;
  auto k = gemm_splitk_kernel<BN, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  const int tiles = (N + BN - 1) / BN;
  const int rc = osb_launch_cluster(k, dim3(tiles * cs), dim3(NUM_THREADS), (size_t)G::SMEM_BYTES, stream, cs, ma, mb, y, yf,
                                    bias, bf, M, N, K, cs, err, wait_limit);
  return rc ? rc : osb_last_error();
}
}  // namespace

// 1 when osb_gemm_splitk_bf16 takes a projection of N rows of W over K for M rows of x: 1 <= M <= 128, K a multiple of
// 8, and no more tiles of 64 rows of W than the GPU has SMs.
OSB_API int osb_gemm_splitk_supported(int M, int N, int K) {
  if (M <= 0 || M > BM || N <= 0 || K <= 0 || (K & 7)) return 0;
  int bn, cs;
  plan(N, K, &bn, &cs);
  return bn != 0;
}

// y[M,N] (+ bias), y bf16 or fp32, for M <= 128 rows. Needs K % 8 == 0 and 16-byte aligned x and w (TMA); refuses
// other shapes with OSB_ERR_UNSUPPORTED. *err receives 151..153 if a wait inside the kernel ran out (the kernel then
// returns early; the result is not meaningful).
OSB_API int osb_gemm_splitk_bf16(void* y, int y_dtype, const void* x, const void* w, const void* bias, int bias_dtype, int M,
                                 int N, int K, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (M > BM || K <= 0 || (K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return OSB_ERR_UNSUPPORTED;
  int bn, cs;
  plan(N, K, &bn, &cs);
  if (bn == 0) return OSB_ERR_UNSUPPORTED;
  const int yf = y_dtype == OSB_F32, bf = bias_dtype == OSB_F32;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, x, M, K, BM);
  if (rc) return rc;
  rc = make_map(&mb, w, N, K, bn);
  if (rc) return rc;
  if (bn == 128) return launch<128, 6>(ma, mb, y, yf, bias, bf, M, N, K, cs, err, WAIT_LIMIT, stream);
  if (bn == 96) return launch<96, 7>(ma, mb, y, yf, bias, bf, M, N, K, cs, err, WAIT_LIMIT, stream);
  return launch<64, 8>(ma, mb, y, yf, bias, bf, M, N, K, cs, err, WAIT_LIMIT, stream);
}
