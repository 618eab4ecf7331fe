// y[M,N] = x[M,K] * W[N,K]^T (+ bias) for many rows with two SMs on one tile: tcgen05.mma.cta_group::2.
//
// A cluster of two CTAs computes a 256 x BN tile of y. Each CTA loads its own 128 rows of x and its own
// half (BN/2 rows) of the W tile by TMA into its own shared memory; one thread of the even CTA issues
// MMAs of shape 256 x BN x 16 that read both CTAs' shared memory and write both CTAs' tensor memory
// (each CTA keeps the accumulator of its 128 rows). Per CTA a k-block costs 16 KB of x and BN/2 x 128
// bytes of W for 128 x BN x 64 multiply-adds: half the W traffic per flop of a single-CTA tile, which is
// what lets the tensor cores run from the L2.
//
// Hand-over between the two CTAs uses no loads with multicast: each TMA copy lands in the shared memory
// of the CTA that issued it and reports its bytes to the even CTA's full barrier; the even CTA's
// tcgen05.commit arrives on the empty / accumulator-full barriers of both CTAs (commit with a CTA mask);
// the odd CTA's epilogue warps arrive on the even CTA's accumulator-empty barrier with a remote
// mbarrier.arrive. Roles per CTA: warp 0 TMA producer, warp 1 tensor-memory allocation (and, in the even
// CTA, the MMA issuer), warps 2-9 epilogue. Epilogues as in gemm_tcgen05.cu: plain (bias) and SwiGLU (the
// even CTA loads gate rows, the odd CTA the matching up rows, so accumulator columns [0, BN/2) are gate
// and [BN/2, BN) up; omniserve/kernels/fused_ops.py:111-119).
//
// Every wait on an mbarrier is bounded; a CTA that gives up records a code in *err, waits (bounded) for its
// copies in flight and goes to the common exit, where the pair meets at a cluster barrier and frees its
// tensor memory. The partner's waits then run out as well.
#include "tc_utils.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;  // rows per CTA; the pair's tile has 256
constexpr int BK = 64;
constexpr int NUM_THREADS = 320;  // 10 warps: TMA, MMA, 8 epilogue
enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared-memory window, of this CTA's variable `p` in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile into this CTA's shared memory; the bytes are reported to the barrier at `bar_cluster_addr`
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair when the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_addr(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// Stores 32 consecutive output columns of one row (fp32 values in v) as bf16 or fp32.
__device__ __forceinline__ void store_row32(void* y, int y_is_f32, size_t row_off, int col, int ncols, const float* v,
                                            bool vec_ok) {
  if (y_is_f32) {
    float* yp = (float*)y + row_off + col;
    if (vec_ok && col + 32 <= ncols) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(yp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (col + j < ncols) yp[j] = v[j];
    }
  } else {
    bf16* yp = (bf16*)y + row_off + col;
    if (vec_ok && col + 32 <= ncols) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
        h[0] = __floats2bfloat162_rn(v[j], v[j + 1]);
        h[1] = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        h[2] = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        h[3] = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        *reinterpret_cast<uint4*>(yp + j) = u;
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col + j < ncols) yp[j] = __float2bfloat16_rn(v[j]);
    }
  }
}

// Persistent: pair p computes tiles p, p + pairs, ... (tile t = column block t / m_blocks, 256-row block
// t % m_blocks, so that pairs running together share W tiles through the L2). The accumulator is
// double-buffered in tensor memory (2 x BN columns in each CTA).
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_tcgen05_2cta_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ y,
    int y_is_f32, const void* __restrict__ bias, int bias_is_f32, int M, int N, int K, int I, int m_blocks,
    int num_tiles, int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int OUT_COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;
  constexpr uint32_t TMEM_COLS = 2 * BN <= 256 ? 256 : 512;
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float bias_s[8][BN];  // a copy per epilogue warp (no CTA barrier)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // used in the even CTA only: its expect_tx arrival, bytes of both CTAs' copies
      mbar_init(&empty_bar[s], 1);  // one commit, delivered to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);  // used in the even CTA only: eight epilogue warps of each CTA
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc_pair(&tmem_base_slot, TMEM_COLS);
  // The kernel is launched with programmatic stream serialization: it may begin while the kernel before it in the
  // stream is still writing x. Only the set-up above runs before that kernel has completed.
  pdl_wait();
  fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other CTA
  fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* vabort = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int issued = 0;
      for (int tile = pair; tile < num_tiles && !*vabort; tile += pairs) {
        const int m0 = (tile % m_blocks) * (2 * BM) + (int)rank * BM;
        const int nt = tile / m_blocks;
        // this CTA's half of the W tile
        const int b_row = EPI == EPI_SWIGLU ? (rank == 0 ? nt * OUT_COLS : I + nt * OUT_COLS) : nt * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++issued) {
          const int s = issued % STAGES;
          const uint32_t ph = (uint32_t)(issued / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, vabort)) {
            if (!*vabort) atomicExch(err, 121);
            *vabort = 1;
            break;
          }
          unsigned char* a_dst = tiles + (size_t)s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          const uint32_t full0 = map_to_cta(&full_bar[s], 0);
          tma_load_2d_pair(a_dst, &map_a, full0, kb * BK, m0);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, full0, kb * BK, b_row);
        }
      }
      if (*vabort) {
        // Copies already started still write into this CTA's shared memory. Their completion is counted on the
        // even CTA's barriers, which the odd CTA cannot wait on, and the even CTA's count includes the odd
        // CTA's copies: both simply give the copies far more time than they take before going to the exit.
        for (int i = 0; i < 64; ++i) __nanosleep(4000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN);
      int consumed = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
        const int buf = local & 1;
        const uint32_t aph = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u, vabort)) {  // both CTAs' epilogues have drained this accumulator
          if (!*vabort) atomicExch(err, 124);
          *vabort = 1;
          ok = false;
          break;
        }
        fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t ph = (uint32_t)(consumed / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, vabort)) {
            if (!*vabort) atomicExch(err, 122);
            *vabort = 1;
            ok = false;
            break;
          }
          fence_after();
          const unsigned char* a_src = tiles + (size_t)s * STAGE_BYTES;
          const uint64_t adesc = desc_kmajor(a_src);
          const uint64_t bdesc = desc_kmajor(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_pair(tmem_acc, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[s]);  // frees the stage in both CTAs when these MMAs have read it
        }
        umma_commit_pair(&acc_full[buf]);  // also on the abort path: fires when every MMA issued so far has completed
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 2..9 of both CTAs
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int ew = warp - 2;           // two warps per quarter: each takes half of the tile's columns
    const int c_begin = (ew >> 2) * (OUT_COLS / 2), c_end = c_begin + OUT_COLS / 2;
    const int ncols = EPI == EPI_SWIGLU ? I : N;
    const bool vec_ok = y_is_f32 ? ((ncols & 3) == 0) : ((ncols & 7) == 0);
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += pairs, ++local) {
      const int m0 = (tile % m_blocks) * (2 * BM) + (int)rank * BM;
      const int n0 = (tile / m_blocks) * OUT_COLS;
      const int buf = local & 1;
      const uint32_t aph = (uint32_t)(local >> 1) & 1u;
      const int row = m0 + q * 32 + lane;
      if (EPI == EPI_PLAIN && bias) {
        __syncwarp();
        for (int j = lane; j < BN; j += 32) {
          const int col = n0 + j;
          bias_s[ew][j] = col < N ? (bias_is_f32 ? ((const float*)bias)[col] : __bfloat162float(((const bf16*)bias)[col])) : 0.0f;
        }
        __syncwarp();
      }
      bool ok = mbar_wait(&acc_full[buf], aph, vabort);
      if (!ok && lane == 0) {
        if (!*vabort) atomicExch(err, 123);
        *vabort = 1;
      }
      ok = ok && !*vabort;
      if (!__all_sync(0xffffffffu, ok)) break;
      fence_after();
      const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(q * 32) << 16);
      const size_t row_off = (size_t)row * ncols;
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        float v[32];
        if (EPI == EPI_SWIGLU) {
          uint32_t g[32], u[32];
          tmem_ld32(tmem_acc + (uint32_t)c0, g);
          tmem_ld32(tmem_acc + (uint32_t)(BN / 2 + c0), u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            // the two-kernel path rounds gate and up to bf16 before the activation; keep that rounding
            const float gg = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j])));
            const float uu = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j])));
            v[j] = __fdividef(gg, 1.0f + __expf(-gg)) * uu;
          }
        } else {
          uint32_t r[32];
          tmem_ld32(tmem_acc + (uint32_t)c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += bias_s[ew][c0 + j];
          }
        }
        if (row < M && n0 + c0 < ncols) store_row32(y, y_is_f32, row_off, n0 + c0, ncols, v, vec_ok);
      }
      // this warp has read its part of the accumulator: tell the MMA issuer (in the even CTA)
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[buf], 0));
    }
  }
  fence_before();
  __syncthreads();
  cluster_sync_all();  // nothing of the partner is touched after this
  if (warp == 1) {
    fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

template <int BN, int STAGES, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* y, int yf, const void* bias, int bf, int M, int N, int K,
           int I, int* err, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + (BN / 2) * BK * 2) + 1024;
  auto k = gemm_tcgen05_2cta_kernel<BN, STAGES, EPI>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int out_cols = EPI == EPI_SWIGLU ? I : N;
  const int cols_per_tile = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const int m_blocks = (M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = m_blocks * ((out_cols + cols_per_tile - 1) / cols_per_tile);
  const int max_pairs = sm_count() / 2;
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  const int rc = osb_launch_cluster(k, dim3(2 * pairs), dim3(NUM_THREADS), smem, stream, 2, ma, mb, y, yf, bias, bf, M, N,
                                    K, I, m_blocks, num_tiles, err);
  return rc ? rc : osb_last_error();
}

// full waves of tiles over the SM pairs, in units of tile columns
static inline long long wave_cost(int M, int out_cols, int cols_per_tile, int width) {
  const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((out_cols + cols_per_tile - 1) / cols_per_tile);
  const long long pairs = sm_count() / 2;
  return ((tiles + pairs - 1) / pairs) * width;
}
}  // namespace

// As osb_gemm_tcgen05_bf16 (same arguments and modes), computed by pairs of CTAs on 256-row tiles.
// *err receives 121..124 if a wait inside the kernel ran out.
OSB_API int osb_gemm_tcgen05_2cta_bf16(void* y, int y_dtype, const void* x, const void* w, const void* bias,
                                       int bias_dtype, int M, int N, int K, int mode, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (K <= 0 || (K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return OSB_ERR_UNSUPPORTED;
  const int yf = y_dtype == OSB_F32, bf = bias_dtype == OSB_F32;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, x, M, K, BM);
  if (rc) return rc;
  if (mode == 1) {
    if ((N & 1) || bias || yf) return OSB_ERR_BAD_SHAPE;
    const int I = N / 2;
    rc = make_map(&mb, w, N, K, 128);
    if (rc) return rc;
    return launch<256, 6, EPI_SWIGLU>(ma, mb, y, 0, nullptr, 0, M, N, K, I, err, stream);
  }
  if (mode != 0) return OSB_ERR_BAD_SHAPE;
  if (wave_cost(M, N, 256, 256) <= wave_cost(M, N, 192, 192)) {
    rc = make_map(&mb, w, N, K, 128);
    if (rc) return rc;
    return launch<256, 6, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, stream);
  }
  rc = make_map(&mb, w, N, K, 96);
  if (rc) return rc;
  return launch<192, 7, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, stream);
}
