// y[M,N] = x[M,K] * W[N,K]^T (+ bias) for many rows (prompt portions), bf16 operands, on the
// fifth-generation tensor cores: tcgen05.mma issued by one thread, operands staged in shared
// memory by TMA (128-byte swizzle), the fp32 accumulator tile in tensor memory (TMEM), read back
// with tcgen05.ld for the epilogue.
//
// One CTA computes a 128 x BN tile of y. Warp 0 drives TMA (one lane), warp 1 allocates TMEM and
// issues the MMAs (one lane), warps 2-9 run the epilogue (32 TMEM lanes = 32 rows and half of the columns each).
// Stages of the ring are handed over with mbarriers: full[s] (TMA -> MMA, transaction bytes) and
// empty[s] (MMA -> TMA, by tcgen05.commit); acc_full tells the epilogue the accumulator is complete.
//
// Epilogues: plain (bias, bf16 or fp32 output) and SwiGLU: W is [2I, K] with the gate rows first;
// the B tile of a CTA is 64 gate rows and the 64 matching up rows, and the CTA writes
// silu(gate) * up for its 64 features (omniserve/kernels/fused_ops.py:111-119), so the [M, 2I]
// intermediate never reaches memory.
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records an error code in
// *err, stops issuing work, waits (bounded) for the copies it already started, frees its TMEM
// and returns.
#include "tc_utils.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320; // 10 warps: TMA, MMA, 8 epilogue

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

// Stores 32 consecutive output columns of one row (fp32 values in r) as bf16 or fp32.
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

// Persistent kernel: CTA c computes tiles c, c + gridDim.x, ... (tile t = column block t / m_blocks,
// row block t % m_blocks, so that CTAs running together share weight tiles through the L2). The
// accumulator is double-buffered in TMEM (2 x BN columns): the epilogue of a tile overlaps the
// main loop of the next.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ y,
    int y_is_f32, const void* __restrict__ bias, int bias_is_f32, int M, int N, int K, int I, int m_blocks,
    int num_tiles, int* __restrict__ err, uint32_t wait_limit, uint32_t tx_extra) {
  // wait_limit: try_wait calls before a wait gives up; tx_extra: bytes that the producer announces beyond what it
  // copies (0; the test of the give-up path passes 16, so that no stage ever becomes full)
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int OUT_COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;  // output columns per tile
  constexpr int TMEM_COLS = 2 * BN <= 256 ? 256 : 512;       // two accumulators; allocations are powers of two
  // 1024-byte alignment of every tile (required by the 128-byte swizzle)
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float bias_s[8][BN];  // the bias of a tile's columns: each epilogue warp stages a copy of its own (no CTA barrier)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) {  // TMEM: two accumulators of BN fp32 columns x 128 lanes
    tmem_alloc(&tmem_base_slot, (uint32_t)TMEM_COLS);
  }
  // the set-up above may run while the kernel before this one in the stream finishes; x (and whatever shares y's
  // memory) belongs to that kernel until here
  pdl_wait();
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* vabort = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = 0;  // k-blocks issued over all tiles
      for (int tile = blockIdx.x; tile < num_tiles && !*vabort; tile += gridDim.x) {
        const int m0 = (tile % m_blocks) * BM;
        const int n0 = (tile / m_blocks) * OUT_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++issued) {
          const int s = issued % STAGES;
          const uint32_t ph = (uint32_t)(issued / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, vabort, wait_limit)) {
            if (!*vabort) atomicExch(err, 101);
            *vabort = 1;
            break;
          }
          unsigned char* a_dst = tiles + (size_t)s * STAGE_BYTES;
          unsigned char* b_dst = a_dst + A_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES + tx_extra);
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * BK, m0);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(b_dst, &map_b, &full_bar[s], kb * BK, n0);                    // gate rows
            tma_load_2d(b_dst + B_BYTES / 2, &map_b, &full_bar[s], kb * BK, I + n0);  // up rows
          } else {
            tma_load_2d(b_dst, &map_b, &full_bar[s], kb * BK, n0);
          }
        }
      }
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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int consumed = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t aph = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u, vabort, wait_limit)) {  // the epilogue has drained this accumulator
          if (!*vabort) atomicExch(err, 104);
          *vabort = 1;
          ok = false;
          break;
        }
        fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t ph = (uint32_t)(consumed / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, vabort, wait_limit)) {
            if (!*vabort) atomicExch(err, 102);
            *vabort = 1;
            ok = false;
            break;
          }
          fence_after();
          const unsigned char* a_src = tiles + (size_t)s * STAGE_BYTES;
          const uint64_t adesc = desc_kmajor(a_src);
          const uint64_t bdesc = desc_kmajor(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 elements (32 bytes) along K inside the swizzled row: +2 in the address field
            umma_bf16(tmem_acc, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
        }
        umma_commit(&acc_full[buf]);  // fires when every MMA issued so far has completed (also on the abort path)
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 2..9
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int ew = warp - 2;           // two warps per quarter: each takes half of the tile's columns
    const int c_begin = (ew >> 2) * (OUT_COLS / 2), c_end = c_begin + OUT_COLS / 2;
    const int ncols = EPI == EPI_SWIGLU ? I : N;
    const bool vec_ok = y_is_f32 ? ((ncols & 3) == 0) : ((ncols & 7) == 0);
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % m_blocks) * BM;
      const int n0 = (tile / m_blocks) * OUT_COLS;
      const int buf = local & 1;
      const uint32_t aph = (uint32_t)(local >> 1) & 1u;
      const int row = m0 + q * 32 + lane;
      if (EPI == EPI_PLAIN && bias) {
        // while the tile is still being computed: its bias into shared memory, once, as fp32
        __syncwarp();
        for (int j = lane; j < BN; j += 32) {
          const int col = n0 + j;
          bias_s[ew][j] = col < N ? (bias_is_f32 ? ((const float*)bias)[col] : __bfloat162float(((const bf16*)bias)[col])) : 0.0f;
        }
        __syncwarp();
      }
      bool ok = mbar_wait(&acc_full[buf], aph, vabort, wait_limit);
      if (!ok && lane == 0) {
        if (!*vabort) atomicExch(err, 103);
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
      // this warp has read its part of the accumulator: hand the buffer back to the MMA issuer
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, (uint32_t)TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
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

template <int BN, int STAGES, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* y, int yf, const void* bias, int bf, int M, int N, int K,
           int I, int* err, uint32_t wait_limit, uint32_t tx_extra, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto k = gemm_tcgen05_kernel<BN, STAGES, EPI>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int out_cols = EPI == EPI_SWIGLU ? I : N;
  const int cols_per_tile = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const int m_blocks = (M + BM - 1) / BM;
  const int num_tiles = m_blocks * ((out_cols + cols_per_tile - 1) / cols_per_tile);
  const int ctas = num_tiles < sm_count() ? num_tiles : sm_count();
  const int rc = osb_launch(k, dim3(ctas), dim3(NUM_THREADS), smem, stream, ma, mb, y, yf, bias, bf, M, N, K, I, m_blocks,
                            num_tiles, err, wait_limit, tx_extra);
  return rc ? rc : osb_last_error();
}

// Time of a shape in units of "one 128-column tile on one SM": full waves over the SMs.
static inline long long wave_cost(int M, int out_cols, int cols_per_tile, int width) {
  const long long tiles = (long long)((M + BM - 1) / BM) * ((out_cols + cols_per_tile - 1) / cols_per_tile);
  const long long waves = (tiles + sm_count() - 1) / sm_count();
  return waves * width;
}
}  // namespace

// mode 0: y[M,N] (+bias), y bf16 or fp32. mode 1 (SwiGLU): w is [2I, K], N = 2I, y [M, I] bf16, no bias.
// Needs K % 8 == 0 and 16-byte aligned x and w (TMA); refuses other shapes with OSB_ERR_UNSUPPORTED.
// *err receives 101..104 if a wait inside the kernel ran out (the kernel then returns early).
// wait_limit / tx_extra: 0 / 0 but in the test of the give-up path: so many polls per wait; so many bytes announced
// to a stage's barrier beyond those copied, which keeps every stage from ever becoming full.
OSB_API int osb_gemm_tcgen05_bf16_ex(void* y, int y_dtype, const void* x, const void* w, const void* bias, int bias_dtype,
                                     int M, int N, int K, int mode, int* err, unsigned wait_limit, unsigned tx_extra,
                                     cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (wait_limit == 0) wait_limit = WAIT_LIMIT;
  if (K <= 0 || (K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return OSB_ERR_UNSUPPORTED;
  const int yf = y_dtype == OSB_F32, bf = bias_dtype == OSB_F32;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, x, M, K, BM);
  if (rc) return rc;
  if (mode == 1) {
    if ((N & 1) || bias || yf) return OSB_ERR_BAD_SHAPE;
    const int I = N / 2;
    // 256-wide B tiles (128 features) unless 128-wide ones fill the SMs better
    if (wave_cost(M, I, 128, 2) <= wave_cost(M, I, 64, 1)) {  // cost in units of 128 B-tile rows
      rc = make_map(&mb, w, N, K, 128);
      if (rc) return rc;
      return launch<256, 4, EPI_SWIGLU>(ma, mb, y, 0, nullptr, 0, M, N, K, I, err, wait_limit, tx_extra, stream);
    }
    rc = make_map(&mb, w, N, K, 64);
    if (rc) return rc;
    return launch<128, 6, EPI_SWIGLU>(ma, mb, y, 0, nullptr, 0, M, N, K, I, err, wait_limit, tx_extra, stream);
  }
  if (mode != 0) return OSB_ERR_BAD_SHAPE;
  // tile width: the one whose full waves over the SMs cost least; wider wins ties (less operand traffic)
  const long long c256 = wave_cost(M, N, 256, 256), c192 = wave_cost(M, N, 192, 192), c128 = wave_cost(M, N, 128, 128);
  if (c256 <= c192 && c256 <= c128) {
    rc = make_map(&mb, w, N, K, 256);
    if (rc) return rc;
    return launch<256, 4, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, wait_limit, tx_extra, stream);
  }
  if (c192 <= c128) {
    rc = make_map(&mb, w, N, K, 192);
    if (rc) return rc;
    return launch<192, 4, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, wait_limit, tx_extra, stream);
  }
  rc = make_map(&mb, w, N, K, 128);
  if (rc) return rc;
  return launch<128, 6, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, wait_limit, tx_extra, stream);
}

OSB_API int osb_gemm_tcgen05_bf16(void* y, int y_dtype, const void* x, const void* w, const void* bias, int bias_dtype,
                                  int M, int N, int K, int mode, int* err, cudaStream_t stream) {
  return osb_gemm_tcgen05_bf16_ex(y, y_dtype, x, w, bias, bias_dtype, M, N, K, mode, err, 0u, 0u, stream);
}
