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
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320; // 10 warps: TMA, MMA, 8 epilogue
constexpr uint32_t WAIT_LIMIT = 1u << 20;  // try_wait calls (each may block for a short hardware-defined time)

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the bound was hit or another thread of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"((uint64_t)map), "r"(smem_addr(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is unused (1),
// descriptor version 1, layout type 2 (SWIZZLE_128B). Bits: [0,14) address >> 4, [16,30) LBO >> 4,
// [32,46) SBO >> 4, [46,48) version, [61,64) layout type.
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
  const uint64_t addr = (uint64_t)((smem_addr(tile) & 0x3FFFFu) >> 4);
  return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor for kind::f16: fp32 accumulator (bits [4,6) = 1), A and B bf16
// (bits [7,10) = [10,13) = 1), both K-major (bits 15, 16 = 0), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

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
    int num_tiles, int* __restrict__ err) {
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
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM: two accumulators of BN fp32 columns x 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
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
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, vabort)) {
            if (!*vabort) atomicExch(err, 101);
            *vabort = 1;
            break;
          }
          unsigned char* a_dst = tiles + (size_t)s * STAGE_BYTES;
          unsigned char* b_dst = a_dst + A_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
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
          for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(&full_bar[s], ph); ++w) {
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
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u, vabort)) {  // the epilogue has drained this accumulator
          if (!*vabort) atomicExch(err, 104);
          *vabort = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t ph = (uint32_t)(consumed / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, vabort)) {
            if (!*vabort) atomicExch(err, 102);
            *vabort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const unsigned char* a_src = tiles + (size_t)s * STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(a_src);
          const uint64_t bdesc = make_smem_desc(a_src + A_BYTES);
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
      bool ok = mbar_wait(&acc_full[buf], aph, vabort);
      if (!ok && lane == 0) {
        if (!*vabort) atomicExch(err, 103);
        *vabort = 1;
      }
      ok = ok && !*vabort;
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// A [rows, K] bf16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 elements.
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return OSB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OSB_OK : OSB_ERR_BAD_SHAPE;
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
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto k = gemm_tcgen05_kernel<BN, STAGES, EPI>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int out_cols = EPI == EPI_SWIGLU ? I : N;
  const int cols_per_tile = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const int m_blocks = (M + BM - 1) / BM;
  const int num_tiles = m_blocks * ((out_cols + cols_per_tile - 1) / cols_per_tile);
  const int ctas = num_tiles < sm_count() ? num_tiles : sm_count();
  k<<<ctas, NUM_THREADS, smem, stream>>>(ma, mb, y, yf, bias, bf, M, N, K, I, m_blocks, num_tiles, err);
  return osb_last_error();
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
// *err receives 101..103 if a wait inside the kernel ran out (the kernel then returns early).
OSB_API int osb_gemm_tcgen05_bf16(void* y, int y_dtype, const void* x, const void* w, const void* bias, int bias_dtype,
                                  int M, int N, int K, int mode, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
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
      return launch<256, 4, EPI_SWIGLU>(ma, mb, y, 0, nullptr, 0, M, N, K, I, err, stream);
    }
    rc = make_map(&mb, w, N, K, 64);
    if (rc) return rc;
    return launch<128, 6, EPI_SWIGLU>(ma, mb, y, 0, nullptr, 0, M, N, K, I, err, stream);
  }
  if (mode != 0) return OSB_ERR_BAD_SHAPE;
  // tile width: the one whose full waves over the SMs cost least; wider wins ties (less operand traffic)
  const long long c256 = wave_cost(M, N, 256, 256), c192 = wave_cost(M, N, 192, 192), c128 = wave_cost(M, N, 128, 128);
  if (c256 <= c192 && c256 <= c128) {
    rc = make_map(&mb, w, N, K, 256);
    if (rc) return rc;
    return launch<256, 4, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, stream);
  }
  if (c192 <= c128) {
    rc = make_map(&mb, w, N, K, 192);
    if (rc) return rc;
    return launch<192, 4, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, stream);
  }
  rc = make_map(&mb, w, N, K, 128);
  if (rc) return rc;
  return launch<128, 6, EPI_PLAIN>(ma, mb, y, yf, bias, bf, M, N, K, 0, err, stream);
}
