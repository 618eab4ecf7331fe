// y[M,N] = x[M,K] * W[N,K]^T (+ bias) for few rows (M <= 64), bf16 operands, fp32 accumulation:
// the shape of every projection in a decode step, where time is the time to stream W once.
//
// One CTA owns 16 weight rows (output features) and all M tokens. W is the A operand of the
// m16n8k16 MMA and goes from global memory straight into registers with 16-byte loads: a lane's
// 16 bytes (8 consecutive k of one weight row) feed two MMAs whose k index is permuted the same
// way for the activations, which is legal because a dot product does not care about the order of
// k. The warps of the CTA split K; their partial tiles are summed through shared memory in warp
// order (the result does not depend on timing). Activations are read through L1.
//
// mode 1 fuses the SwiGLU activation (omniserve/kernels/fused_ops.py:111-119): W is [2I, K] with the
// gate rows first; a CTA takes 8 gate rows and the 8 matching up rows and writes
// silu(gate) * up for its 8 features, so the [M, 2I] intermediate never exists.
#include "mma_utils.cuh"

namespace {

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// DEEP: two groups of blocks in flight per warp (more registers, fewer CTAs per SM): for grids of many
// waves. Otherwise one group and at least 8 CTAs of 4 warps per SM: a grid of about a thousand CTAs
// then runs as one wave instead of one and a half.
template <int WARPS, int NT, bool DEEP>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? (DEEP ? 5 : 8) : 1) gemm_skinny_kernel(void* __restrict__ y, int y_is_f32,
                                                                 const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ w,
                                                                 const void* __restrict__ bias, int bias_is_f32,
                                                                 int M, int N, int K, int mode, int I) {
  extern __shared__ float red[];  // [WARPS][NT*8][16]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  // weight rows of this lane: A rows g and g + 8
  int row_a, row_b;
  if (mode == 1) {
    row_a = blockIdx.x * 8 + g;       // gate row
    row_b = I + blockIdx.x * 8 + g;   // up row
    if (row_a >= I) row_a = row_b = -1;
  } else {
    row_a = blockIdx.x * 16 + g;
    row_b = row_a + 8;
    if (row_a >= N) row_a = -1;
    if (row_b >= N) row_b = -1;
  }
  const bf16* wa = w + (size_t)(row_a < 0 ? 0 : row_a) * K;
  const bf16* wb = w + (size_t)(row_b < 0 ? 0 : row_b) * K;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

  const int nblocks = (K + 63) >> 6;  // blocks of 64 k
  const int b_begin = (int)(((long long)warp * nblocks) / WARPS);
  const int b_end = (int)(((long long)(warp + 1) * nblocks) / WARPS);
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

  // Blocks are processed in groups of PF with the next group's weights (and, for few tokens, the
  // next group's activations) already in flight.
  constexpr int PF = DEEP ? 2 : 1;
  constexpr bool PFX = NT <= 2;  // activations of the next group fit in registers too
  uint4 cur_lo[PF][2], cur_hi[PF][2], nxt_lo[PF][2], nxt_hi[PF][2];
  uint4 cur_x[PFX ? PF : 1][2][PFX ? NT : 1], nxt_x[PFX ? PF : 1][2][PFX ? NT : 1];
  auto load_w = [&](int b0, uint4 (&lo)[PF][2], uint4 (&hi)[PF][2]) {
#pragma unroll
    for (int u = 0; u < PF; ++u) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int k = (b0 + u) * 64 + c * 8 + hf * 32;
        const bool ok = (b0 + u) < b_end && k < K;
        lo[u][hf] = (ok && row_a >= 0) ? ld_stream16(wa + k) : zero4;
        hi[u][hf] = (ok && row_b >= 0) ? ld_stream16(wb + k) : zero4;
      }
    }
  };
  auto load_x = [&](int b0, uint4 (&xs)[PFX ? PF : 1][2][PFX ? NT : 1]) {
    if (!PFX) return;
#pragma unroll
    for (int u = 0; u < PF; ++u) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int k = (b0 + u) * 64 + c * 8 + hf * 32;
        const bool ok = (b0 + u) < b_end && k < K;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int tok = j * 8 + g;
          xs[PFX ? u : 0][hf][PFX ? j : 0] =
              (ok && tok < M) ? *reinterpret_cast<const uint4*>(x + (size_t)tok * K + k) : zero4;
        }
      }
    }
  };
  auto load_group = [&](int b0, uint4 (&lo)[PF][2], uint4 (&hi)[PF][2], uint4 (&xs)[PFX ? PF : 1][2][PFX ? NT : 1]) {
    load_w(b0, lo, hi);
    load_x(b0, xs);
  };
  // The weights do not depend on the kernel before this one: their first loads are already in
  // flight while that kernel finishes; the activations are read only after it has completed.
  load_w(b_begin, cur_lo, cur_hi);
  pdl_wait();
  load_x(b_begin, cur_x);
  for (int b = b_begin; b < b_end; b += PF) {
    load_group(b + PF, nxt_lo, nxt_hi, nxt_x);
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      if (b + u < b_end) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int k = (b + u) * 64 + c * 8 + hf * 32;
          const unsigned a0[4] = {cur_lo[u][hf].x, cur_hi[u][hf].x, cur_lo[u][hf].y, cur_hi[u][hf].y};
          const unsigned a1[4] = {cur_lo[u][hf].z, cur_hi[u][hf].z, cur_lo[u][hf].w, cur_hi[u][hf].w};
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            uint4 xv;
            if (PFX) {
              xv = cur_x[PFX ? u : 0][hf][PFX ? j : 0];
            } else {
              const int tok = j * 8 + g;
              xv = zero4;
              if (tok < M && k < K) xv = *reinterpret_cast<const uint4*>(x + (size_t)tok * K + k);
            }
            mma_bf16_16816(acc[j], a0, xv.x, xv.y);
            mma_bf16_16816(acc[j], a1, xv.z, xv.w);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < PF; ++u) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        cur_lo[u][hf] = nxt_lo[u][hf];
        cur_hi[u][hf] = nxt_hi[u][hf];
        if (PFX) {
#pragma unroll
          for (int j = 0; j < NT; ++j) cur_x[PFX ? u : 0][hf][PFX ? j : 0] = nxt_x[PFX ? u : 0][hf][PFX ? j : 0];
        }
      }
    }
  }

  pdl_trigger();
  // partial tiles -> shared memory: red[warp][token][row]
  float* mine = red + (size_t)warp * (NT * 8 * 16);
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int t0 = j * 8 + c * 2;
    mine[t0 * 16 + g] = acc[j][0];
    mine[(t0 + 1) * 16 + g] = acc[j][1];
    mine[t0 * 16 + g + 8] = acc[j][2];
    mine[(t0 + 1) * 16 + g + 8] = acc[j][3];
  }
  __syncthreads();
  if (mode == 1) {
    for (int idx = threadIdx.x; idx < M * 8; idx += WARPS * 32) {
      const int tok = idx >> 3, r = idx & 7;
      const int f = blockIdx.x * 8 + r;
      if (f >= I) continue;
      float gt = 0.0f, up = 0.0f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) {
        gt += red[(size_t)wi * (NT * 8 * 16) + tok * 16 + r];
        up += red[(size_t)wi * (NT * 8 * 16) + tok * 16 + r + 8];
      }
      // the separate kernels round gate and up to bf16 before the activation; keep that rounding
      gt = __bfloat162float(__float2bfloat16_rn(gt));
      up = __bfloat162float(__float2bfloat16_rn(up));
      const float v = (gt / (1.0f + expf(-gt))) * up;
      if (y_is_f32) ((float*)y)[(size_t)tok * I + f] = v;
      else ((bf16*)y)[(size_t)tok * I + f] = __float2bfloat16_rn(v);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < M * 16; idx += WARPS * 32) {
    const int tok = idx >> 4, r = idx & 15;
    const int n = blockIdx.x * 16 + r;
    if (n >= N) continue;
    float v = 0.0f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) v += red[(size_t)wi * (NT * 8 * 16) + tok * 16 + r];
    if (bias) v += bias_is_f32 ? ((const float*)bias)[n] : __bfloat162float(((const bf16*)bias)[n]);
    if (y_is_f32) ((float*)y)[(size_t)tok * N + n] = v;
    else ((bf16*)y)[(size_t)tok * N + n] = __float2bfloat16_rn(v);
  }
}


template <int WARPS, int NT, bool DEEP>
int launch(void* y, int y_is_f32, const bf16* x, const bf16* w, const void* bias, int bias_is_f32, int M, int N,
           int K, int mode, int I, cudaStream_t stream) {
  const size_t smem = (size_t)WARPS * NT * 8 * 16 * sizeof(float);
  auto k = gemm_skinny_kernel<WARPS, NT, DEEP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int ctas = mode == 1 ? (I + 7) / 8 : (N + 15) / 16;
  const int rc = osb_launch(k, dim3(ctas), dim3(WARPS * 32), smem, stream, y, y_is_f32, x, w, bias, bias_is_f32, M, N, K,
                            mode, I);
  return rc ? rc : osb_last_error();
}

template <int WARPS, bool DEEP>
int launch_nt(int nt, void* y, int y_is_f32, const bf16* x, const bf16* w, const void* bias, int bias_is_f32, int M,
              int N, int K, int mode, int I, cudaStream_t stream) {
  switch (nt) {
    case 1: return launch<WARPS, 1, DEEP>(y, y_is_f32, x, w, bias, bias_is_f32, M, N, K, mode, I, stream);
    case 2: return launch<WARPS, 2, DEEP>(y, y_is_f32, x, w, bias, bias_is_f32, M, N, K, mode, I, stream);
    case 3:
    case 4: return launch<WARPS, 4, DEEP>(y, y_is_f32, x, w, bias, bias_is_f32, M, N, K, mode, I, stream);
    default: return launch<WARPS, 8, DEEP>(y, y_is_f32, x, w, bias, bias_is_f32, M, N, K, mode, I, stream);
  }
}
}  // namespace

// y: bf16 (y_dtype 1) or fp32 (0); bias may be null. mode 0: y[M,N]. mode 1 (SwiGLU): w is [2I, K],
// N must be 2I, y is [M, I], bias must be null. Refuses (OSB_ERR_UNSUPPORTED) M > 64 and K not a multiple of 8.
// warps: 0 picks the number of warps per CTA (the split of K) from the shape; 4, 8 or 16 force it.
OSB_API int osb_gemm_skinny_bf16(void* y, int y_dtype, const void* x, const void* w, const void* bias,
                                 int bias_dtype, int M, int N, int K, int mode, int warps_req, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (M > 64 || K <= 0 || (K & 7)) return OSB_ERR_UNSUPPORTED;
  int I = 0;
  if (mode == 1) {
    if ((N & 1) || bias) return OSB_ERR_BAD_SHAPE;
    I = N / 2;
  } else if (mode != 0) {
    return OSB_ERR_BAD_SHAPE;
  }
  const int ctas = mode == 1 ? (I + 7) / 8 : (N + 15) / 16;
  const int nblocks = (K + 63) / 64;
  int warps = ctas >= 148 * 6 ? 4 : (ctas >= 148 * 2 ? 8 : 16);
  if (warps_req == 4 || warps_req == 8 || warps_req == 16) warps = warps_req;
  while (warps > 4 && warps > nblocks) warps >>= 1;
  const int nt = (M + 7) / 8;
  const int yf = y_dtype == OSB_F32, bf = bias_dtype == OSB_F32;
  const bf16 *xx = (const bf16*)x, *ww = (const bf16*)w;
  if (warps == 4) {
    // up to one wave of 8 CTAs per SM: the shallow variant; beyond that the deep one
    if (ctas <= 148 * 8 && nt <= 2) return launch_nt<4, false>(nt, y, yf, xx, ww, bias, bf, M, N, K, mode, I, stream);
    return launch_nt<4, true>(nt, y, yf, xx, ww, bias, bf, M, N, K, mode, I, stream);
  }
  if (warps == 8) return launch_nt<8, true>(nt, y, yf, xx, ww, bias, bf, M, N, K, mode, I, stream);
  return launch_nt<16, true>(nt, y, yf, xx, ww, bias, bf, M, N, K, mode, I, stream);
}
