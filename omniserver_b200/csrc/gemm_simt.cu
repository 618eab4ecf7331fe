// y[M,N] = x[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores with fp32 accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of reduced precision is
// involved) and the fall-back for operand types and shapes the tensor-core kernels refuse.
// Every output element is one chain acc = fma(x[m,k], w[n,k], acc) over k = 0..K-1 from acc = 0,
// then + bias: the result of a row does not depend on M, on the tile it falls in, or on the
// other rows of the batch.
// The contractions it stands for: omniserve/model/qwen2_llm.py:82-83 (qkv, o), 120-121 (gate_up, down),
// 167 (LM head).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename XT, typename WT, typename BT, typename OT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(OT* __restrict__ y, const XT* __restrict__ x,
                                                        const WT* __restrict__ w, const BT* __restrict__ bias,
                                                        int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // loader mapping: 64 rows x 16 k per tile, 4 consecutive k per thread
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int gm = m0 + lrow;
      const int gn = n0 + lrow;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gk = k0 + lk + i;
        As[lk + i][lrow] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * K + gk]) : 0.0f;
        Bs[lk + i][lrow] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32(bias[gn]);
      y[(size_t)gm * N + gn] = from_f32<OT>(v);
    }
  }
}
}  // namespace

// Padding K with zeros adds fma(0,0,acc) = acc, so the tail tile keeps the chain exact.
OSB_API int osb_gemm_simt(void* y, int y_dtype, const void* x, int x_dtype, const void* w, int w_dtype,
                          const void* bias, int bias_dtype, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return OSB_OK;
  if (K <= 0) return OSB_ERR_BAD_SHAPE;
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return OSB_ERR_TOO_LARGE;
  return osb_dispatch(x_dtype, [&](auto xt) {
    typedef OSB_T(xt) XT;
    return osb_dispatch(w_dtype, [&](auto wt) {
      typedef OSB_T(wt) WT;
      return osb_dispatch(y_dtype, [&](auto ot) {
        typedef OSB_T(ot) OT;
        return osb_dispatch(bias ? bias_dtype : w_dtype, [&](auto bt) {
          typedef OSB_T(bt) BT;
          gemm_simt_kernel<XT, WT, BT, OT><<<grid, 256, 0, stream>>>((OT*)y, (const XT*)x, (const WT*)w,
                                                                     (const BT*)bias, M, N, K);
          return osb_last_error();
        });
      });
    });
  });
}
