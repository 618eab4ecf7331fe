// RMSNorm fused with the residual add.
//   r = residual + x   (or x when there is no residual yet), in fp32
//   y = r * (1 / sqrt(mean(r^2) + eps)) * w, in fp32, rounded once at the store
// The residual stream itself is kept in fp32 in every path. Formulas:
// omniserve/kernels/fused_ops.py:21-29 (norm) and 43-57 (add + norm).
#include "common.cuh"

// One block per output row. ``rows`` (optional) picks input rows; in that mode nothing is
// written back to the residual (used for the final norm at the rows whose logits are wanted).
template <typename XT, typename WT, typename OT>
__global__ void add_rmsnorm_kernel(OT* __restrict__ y, float* res_out,
                                   const float* res_in, const XT* __restrict__ x,
                                   const WT* __restrict__ w, float eps, int H,
                                   const int* __restrict__ rows) {
  __shared__ float red[32];
  extern __shared__ float rbuf[];  // H floats: the summed row
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  const XT* xr = x + (size_t)irow * H;
  const float* rr = res_in ? res_in + (size_t)irow * H : nullptr;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float r = to_f32(xr[i]);
    if (rr) r = rr[i] + r;
    rbuf[i] = r;
    ss += r * r;
  }
  ss = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
  float* ro = res_out ? res_out + (size_t)irow * H : nullptr;
  OT* yr = y + (size_t)orow * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float r = rbuf[i];
    if (ro) ro[i] = r;
    yr[i] = from_f32<OT>(r * rstd * to_f32(w[i]));
  }
}

// y[R,H] = norm(res_in[row] + x[row]) * w.  res_in may be null (first layer: r = x).
// res_out may be null (no write-back), may alias res_in. rows may be null (identity, R rows).
OSB_API int osb_add_rmsnorm(void* y, int y_dtype, float* res_out, const float* res_in, const void* x, int x_dtype,
                            const void* w, int w_dtype, float eps, int R, int H, const int* rows,
                            cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  if (H <= 0) return OSB_ERR_BAD_SHAPE;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return OSB_ERR_TOO_LARGE;
  int threads = 128;
  if (H >= 4096) threads = 512;
  else if (H >= 1024) threads = 256;
  return osb_dispatch(x_dtype, [&](auto xt) {
    typedef OSB_T(xt) XT;
    return osb_dispatch(w_dtype, [&](auto wt) {
      typedef OSB_T(wt) WT;
      return osb_dispatch(y_dtype, [&](auto ot) {
        typedef OSB_T(ot) OT;
        auto k = add_rmsnorm_kernel<XT, WT, OT>;
        if (smem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
          if (e != cudaSuccess) return (int)e;
        }
        k<<<R, threads, smem, stream>>>((OT*)y, res_out, res_in, (const XT*)x, (const WT*)w, eps, H, rows);
        return osb_last_error();
      });
    });
  });
}
