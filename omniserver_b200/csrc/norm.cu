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

// Vector version for H % 8 == 0: every thread keeps CH chunks of 8 elements in registers, so each
// input is read once with 16-byte loads and nothing is staged in shared memory.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <typename XT, typename WT, typename OT, int CH>
__global__ void add_rmsnorm_vec_kernel(OT* __restrict__ y, float* res_out, const float* res_in,
                                       const XT* __restrict__ x, const WT* __restrict__ w, float eps, int H,
                                       const int* __restrict__ rows) {
  __shared__ float red[32];
  pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  const XT* xr = x + (size_t)irow * H;
  const float* rr = res_in ? res_in + (size_t)irow * H : nullptr;
  float r[CH][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int e = (threadIdx.x + i * blockDim.x) * 8;
    if (e < H) {
      load8(xr + e, r[i]);
      if (rr) {
        float q[8];
        load8(rr + e, q);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[i][j] = q[j] + r[i][j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += r[i][j] * r[i][j];
    }
  }
  ss = block_sum(ss, red);
  pdl_trigger();
  const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
  float* ro = res_out ? res_out + (size_t)irow * H : nullptr;
  OT* yr = y + (size_t)orow * H;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int e = (threadIdx.x + i * blockDim.x) * 8;
    if (e < H) {
      if (ro) store8(ro + e, r[i]);
      float wv[8], o[8];
      load8(w + e, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = r[i][j] * rstd * wv[j];
      store8(yr + e, o);
    }
  }
}

// y[R,H] = norm(res_in[row] + x[row]) * w.  res_in may be null (first layer: r = x).
// res_out may be null (no write-back), may alias res_in. rows may be null (identity, R rows).
OSB_API int osb_add_rmsnorm(void* y, int y_dtype, float* res_out, const float* res_in, const void* x, int x_dtype,
                            const void* w, int w_dtype, float eps, int R, int H, const int* rows,
                            cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  if (H <= 0) return OSB_ERR_BAD_SHAPE;
  const bool vec_ok = (H % 8 == 0) && H <= 8 * 8 * 256 && (((uintptr_t)y | (uintptr_t)x | (uintptr_t)w |
                                                           (uintptr_t)res_out | (uintptr_t)res_in) & 15) == 0;
  if (vec_ok) {
    const int chunks = H / 8;
    const int ch = chunks <= 256 ? 1 : (chunks <= 512 ? 2 : (chunks <= 1024 ? 4 : 8));
    int vthreads = ((chunks + ch - 1) / ch + 31) & ~31;
    return osb_dispatch(x_dtype, [&](auto xt) {
      typedef OSB_T(xt) XT;
      return osb_dispatch(w_dtype, [&](auto wt) {
        typedef OSB_T(wt) WT;
        return osb_dispatch(y_dtype, [&](auto ot) {
          typedef OSB_T(ot) OT;
          OT* yy = (OT*)y;
          const XT* xx = (const XT*)x;
          const WT* ww = (const WT*)w;
          int rc = 0;
          if (ch == 1) rc = osb_launch(add_rmsnorm_vec_kernel<XT, WT, OT, 1>, dim3(R), dim3(vthreads), 0, stream, yy, res_out, (const float*)res_in, xx, ww, eps, H, rows);
          else if (ch == 2) rc = osb_launch(add_rmsnorm_vec_kernel<XT, WT, OT, 2>, dim3(R), dim3(vthreads), 0, stream, yy, res_out, (const float*)res_in, xx, ww, eps, H, rows);
          else if (ch == 4) rc = osb_launch(add_rmsnorm_vec_kernel<XT, WT, OT, 4>, dim3(R), dim3(vthreads), 0, stream, yy, res_out, (const float*)res_in, xx, ww, eps, H, rows);
          else rc = osb_launch(add_rmsnorm_vec_kernel<XT, WT, OT, 8>, dim3(R), dim3(vthreads), 0, stream, yy, res_out, (const float*)res_in, xx, ww, eps, H, rows);
          return rc ? rc : osb_last_error();
        });
      });
    });
  }
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
