// SiLU(gate) * up on a fused [T, 2I] tensor (gate first, up second), fp32 math, one rounding.
// Formula: omniserve/kernels/fused_ops.py:111-119.
#include "common.cuh"

template <typename XT, typename OT>
__global__ void silu_mul_kernel(OT* __restrict__ out, const XT* __restrict__ gu, int I, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + i]);
    const float u = to_f32(gu[t * 2 * I + I + i]);
    const float sig = 1.0f / (1.0f + expf(-g));
    out[idx] = from_f32<OT>((g * sig) * u);
  }
}

// out[T,I] = silu(gu[:, :I]) * gu[:, I:]
OSB_API int osb_silu_mul(void* out, int out_dtype, const void* gu, int gu_dtype, int T, int I, cudaStream_t stream) {
  if (T <= 0 || I <= 0) return OSB_OK;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  return osb_dispatch(gu_dtype, [&](auto xt) {
    typedef OSB_T(xt) XT;
    return osb_dispatch(out_dtype, [&](auto ot) {
      typedef OSB_T(ot) OT;
      silu_mul_kernel<XT, OT><<<(int)blocks, threads, 0, stream>>>((OT*)out, (const XT*)gu, I, total);
      return osb_last_error();
    });
  });
}
