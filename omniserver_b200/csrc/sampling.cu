// Next-token choice from fp32 logits rows.
//   greedy: argmax, ties to the lowest index (omniserve/runners/multimodal.py:306-310,376-377)
//   temperature: p = softmax(logits / T) in fp32 (omniserve/runners/multimodal.py:378), then the
//   smallest index whose cumulative probability reaches u * total for a given uniform u in [0,1).
//   The reference draws with torch.multinomial from the global generator (multimodal.py:379); a
//   uniform supplied per (request, step) makes the draw repeatable and independent of the batch.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}

__device__ int block_argmax(const float* row, int V, float* sv, int* si) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (!(v != v)) argmax_combine(bv, bi, v, i);  // NaN never wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  bv = lane < nwarps ? sv[lane] : -INFINITY;
  bi = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  return bi == 0x7fffffff ? 0 : bi;
}

// One block per row. temperature[r] <= 0 means greedy for that row.
__global__ void __launch_bounds__(THREADS) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                         const float* __restrict__ temperature,
                                                         const float* __restrict__ uniform, int V) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float part[THREADS];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float temp = temperature ? temperature[r] : 0.0f;
  const int amax = block_argmax(row, V, sv, si);
  if (!(temp > 0.0f)) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  const float mx = row[amax];
  // contiguous chunk per thread so the cumulative sum runs in index order
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk;
  const int hi = min(lo + chunk, V);
  float s = 0.0f;
  for (int i = lo; i < hi; ++i) s += expf((row[i] - mx) / temp);
  part[threadIdx.x] = s;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.0f;
    for (int i = 0; i < (int)blockDim.x; ++i) {  // exclusive prefix in thread order
      const float v = part[i];
      part[i] = run;
      run += v;
    }
    sv[0] = run;  // total
  }
  __syncthreads();
  const float total = sv[0];
  const float target = uniform[r] * total;
  const float begin = part[threadIdx.x];
  const float end = (threadIdx.x + 1 < (int)blockDim.x) ? part[threadIdx.x + 1] : total;
  if (lo < hi && target >= begin && (target < end || (threadIdx.x + 1 == (int)blockDim.x))) {
    float run = begin;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      run += expf((row[i] - mx) / temp);
      if (run > target) {
        pick = i;
        break;
      }
    }
    if (pick < 0) pick = hi - 1;
    atomicMax(&chosen, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = chosen >= 0 ? chosen : amax;
}
}  // namespace

// out[R] int32; logits [R,V] fp32; temperature/uniform [R] fp32 (temperature may be null: all greedy).
OSB_API int osb_sample(int* out, const float* logits, const float* temperature, const float* uniform, int R, int V,
                       cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  if (V <= 0) return OSB_ERR_BAD_SHAPE;
  sample_kernel<<<R, THREADS, 0, stream>>>(out, logits, temperature, uniform, V);
  return osb_last_error();
}
