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
                                                         const float* __restrict__ uniform, int V,
                                                         int* __restrict__ keep, const int* __restrict__ keep_at) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float part[THREADS];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float temp = temperature ? temperature[r] : 0.0f;
  const int amax = block_argmax(row, V, sv, si);
  if (!(temp > 0.0f)) {
    if (threadIdx.x == 0) {
      out[r] = amax;
      if (keep) keep[keep_at[r]] = amax;
    }
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
  if (threadIdx.x == 0) {
    const int tok = chosen >= 0 ? chosen : amax;
    out[r] = tok;
    if (keep) keep[keep_at[r]] = tok;
  }
}

// Greedy over many CTAs: each block takes a slice of the row, the last step combines the slices.
constexpr int ARGMAX_SLICES = 32;

__global__ void __launch_bounds__(256) argmax_partial_kernel(float* __restrict__ pv, int* __restrict__ pi,
                                                             const float* __restrict__ logits, int V) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int r = blockIdx.y, sl = blockIdx.x;
  const int per = (((V + ARGMAX_SLICES - 1) / ARGMAX_SLICES) + 3) & ~3;
  const int lo = sl * per, hi = min(V, lo + per);
  const float* row = logits + (size_t)r * V;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const bool vec = ((V & 3) == 0);  // rows stay 16-byte aligned
  if (vec) {
    for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      if (!(v.x != v.x)) argmax_combine(bv, bi, v.x, i);
      if (!(v.y != v.y)) argmax_combine(bv, bi, v.y, i + 1);
      if (!(v.z != v.z)) argmax_combine(bv, bi, v.z, i + 2);
      if (!(v.w != v.w)) argmax_combine(bv, bi, v.w, i + 3);
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = row[i];
      if (!(v != v)) argmax_combine(bv, bi, v, i);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    bv = lane < nwarps ? sv[lane] : -INFINITY;
    bi = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_combine(bv, bi, ov, oi);
    }
    if (lane == 0) {
      pv[r * ARGMAX_SLICES + sl] = bv;
      pi[r * ARGMAX_SLICES + sl] = bi;
    }
  }
}

__global__ void argmax_final_kernel(int* __restrict__ out, const float* __restrict__ pv, const int* __restrict__ pi,
                                    int* __restrict__ keep, const int* __restrict__ keep_at) {
  const int r = blockIdx.x, lane = threadIdx.x;
  float bv = pv[r * ARGMAX_SLICES + lane];
  int bi = pi[r * ARGMAX_SLICES + lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(bv, bi, ov, oi);
  }
  if (lane == 0) {
    const int tok = bi == 0x7fffffff ? 0 : bi;
    out[r] = tok;
    if (keep) keep[keep_at[r]] = tok;
  }
}
}  // namespace

// Greedy for all rows with the row spread over 32 CTAs. scratch: R*32 floats and R*32 ints.
// keep/keep_at (may be null): the token of row r is also stored at keep[keep_at[r]], from where the next
// step's embedding lookup can take it without a trip to the host.
OSB_API int osb_argmax(int* out, const float* logits, float* scratch_v, int* scratch_i, int R, int V, int* keep,
                       const int* keep_at, cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  if (V <= 0) return OSB_ERR_BAD_SHAPE;
  static_assert(ARGMAX_SLICES == 32, "the final step is one warp");
  argmax_partial_kernel<<<dim3(ARGMAX_SLICES, R), 256, 0, stream>>>(scratch_v, scratch_i, logits, V);
  int rc = osb_last_error();
  if (rc) return rc;
  argmax_final_kernel<<<R, 32, 0, stream>>>(out, scratch_v, scratch_i, keep, keep_at);
  return osb_last_error();
}

// out[R] int32; logits [R,V] fp32; temperature/uniform [R] fp32 (temperature may be null: all greedy).
OSB_API int osb_sample(int* out, const float* logits, const float* temperature, const float* uniform, int R, int V,
                       int* keep, const int* keep_at, cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  if (V <= 0) return OSB_ERR_BAD_SHAPE;
  sample_kernel<<<R, THREADS, 0, stream>>>(out, logits, temperature, uniform, V, keep, keep_at);
  return osb_last_error();
}
