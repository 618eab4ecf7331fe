// Token embedding lookup and row overwrite (the hook by which supplied embeddings replace
// looked-up rows). Behaviour: omniserve/model/qwen2_llm.py:164, omniserve/runners/multimodal.py:123-126.
#include "common.cuh"

template <typename TT, typename OT>
__global__ void embed_lookup_kernel(OT* __restrict__ out, const TT* __restrict__ table,
                                    const int* __restrict__ ids, const int* __restrict__ src_slots,
                                    const int* __restrict__ last_token, int H, int V, int* __restrict__ err) {
  const int t = blockIdx.x;
  // a token that was sampled on the device and has not been to the host yet is taken from its request's slot
  const int slot = src_slots ? src_slots[t] : -1;
  const int id = slot >= 0 ? last_token[slot] : ids[t];
  const bool ok = (id >= 0 && id < V);
  if (!ok && threadIdx.x == 0) atomicExch(err, 1);
  const TT* src = table + (size_t)(ok ? id : 0) * H;
  OT* dst = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? from_f32<OT>(to_f32(src[i])) : from_f32<OT>(0.0f);
}

template <typename VT, typename OT>
__global__ void scatter_rows_kernel(OT* __restrict__ out, const int* __restrict__ rows,
                                    const VT* __restrict__ vals, int H, int T, int* __restrict__ err) {
  const int r = blockIdx.x;
  const int row = rows[r];
  if (row < 0 || row >= T) {
    if (threadIdx.x == 0) atomicExch(err, 2);
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)row * H + i] = from_f32<OT>(to_f32(vals[(size_t)r * H + i]));
}

// out[T,H] = table[ids]; an id outside [0,V) sets *err = 1 and writes zeros. With src_slots [T] and
// last_token given, token t is last_token[src_slots[t]] where src_slots[t] >= 0 (the caller keeps the
// slots inside last_token).
OSB_API int osb_embed_lookup(void* out, int out_dtype, const void* table, int table_dtype, const int* ids,
                             const int* src_slots, const int* last_token, int T, int H, int V, int* err,
                             cudaStream_t stream) {
  if (T <= 0) return OSB_OK;
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  return osb_dispatch(table_dtype, [&](auto tt) {
    typedef OSB_T(tt) TT;
    return osb_dispatch(out_dtype, [&](auto ot) {
      typedef OSB_T(ot) OT;
      embed_lookup_kernel<TT, OT><<<T, threads, 0, stream>>>((OT*)out, (const TT*)table, ids, src_slots, last_token, H, V,
                                                             err);
      return osb_last_error();
    });
  });
}

// out[rows[r], :] = vals[r, :]; a row outside [0,T) sets *err = 2 and is skipped.
OSB_API int osb_scatter_rows(void* out, int out_dtype, const int* rows, const void* vals, int vals_dtype,
                             int R, int H, int T, int* err, cudaStream_t stream) {
  if (R <= 0) return OSB_OK;
  return osb_dispatch(vals_dtype, [&](auto vt) {
    typedef OSB_T(vt) VT;
    return osb_dispatch(out_dtype, [&](auto ot) {
      typedef OSB_T(ot) OT;
      scatter_rows_kernel<VT, OT><<<R, 128, 0, stream>>>((OT*)out, rows, (const VT*)vals, H, T, err);
      return osb_last_error();
    });
  });
}
