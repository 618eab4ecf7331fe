// Rotary position encoding on three position axes (M-RoPE) and the write of keys/values into pages.
//
// Tables (once per step): ang[t, j] = float(pos[axis_of[j], t]) * inv_freq[j]; cos/sin in fp32.
//   omniserve/model/qwen2_llm.py:172-177 (angles), 64-69 (which axis drives frequency j).
// Rotation (per layer): pair (d, d + rot/2): x' = x*cos + rotate_half(x)*sin, in fp32.
//   omniserve/model/qwen2_llm.py:59-61,70-72.  Keys are stored rotated (qwen2_llm.py:93 precedes the
//   cache write at omniserve/cache/kv_prealloc.py:129-132).
// Positions come either from the step's explicit [3,T] table or, per request, from the request's
// state slot: cursor + rope_delta + offset on all axes (omniserve/models/qwen2_vl.py:108-112).
#include "common.cuh"

__global__ void rope_tables_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t,
                                   const int* __restrict__ pos,        // [3, T] explicit positions
                                   const int* __restrict__ pos_mode,   // [S] 0 explicit, 1 from state
                                   const int* __restrict__ tok_seq,    // [T]
                                   const int* __restrict__ cu_q,       // [S+1]
                                   const int* __restrict__ state_slot, // [S]
                                   const int* __restrict__ cursor,     // [slots, 2] (cursor, rope_delta)
                                   const float* __restrict__ inv_freq, // [half]
                                   const int* __restrict__ axis_of,    // [half] in {0,1,2}
                                   int T, int half) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, j = idx - t * half;
  const int s = tok_seq[t];
  int p;
  if (pos_mode[s] == 0) {
    p = pos[axis_of[j] * T + t];
  } else {
    const int slot = state_slot[s];
    p = cursor[slot * 2] + cursor[slot * 2 + 1] + (t - cu_q[s]);
  }
  const float ang = (float)p * inv_freq[j];
  cos_t[idx] = cosf(ang);
  sin_t[idx] = sinf(ang);
}

OSB_API int osb_rope_tables(float* cos_t, float* sin_t, const int* pos, const int* pos_mode, const int* tok_seq,
                            const int* cu_q, const int* state_slot, const int* cursor, const float* inv_freq,
                            const int* axis_of, int T, int half, cudaStream_t stream) {
  if (T <= 0 || half <= 0) return OSB_OK;
  const int total = T * half;
  rope_tables_kernel<<<(total + 255) / 256, 256, 0, stream>>>(cos_t, sin_t, pos, pos_mode, tok_seq, cu_q,
                                                             state_slot, cursor, inv_freq, axis_of, T, half);
  return osb_last_error();
}

// After a step: cursor[slot] += number of tokens the request brought.
__global__ void advance_cursor_kernel(int* __restrict__ cursor, const int* __restrict__ state_slot,
                                      const int* __restrict__ cu_q, int S) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  cursor[state_slot[s] * 2] += cu_q[s + 1] - cu_q[s];
}

OSB_API int osb_advance_cursor(int* cursor, const int* state_slot, const int* cu_q, int S, cudaStream_t stream) {
  if (S <= 0) return OSB_OK;
  advance_cursor_kernel<<<(S + 127) / 128, 128, 0, stream>>>(cursor, state_slot, cu_q, S);
  return osb_last_error();
}

// One block per (token, head) of the fused qkv row. q heads are rotated in place; k heads are rotated
// and written to the key pages; v heads are copied to the value pages.
// Page layout: [num_pages, kv_heads, page_size, head_dim]; slot = page * page_size + offset.
template <typename XT, typename CT>
__global__ void rope_kv_write_kernel(XT* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, CT* __restrict__ k_cache,
                                     CT* __restrict__ v_cache, const int* __restrict__ slot_map, int nh, int nkv,
                                     int hd, int rot, int page_size, int num_slots, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();  // a tiny kernel: the next one may begin to launch at once
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // [0,nh) q, [nh,nh+nkv) k, [nh+nkv, nh+2nkv) v
  const int row_stride = (nh + 2 * nkv) * hd;
  XT* x = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const int half = rot / 2;
  const float* c = cos_t + (size_t)t * half;
  const float* s = sin_t + (size_t)t * half;
  const bool is_q = head < nh;
  const bool is_k = !is_q && head < nh + nkv;
  CT* dst = nullptr;
  if (!is_q) {
    if (slot_map == nullptr) return;  // this entry borrows another entry's cache: nothing to write
    const int slot = slot_map[t];
    if (slot < 0 || slot >= num_slots) {
      if (threadIdx.x == 0) atomicExch(err, 3);
      return;
    }
    const int page = slot / page_size, off = slot - page * page_size;
    const int kvh = is_k ? head - nh : head - nh - nkv;
    dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
  }
  if (is_q || is_k) {
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
      const float x1 = to_f32(x[d]), x2 = to_f32(x[d + half]);
      const float cs = c[d], sn = s[d];
      const float y1 = x1 * cs - x2 * sn;
      const float y2 = x2 * cs + x1 * sn;
      if (is_q) {
        x[d] = from_f32<XT>(y1);
        x[d + half] = from_f32<XT>(y2);
      } else {
        dst[d] = from_f32<CT>(y1);
        dst[d + half] = from_f32<CT>(y2);
      }
    }
    if (is_k)
      for (int d = rot + threadIdx.x; d < hd; d += blockDim.x) dst[d] = from_f32<CT>(to_f32(x[d]));
  } else {
    for (int d = threadIdx.x; d < hd; d += blockDim.x) dst[d] = from_f32<CT>(to_f32(x[d]));
  }
}


// bf16 activations and cache, all of the head rotated, head size a multiple of 16: one thread moves
// the 8 elements at d0..d0+7 of the first half and their partners of the second half with 16-byte
// accesses (prompt portions bring thousands of rows; the scalar kernel above took 35 us for 2048).
__global__ void __launch_bounds__(256) rope_kv_write_vec_kernel(
    bf16* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t, bf16* __restrict__ k_cache,
    bf16* __restrict__ v_cache, const int* __restrict__ slot_map, int T, int nh, int nkv, int hd, int page_size,
    int num_slots, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();
  const int half = hd >> 1, per_head = half >> 3, heads = nh + 2 * nkv;
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= (long long)T * heads * per_head) return;
  const int i = (int)(id % per_head);
  const int head = (int)((id / per_head) % heads);
  const int t = (int)(id / ((long long)per_head * heads));
  const int d0 = i * 8;
  bf16* x = qkv + (size_t)t * heads * hd + (size_t)head * hd + d0;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  bf16* dst = x;
  if (!is_q) {
    if (slot_map == nullptr) return;
    const int slot = slot_map[t];
    if (slot < 0 || slot >= num_slots) {
      if (i == 0) atomicExch(err, 3);
      return;
    }
    const int page = slot / page_size, off = slot - page * page_size;
    const int kvh = is_k ? head - nh : head - nh - nkv;
    dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd + d0;
  }
  uint4 a = *reinterpret_cast<const uint4*>(x), b = *reinterpret_cast<const uint4*>(x + half);
  if (is_q || is_k) {
    const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)t * half + d0);
    const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)t * half + d0 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)t * half + d0);
    const float4 s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)t * half + d0 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
    __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x1 = __bfloat1622float2(pa[e]), x2 = __bfloat1622float2(pb[e]);
      pa[e] = __floats2bfloat162_rn(x1.x * cs[2 * e] - x2.x * sn[2 * e], x1.y * cs[2 * e + 1] - x2.y * sn[2 * e + 1]);
      pb[e] = __floats2bfloat162_rn(x2.x * cs[2 * e] + x1.x * sn[2 * e], x2.y * cs[2 * e + 1] + x1.y * sn[2 * e + 1]);
    }
  }
  if (is_q || is_k || dst != x) {
    *reinterpret_cast<uint4*>(dst) = a;
    *reinterpret_cast<uint4*>(dst + half) = b;
  }
}

// qkv [T, (nh + 2 nkv) * hd]; cos/sin [T, rot/2] (may be null when rot == 0).
OSB_API int osb_rope_kv_write(void* qkv, int x_dtype, const float* cos_t, const float* sin_t, void* k_cache,
                              void* v_cache, int cache_dtype, const int* slot_map, int T, int nh, int nkv, int hd,
                              int rot, int page_size, int num_slots, int* err, cudaStream_t stream) {
  if (T <= 0) return OSB_OK;
  if (rot < 0 || rot > hd || (rot & 1)) return OSB_ERR_BAD_SHAPE;
  if (x_dtype == OSB_BF16 && cache_dtype == OSB_BF16 && rot == hd && hd % 16 == 0 &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
      ((uintptr_t)cos_t & 15) == 0 && ((uintptr_t)sin_t & 15) == 0 && (hd / 2) % 4 == 0) {
    const long long n = (long long)T * (nh + 2 * nkv) * (hd / 16);
    const int rc = osb_launch(rope_kv_write_vec_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                              (bf16*)qkv, cos_t, sin_t, (bf16*)k_cache, (bf16*)v_cache, slot_map, T, nh, nkv, hd,
                              page_size, num_slots, err);
    return rc ? rc : osb_last_error();
  }
  const dim3 grid(T, nh + 2 * nkv);
  int threads = 32;
  while (threads < hd / 2 && threads < 128) threads <<= 1;
  return osb_dispatch(x_dtype, [&](auto xt) {
    typedef OSB_T(xt) XT;
    return osb_dispatch(cache_dtype, [&](auto ct) {
      typedef OSB_T(ct) CT;
      const int rc = osb_launch(rope_kv_write_kernel<XT, CT>, grid, dim3(threads), 0, stream, (XT*)qkv, cos_t, sin_t,
                                (CT*)k_cache, (CT*)v_cache, slot_map, nh, nkv, hd, rot, page_size, num_slots, err);
      return rc ? rc : osb_last_error();
    });
  });
}
