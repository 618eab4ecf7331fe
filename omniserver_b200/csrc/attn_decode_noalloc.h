// Decode attention over the paged cache for hosts that cannot allocate device memory.
//
// This entry point has no counterpart in the reference engine; it exists for users of this
// library, not for parity.
//
// Who it is for. The regular entry point (osb_paged_attn_bf16) takes two scratch buffers from
// its caller, who allocates them. Some callers cannot: an embedding runtime that reserves all
// device memory when it starts and treats any later cudaMalloc as an error; a plug-in loaded into
// a process that owns the allocator and gives the plug-in none; a real-time loop in which an
// allocator call (a possible device synchronisation) is forbidden. Such a caller still owns its
// inputs and outputs and passes them in; only the scratch comes from the library.
//
// What it does. Same computation and same result as osb_paged_attn_bf16 for the requests of the
// step that bring exactly one token (decode_index[s] >= 0): attention of that token's query heads
// over the request's cached keys and values, keys split at multiples of `chunk`, splits merged in
// order. Requests that bring several tokens are left alone. It calls no cudaMalloc, cudaFree or
// allocating library routine.
//
// The scratch. A file-scope array in device memory of osb_attn_decode_noalloc_capacity() floats
// (4 MiB). Every GPU on which this library is loaded holds that array until the process exits.
// A call needs n_decode * nh * nsplits * (hd + 2) floats plus one counter per (request, kv head)
// (rounded up a little); a call that needs more is refused with 10004 (too large) and nothing is
// launched. With nsplits == 1 no scratch is used. The array is shared by all calls and keeps the
// last call's contents. Only the counters have to start at zero, and every call clears them on
// its stream before its launch; all other values a call reads it has written itself. Two calls
// that may overlap on the GPU (different streams, no ordering between them) race on the array;
// order them.
//
// First call. The first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and keeps it. Make that first call before any
// stream capture begins on that device.
//
// Arguments as osb_paged_attn_bf16: out [T, nh*hd] bf16; q rows of q_row_stride elements;
// caches [pages, kv_heads, page_size, head_dim] bf16; block_table [S, bt_stride]; cu_q [S+1];
// seq_lens [S]; decode_index [S]; chunk a multiple of 64; nsplits = ceil(max kv length / chunk).
// n_decode must be larger than every value in decode_index: the call sizes its regions of the array
// from it and does not read decode_index on the host.
// Returns 0, a cudaError value, or a status >= 10001.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long osb_attn_decode_noalloc_capacity(void);

int osb_attn_decode_noalloc(void* out, const void* q, int q_row_stride, const void* k_cache, const void* v_cache,
                            const int* block_table, int bt_stride, const int* cu_q, const int* seq_lens,
                            const int* decode_index, int S, int nh, int nkv, int hd, int page_size, int num_pages,
                            float scale, int window, int n_decode, int chunk, int nsplits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
