// An entry point of the split-key decode attention that allocates nothing.
// It has no counterpart in the reference engine.
//
// Who needs it: a caller that cannot ask for device memory while it runs. A
// serving process that hands all free device memory to its own pools at
// start-up has none left for the driver's allocator, and a cudaMalloc there
// may also stall every stream of the device; a thin binding from C, Rust or
// ctypes has no tensor library to allocate scratch from. The ordinary entry
// point (mxb_paged_attention_decode) wants a scratch buffer from its caller;
// this one brings its own, a fixed array inside the library.
//
// Limits and rules:
//  * The scratch is MXB_NOALLOC_SCRATCH_BYTES (16 MiB) of device memory per
//    GPU that loads the library, held until the process exits.
//    rows * heads * splits * (head_dim + 2) * 4 bytes must fit, where
//    splits = ceil(longest_context / 128); a larger call is refused with
//    cudaErrorInvalidValue (1) and a message on stderr, and nothing runs.
//  * The first call on each device looks up the array's device address
//    (with that device current). Make that first call outside any stream
//    capture.
//  * All calls share the one array, and it keeps what the last call left.
//    Nothing in it has to start at zero: every value a call reads it has
//    written itself. Two calls that overlap on the GPU (different streams)
//    race on it; keep calls on one stream or order them with events.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
//
// Arguments and result are those of mxb_paged_attention_decode without the
// scratch pointer: q and out [tokens, heads, head_dim], cache
// [pages, 2, kv_heads, page_tokens, head_dim], block_tables
// [requests, max_pages] int32, row_token / row_request [rows] int32 (a
// negative row_token is a padding row), positions [tokens] int32; dtype 0 is
// float32, 1 is bfloat16; status is a device int32 the kernels OR error bits
// into. Returns a cudaError_t value, 0 on success.
#pragma once

#include <cuda_runtime.h>

#define MXB_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int mxb_paged_attention_decode_noalloc(const void* q, const void* cache, void* out,
                                       const int* block_tables, int max_pages, const int* row_token,
                                       const int* row_request, const int* positions, int rows,
                                       int heads, int kv_heads, int head_dim, int page_tokens,
                                       int num_pages, int longest_context, int window, float scale,
                                       int dtype, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
