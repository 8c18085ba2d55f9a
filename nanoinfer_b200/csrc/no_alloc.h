// Entry points of libnanoinfer_b200.so that allocate no memory of any kind.
//
// This header has no counterpart in the reference (AustinJiangg/nanoinfer): its CUDA backend hands
// every kernel output and scratch buffer out of a caching device pool that grows with cudaMalloc
// (cpp/src/cuda/cuda_runtime.cu:43-108).
//
// Who needs this: code that runs where a device allocation is not possible or not allowed. Examples
// are a caller inside a region in which the allocator must not be entered (a real-time serving loop
// that has promised not to take the allocator's lock, a callback running on a driver thread, a
// process whose memory budget was handed out in full at start-up), and hosts that are not Python at
// all and so have no torch allocator to lend. The other entry points of this library take their
// scratch memory from the caller; for the split decode attention that scratch is an extra buffer the
// caller would have to allocate per call. The function below needs none: its scratch is an array that
// is part of the library image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of the built-in scratch array. Every GPU that loads the library holds this much device memory
// from load until the process exits, whether or not the function is ever called.
#define NIB_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)

// Attention of single decoded tokens over the paged cache, keys split over `splits` CTAs per
// (token, kv head) and merged in split order: the same kernels, arguments and results as
// nib_attention_decode_mma, except that the partial results live in the library's own scratch array.
//
// Needs n_tokens * heads * splits * (head_dim + 2) * 4 bytes of scratch; a call that needs more than
// NIB_NOALLOC_SCRATCH_BYTES is refused (returns non-zero; nib_last_error() says by how much) and
// launches nothing. The caller still provides every input and the output.
//
// * The first call on a device looks up the device address of the scratch array
//   (cudaGetSymbolAddress, with that device current) and remembers it; make that first call before
//   any stream capture begins on that device.
// * All calls share the one array, and it keeps whatever the last call left. Nothing in it has to be
//   zero: each call overwrites every element it later reads. Two calls that run on the GPU at the
//   same time (different streams, different host threads) race on it: order them.
// * It calls no cudaMalloc, cudaFree or allocating library routine, on any call.
int nib_attention_decode_noalloc(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                 const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                 const void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                 int head_dim, float scale, int window, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
