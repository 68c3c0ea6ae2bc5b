// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Deyu-Kong/mini-infer allocates with
// cudaMalloc wherever it needs a buffer, e.g. src/kernels/rope_kernel.cu:113-128); it exists for
// users of this library who cannot do that:
//   * code that runs where allocation is forbidden or must not happen - inside a real-time or
//     latency-critical loop (cudaMalloc and cudaFree synchronise the device), in a callback that
//     the driver runs, in a process whose device-memory budget was fixed at start-up;
//   * hosts that embed the kernels without PyTorch (the engine itself takes its scratch from
//     PyTorch's allocator) and have no allocator of their own to hand scratch from.
//
// mi_attn_decode_noalloc computes exactly what mi_attn_decode computes (split-KV attention of one
// query token per request over the paged cache, then the merge of the splits), but keeps the
// per-split partial results in a buffer that is part of the library image: a file-scope
// `static __device__` array of MI_ATTN_NOALLOC_SCRATCH_BYTES bytes.  Every GPU on which the
// library is loaded holds that array from load until the process exits.
//
// Rules of use
//   * Sizes: B * nh * max_splits * (d + 2) floats must fit the array; a larger problem is refused
//     with kBadShape (-2) and a message from mi_last_error(), never computed partially.
//   * max_splits must be at least ceil(longest kv_len / mi_attn_decode_split_size()) (splits of 512
//     keys).  The lengths are device data that the host cannot check: with a smaller max_splits the
//     kernels stay inside the array but attend over fewer keys than the request has.
//   * First call on a device: looks up the device address of the array (cudaGetSymbolAddress,
//     with that device current) and remembers it.  Make that first call before any stream
//     capture begins on that device; later calls only launch kernels.
//   * The call allocates nothing and frees nothing, on the host or on the device: no cudaMalloc,
//     cudaFree, or library routine that allocates.
//   * All calls on a device share the one array.  Nothing in it has to be cleared between calls:
//     every partial the merge step reads was written by the split step of the same call.  Two
//     calls whose kernels may overlap on the GPU (different streams, no ordering between them)
//     race on it: order them.
//
// Arguments are those of mi_attn_decode without the two scratch pointers; q, caches and out are
// device pointers of element type `adtype` (0 = float, 1 = bfloat16); block_table, q_start and
// kv_len are device int32 arrays.  Returns 0 when the kernels were queued on `stream`.
#pragma once

#include <cuda_runtime.h>

#define MI_ATTN_NOALLOC_SCRATCH_BYTES (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int mi_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, int adtype,
                           const int* block_table, const int* q_start, const int* kv_len, void* out, int B,
                           int nh, int nkv, int d, int page_size, int max_pages, int max_splits, int window,
                           float scale, cudaStream_t stream);

// Bytes of the built-in scratch array (MI_ATTN_NOALLOC_SCRATCH_BYTES).
unsigned int mi_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
