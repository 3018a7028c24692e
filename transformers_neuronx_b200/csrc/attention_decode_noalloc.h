// tnx_attention_decode_noalloc: decode attention that allocates nothing.
//
// This entry point has no counterpart in aws-neuron/transformers-neuronx.  It is for callers of
// this library that cannot call cudaMalloc (or any allocating routine, torch's included) at the
// moment they need the kernel:
//   * a serving process that handed all free device memory to its cache pool at start-up, so that
//     a later allocation may simply fail;
//   * a latency-critical loop in which an allocation's implicit device synchronisation is not
//     acceptable;
//   * a host that loads this library through its C symbols from another runtime and has no
//     allocator of this package's to lean on.
// The split-KV form of the kernel needs scratch memory (32-bit partial results and one counter per
// (row, head)); here that scratch is a pair of file-scope device arrays inside the library, so the
// caller passes inputs and outputs only.
//
// Limits and rules:
//   * n_rows * n_heads * n_splits * (head_dim + 2) <= TNX_NOALLOC_MAX_FLOATS and
//     n_rows * n_heads <= TNX_NOALLOC_MAX_COUNTERS when n_splits > 1; beyond that the call returns
//     -2.  With n_splits == 1 no scratch is used and only the kernel's own size rules apply.  Every
//     refusal (a size, an alignment, a count that is not positive) leaves its reason in
//     tnx_attention_decode_noalloc_last_error(), and a refused call queues nothing on the stream.
//   * n_splits * pages_per_split pages must cover the longest context among the rows: the kernel
//     reads positions on the device and cannot refuse a plan that is too short; keys beyond the
//     plan would be left out.
//   * Every GPU that loads the library holds the arrays (about 4.1 MB) until the process exits.
//   * The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress, with
//     that device current).
//   * All calls share the arrays: two calls that overlap on the GPU (on different streams) race on
//     them.  Calls on one stream are safe; the counters are cleared at the start of every call.
//   * Arguments are those of tnx_attention_decode without the scratch and counter pointers.
#pragma once
#include <cuda_runtime.h>

#define TNX_NOALLOC_MAX_FLOATS (1 << 20)     /* 4 MiB of 32-bit partials */
#define TNX_NOALLOC_MAX_COUNTERS (1 << 14)   /* 64 KiB of counters */

#define TNX_NOALLOC_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

TNX_NOALLOC_API int tnx_attention_decode_noalloc(const void* q, int q_stride, const void* cache, const int* block_tables,
                                 int bt_stride, const int* rows, const int* token_request, const int* positions,
                                 void* out, int out_stride, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                 int page_size, int window, float scale, int n_splits, int pages_per_split,
                                 cudaStream_t stream);

/* Text of the last refusal on the calling thread ("" after a successful call). */
TNX_NOALLOC_API const char* tnx_attention_decode_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
