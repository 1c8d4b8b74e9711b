/* Split-key decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference project, whose attention
 * goes through a library call that allocates as it pleases.  It exists for
 * hosts that do all their device allocation up front and must not call an
 * allocator afterwards: a serving loop with a fixed memory plan where a late
 * cudaMalloc may synchronise the device or fail on a fragmented heap, or a
 * plug-in that runs inside another program's callback and is handed buffers but
 * no allocator.  Such a caller passes inputs and outputs as usual; the scratch
 * that the kernel needs between its two passes (partial outputs, maxima and
 * sums of every split) lives in a static array inside the library instead.
 *
 * - The array holds IE_NOALLOC_SCRATCH_FLOATS floats.  Every GPU that loads the
 *   library keeps that much memory until the process exits.
 * - A call needs ie_attention_decode_scratch_floats(n_tokens, n_heads, n_splits) words
 *   (16384 tickets + n_tokens * n_heads * n_splits * (head_dim + 2)) and is refused with
 *   IE_NOALLOC_TOO_LARGE when that exceeds the array.
 * - The first call on a device looks the array's device address up
 *   (cudaGetSymbolAddress) and remembers it; make that first call before any
 *   stream capture begins.  Later calls on the device only launch.
 * - All calls share the array and it keeps what the last call left.  Only the
 *   tickets at its start (one per request and kv head, counting the splits that
 *   have finished) have to be zero when a call starts: static device memory
 *   starts as zeros and every call that completes puts its tickets back to zero.
 *   Everything else is written before it is read.  Two calls that overlap on the
 *   GPU (different streams) race on the array; keep calls on one device in one
 *   stream or order them yourself.
 * - No cudaMalloc, cudaFree or allocating library routine is called.
 * - As with ie_attention_decode, a request takes part only if it brings at most 16
 *   rows (its tokens times the query heads per kv head): the rows of `out` that belong
 *   to a larger request are left untouched, and a model with more than 16 query heads
 *   per kv head is refused (-2).
 *
 * Arguments are those of ie_attention_decode without its scratch pointer; the
 * head size is the one the library was built for (ie_attention_mma_head_dim()).
 * Returns 0, a positive cudaError_t, or a negative refusal code.
 */
#pragma once
#include <cuda_runtime.h>

#define IE_NOALLOC_SCRATCH_FLOATS (1u << 20) /* 4 MiB per device */
#define IE_NOALLOC_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

int ie_attention_decode_noalloc(const void* q, void* out, const void* kpool, const void* vpool,
                                const int* block_table, const int* q_start, const int* ctx_before, int q_stride,
                                int out_stride, int table_stride, int n_requests, int n_tokens, int n_heads,
                                int n_kv_heads, int hd, int page_size, int window, float scale, int n_splits,
                                int split_keys, cudaStream_t stream);

/* Floats of scratch the static array offers (IE_NOALLOC_SCRATCH_FLOATS). */
long long ie_attention_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
