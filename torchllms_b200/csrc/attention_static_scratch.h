/* Paged attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (normster/torchllms calls a library for
 * paged attention and lets that library own its workspace); it exists for embedders of this
 * library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits.  Examples are a host application
 * that has handed the whole device to another memory pool and gives this library no allocator;
 * a latency-critical loop in which the device-wide synchronisation that cudaMalloc / cudaFree
 * imply is not acceptable; and plug-ins that are called inside somebody else's stream and are
 * told not to touch the allocator.  The ordinary entry point, tl_paged_attention, expects the
 * caller to bring a float32 workspace whenever the key range is split over CTAs; this variant
 * brings its own: a fixed array that is part of the library image.
 *
 * The scratch
 *   - is a file-scope `static __device__` array of TL_STATIC_SCRATCH_FLOATS float32 values
 *     (8 MiB).  Every device that loads the library holds this much until the process exits.
 *   - is shared by every call on that device and keeps whatever the last call left in it.  The
 *     kernel writes every partial result it later reads, so nothing has to be cleared between
 *     calls; but two calls that overlap on the device (different streams, or one stream and a
 *     graph replay in flight) race on it.  Serialise them.
 *   - is found once per device: the first call on a device asks the runtime for the array's
 *     device address (cudaGetSymbolAddress, with that device current).  That first call should
 *     be made before any stream capture begins; later calls only launch kernels.
 *
 * Sizes: a step needs n_tokens * n_heads * n_splits * (head_dim + 2) floats, where n_splits is
 * what tl_attention_plan reports.  If that exceeds the array the call launches nothing and
 * returns TL_STATIC_SCRATCH_TOO_SMALL; tl_static_scratch_strerror() has the words for it.
 *
 * Arguments are those of tl_paged_attention without the workspace pointer; the caller still owns
 * q, the page tensors, the block table, the index arrays and the output.  Nothing in this call
 * allocates: no cudaMalloc, no cudaFree, no library routine that allocates.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TL_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TL_STATIC_SCRATCH_TOO_SMALL (-40)
#define TL_STATIC_SCRATCH_NO_ADDRESS (-41)

int tl_paged_attention_static_scratch(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* block_table, int table_stride, const int* q_start,
                                      const int* kv_len, int dtype, int n_tokens, int n_seqs, int n_heads,
                                      int n_kv_heads, int head_dim, int page_size, int max_q_len, int max_kv_len,
                                      int window, float scale, int allow_split, void* stream);

/* Text for the two codes above (and "ok" for 0); other codes are those of tl_paged_attention. */
const char* tl_static_scratch_strerror(int code);

#ifdef __cplusplus
}
#endif
