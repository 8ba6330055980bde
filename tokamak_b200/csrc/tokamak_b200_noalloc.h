/* Entry points of libtokamak_b200 that allocate nothing.
 *
 * This header has no counterpart in WeichunK/tokamak: the reference is Python over
 * PyTorch and leaves every allocation to PyTorch's caching allocator.
 *
 * Who needs this.  The library's C interface can be driven without PyTorch, from a
 * C or C++ serving loop.  Such a caller usually sizes the cache's page pool to
 * whatever memory the device has left once the weights are loaded, so a cudaMalloc
 * in the middle of serving may simply fail; and cudaMalloc and cudaFree synchronise
 * the whole device, which stalls the copies and kernels that the caller has queued
 * on its other streams.  A caller that has handed all device memory to its own pool,
 * or that must not stall, therefore cannot allocate the scratch buffer which
 * tk_attention_decode expects.  For it, the scratch lives inside the library.
 */
#ifndef TOKAMAK_B200_NOALLOC_H
#define TOKAMAK_B200_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error codes beyond cudaError_t (which are positive). */
#define TK_NOALLOC_TOO_LARGE (-2)   /* the call needs more scratch than the library holds */
#define TK_NOALLOC_BAD_DEVICE (-3)  /* the current device has an index the table does not cover */

/* Floats of scratch the library holds on every GPU that loads it (4 MiB), until exit. */
long long tk_attention_decode_noalloc_capacity_floats(void);

/* Human-readable text for a code returned by tk_attention_decode_noalloc. */
const char* tk_noalloc_error_string(int code);

/* Split-K paged decode attention, identical to tk_attention_decode except that the
 * caller passes no scratch: partial results go to a static array in device memory.
 *
 *  - Calls no cudaMalloc, cudaFree or other allocating routine.
 *  - Needs n_items * n_q_heads * n_splits * (head_dim + 2) floats of scratch and
 *    n_items * n_kv_heads arrival counters (the library holds 4096); a call that needs more
 *    than the capacity returns TK_NOALLOC_TOO_LARGE and launches nothing (use fewer splits,
 *    or fewer items per call).  A call with n_splits == 1 uses neither array and has no limit.
 *  - Host threads: the one-time lookup is guarded by a mutex, so threads may call at the same
 *    time as far as the host is concerned; what the next point says about the GPU still holds.
 *  - The first call on a device looks up the array's device address (once per device,
 *    with that device current).  Make that first call outside any stream capture.
 *  - All calls share the arrays, and they keep what the last call left in them.  The
 *    partial results need no clearing: every split writes its result (an empty split
 *    writes a zero sum) before the block that merges reads any.  The arrival counters must
 *    be zero at the start of a call: they are zero when the library is loaded, and the
 *    merging block puts each counter back to zero, so a call that ran to its end leaves
 *    them ready for the next.  Two calls whose kernels overlap on the GPU (different
 *    streams, no ordering between them) race on the arrays; order them on one stream or
 *    with events.
 */
int tk_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                const int* items, const int* positions, const int* tok_req,
                                const int* req_slot, const int* block_table, int* err, int n_items,
                                int n_reqs, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                int max_pages, int num_pages, int window, int n_splits, float scale,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
