/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in YuvGev00/mini-engine; it is an addition of this
 * library.
 *
 * Who needs it.  The split decode kernel writes per-split partial results (a maximum, a sum
 * and an unnormalised output row per head) to scratch memory before a second kernel merges
 * them.  The engine takes that scratch from its workspace.  Some callers have no allocator to
 * take it from and may not call cudaMalloc at that point: code that runs between other
 * libraries' launches under a fixed memory budget, a plug-in inside a host process that owns
 * all device memory, or a latency-critical loop in which an allocation (which may synchronise
 * the device) is not acceptable.  For them the scratch is a fixed array inside this library.
 *
 * What it does.  Exactly what me_attention_decode_bf16 does for the same arguments (every
 * entry brings one query token; see attention_bf16.cu), with the partial results kept in a
 * file-scope device array instead of a caller-supplied buffer.  It calls no cudaMalloc,
 * cudaFree or other allocating routine.  Inputs and outputs are still the caller's.
 *
 * Limits and rules.
 *  - entries * heads * max_splits * (head_dim + 2) must not exceed
 *    ME_NOALLOC_MAX_PARTIAL_FLOATS (2,097,152 floats = 8 MiB); otherwise the call returns
 *    ME_ERR_NOALLOC_TOO_LARGE and launches nothing.  max_splits must cover the longest
 *    context of the call: ceil(context / 128).  The host cannot check that (the context
 *    lengths are on the device); a context that needs more is computed without its keys
 *    beyond 128 * max_splits, never reads or writes outside its own slots, and makes
 *    me_attention_bf16_take_error report 2.  Example: 16 requests x 32 heads x 30 splits
 *    (3,840 tokens of context) x head_dim 128 = 1,996,800 floats.
 *  - Every GPU on which the library is loaded holds the 8 MiB until the process exits.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress,
 *    with that device current) and keeps it; make that first call before any stream capture.
 *    Device ordinals 0..ME_NOALLOC_MAX_DEVICES-1 are served.
 *  - All calls share the one array, which keeps whatever the last call left in it.  Nothing
 *    in it has to start at zero: the merge kernel reads only the partials that the same call
 *    wrote.  Two calls that overlap on the GPU (different streams, or captured into graphs
 *    that run concurrently) race on it; run them on one stream or otherwise in order.
 *  - Return value: 0, a cudaError_t value, or one of the ME_ERR_* codes below.
 */
#ifndef MINI_ENGINE_B200_ATTENTION_BF16_NOALLOC_H
#define MINI_ENGINE_B200_ATTENTION_BF16_NOALLOC_H

#include <cuda_runtime.h>

#define ME_NOALLOC_MAX_PARTIAL_FLOATS (2 * 1024 * 1024)
#define ME_NOALLOC_MAX_DEVICES 64
#define ME_ERR_NOALLOC_TOO_LARGE 1003

#ifdef __cplusplus
extern "C" {
#endif

int me_attention_decode_bf16_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     const int* cu_tokens, const int* context_lens, void* out, float scale,
                                     int entries, int max_splits, int heads, int kv_heads, int head_dim,
                                     int page_size, int table_width, int window, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif
