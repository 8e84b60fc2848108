/* agave_b200_no_alloc.h: decode attention for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference engine (maci0/agave);
 * it exists for users of this library only.
 *
 * Who needs it.  The regular decode attention (agv_attention_decode) takes its
 * scratch buffers from the caller, and the Python layer gets them from torch's
 * allocator.  Some programs that link this library have no allocator to ask and
 * may not call cudaMalloc themselves:
 *   - a serving process that hands the whole device to one arena at start-up,
 *     so that any later cudaMalloc fails for lack of memory;
 *   - a latency-critical loop that runs beside other streams: cudaMalloc and
 *     cudaFree synchronise the device and would stall those streams;
 *   - a host written in C or another language that loads the shared library
 *     directly and brings only its inputs and outputs.
 * For them the scratch lives inside the library, in one fixed array in device
 * memory (AGV_NO_ALLOC_SCRATCH_FLOATS 32-bit values, 16 MiB).  Every GPU on
 * which the library is loaded holds that array until the process exits.
 *
 * What it does.  The same computation as agv_attention_decode with the same
 * arguments, minus the two scratch pointers: one query token per batch entry
 * against the paged key/value cache.  It calls no cudaMalloc, cudaFree or other
 * allocating routine.
 *
 * Limits and rules.
 *   - The call is refused (negative return, message from agv_last_error) when
 *     B * nh * n_splits * (hd + 2) exceeds AGV_NO_ALLOC_SCRATCH_FLOATS, where
 *     n_splits is what agv_attention_decode_plan reports for max_keys.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call
 *     before any stream capture begins on that device.
 *   - Where many sequences or long contexts make the kernel fetch the cache's pages by
 *     TMA, the first call for a pair of pools encodes two tensor maps and keeps them in
 *     host memory (a host-side table; nothing on the device).
 *   - max_keys must be at least the number of keys any entry attends to
 *     (position + 1, or the window if that is smaller): it sizes the grid.  An
 *     entry with more keys gets no output from that call.  The call clears the
 *     arrival counters it uses before its kernel runs (a memset on the stream),
 *     so such a mistake does not reach later calls.
 *   - B times the number of head groups (nkv * ceil(nh / nkv / 4)) must not exceed
 *     AGV_NO_ALLOC_COUNTERS; the call is refused otherwise.
 *   - All calls share the one array and it keeps what the last call left.  The
 *     kernels write every value they later read, so nothing has to be cleared.
 *     The only thing that must start at zero is a small table of arrival
 *     counters beside the array: every call clears the ones it uses first.  Two calls that overlap on the
 *     GPU (different streams, no ordering between them) race on both.  Order
 *     them, e.g. by using one stream.
 */
#ifndef AGAVE_B200_NO_ALLOC_H
#define AGAVE_B200_NO_ALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AGV_NO_ALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define AGV_NO_ALLOC_COUNTERS 65536

/* dtype: 0 = float32, 1 = bfloat16 (of q, out and the cache pools).
 * Returns 0, or a negative code with a message in agv_last_error(). */
int agv_attention_decode_static(const void* q, long long q_stride, void* out, int dtype,
                                const void* k_pool, const void* v_pool, const int* page_table,
                                const int* slots, const int* positions, int max_pages, int page,
                                int cap, int B, int nh, int nkv, int hd, float scale, int window,
                                int max_keys, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
