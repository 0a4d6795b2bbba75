/* An entry point that allocates nothing.  It has no counterpart in EmersonDowell/AIR.
 *
 * Who it is for: code that may launch kernels but may not obtain device memory at the moment
 * of the call.  Examples are a host program that hands this library a fixed arena and forbids
 * any further cudaMalloc (memory budgets fixed at start-up, other processes sharing the GPU), a
 * caller in the middle of a latency-critical loop where an allocation could block or fail, and
 * a plug-in that runs inside another runtime which owns all allocations.  The split-KV decode
 * attention normally needs scratch memory for the partial results of its splits; the ordinary
 * entry point (air_decode_attention) takes that scratch from its caller, who has to allocate it.
 * This one keeps it inside the library instead.
 *
 *   int air_decode_attention_static(q, cache, block_table, max_blocks, token_seq, positions, out,
 *                                   T, H, K, D, P, window, scale, splits, stream);
 *
 * Arguments and result are those of air_decode_attention without the two scratch pointers: the
 * caller still passes the inputs (q [T,H,D] bf16, cache [page,2,K,P,D] bf16, block_table
 * [slots,max_blocks] int32, token_seq [T], positions [T]) and the output (out [T,H,D] bf16), all
 * device pointers.  Sizes that the kernel does not take (a head size other than 64, 128, 256, heads
 * that are no multiple of the kv heads, a page size that is no multiple of 16) are AIR_ERR_BAD_ARGUMENT
 * (100001) whatever scratch they would need.  It returns 0, a cudaError_t, or one of the AIR_ERR_* codes;
 * air_decode_attention_static_error(code) gives the text.
 *
 * The scratch is a file-scope device array of AIR_STATIC_SCRATCH_FLOATS floats (8 MiB) that every
 * GPU which loads the library holds until the process exits.  A call needs
 * T * H * splits * (D + 2) floats of it when splits > 1 (air_decode_attention_static_need) and
 * nothing otherwise; a call that needs more is refused with AIR_ERR_STATIC_SCRATCH and launches
 * nothing.  For scale: 64 tokens x 28 heads x 8 splits x 130 = 1.9 M floats fits.
 *
 * The function calls no cudaMalloc, no cudaFree and no library routine that allocates.  The first
 * call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current) and keeps it; make that first call outside any stream capture.
 *
 * All calls share the one array, and it keeps what the last call left in it.  Nothing in it has to
 * be zero at the start of a call: for every token that is not padding (token_seq >= 0) the first
 * kernel of a call writes every entry that its second kernel uses; for a padding token the second
 * kernel reads what an earlier call left there and stores nothing.  But two calls whose kernels may overlap on the GPU (different streams, or
 * different host threads without ordering) race on the array and corrupt each other's results:
 * run them in one stream, or order them with events.
 */
#pragma once

#include <cuda_runtime.h>

#define AIR_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define AIR_ERR_STATIC_SCRATCH 100002

#ifdef __cplusplus
extern "C" {
#endif

int air_decode_attention_static(const void* q, const void* cache, const int* block_table, int max_blocks,
                                const int* token_seq, const int* positions, void* out, int T, int H, int K, int D,
                                int P, int window, float scale, int splits, cudaStream_t stream);
long long air_decode_attention_static_capacity(void);
long long air_decode_attention_static_need(int T, int H, int D, int splits);
const char* air_decode_attention_static_error(int code);

#ifdef __cplusplus
}
#endif
