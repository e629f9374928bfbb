/* Split-KV decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in orielhaim/FeLLM; it exists for embedding this library.
 *
 * Who needs it: a host program that took all device memory for its own arena when it started, a
 * process running under a hard device-memory cap, or code on a path where cudaMalloc / cudaFree are
 * unwelcome because they synchronise the whole device.  The ordinary entry point
 * (fellm_attn_decode_mma in attention_mma.cu) wants a scratch buffer and a counter array from its
 * caller; this one brings its own, as arrays of fixed size inside the library image.  Every GPU
 * that loads the library holds them until the process exits:
 *
 *     scratch   FELLM_STATIC_SCRATCH_FLOATS  float32  (4 MiB)
 *     counters  FELLM_STATIC_COUNTERS        int32    (16 KiB)
 *
 * It calls no cudaMalloc, cudaFree or allocating library routine.  Inputs and outputs are still the
 * caller's.  A launch needs T*H*max_splits*(head_dim+2) scratch floats and T*G counters; a launch
 * that needs more is refused: the function returns FELLM_STATIC_TOO_LARGE and writes the reason into
 * `err`.
 *
 * First call on a device: looks up the device addresses of the two arrays (cudaGetSymbolAddress,
 * with that device current) and raises the kernel's shared-memory limit.  Make that first call
 * before any stream capture on the device.
 *
 * The arrays are shared by all calls on a device and keep what the last call left in them.  The
 * counters must start at zero, so every call clears the ones it uses (a cudaMemsetAsync on
 * `stream`) before its kernel; the scratch records are written before they are read.  Two calls
 * that overlap on the GPU (different streams, no ordering between them) race on the arrays: order
 * them.
 *
 * Key ranges: row t reads the keys 0..positions[t] (the last `window` of them if window > 0) in
 * ranges of `split_len` keys, one CTA per (range, kv head, row); the grid has `max_splits` ranges.
 * Choose max_splits >= ceil((largest position + 1) / split_len), so that every range has a CTA of
 * its own.  With fewer, the last range takes all the keys behind it: the result is the same, the
 * launch slower.  More ranges than a row needs cost nothing but scratch.
 *
 * Arguments as fellm_attn_decode_mma, without the scratch and counters; the library is compiled for
 * one head size (-DHD=...) and refuses any other.  Returns 0, a positive cudaError_t, or a negative
 * code (FELLM_ERR_SIZE -1, FELLM_ERR_ARG -2, FELLM_STATIC_TOO_LARGE -3).
 */
#pragma once
#include <cuda_runtime.h>

#define FELLM_STATIC_SCRATCH_FLOATS (1 << 20)
#define FELLM_STATIC_COUNTERS (1 << 12)
#define FELLM_STATIC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C"
#endif
int fellm_attn_decode_static(const void* q, const void* pool, const int* block_table, int max_pages,
                             const int* positions, const int* row_slot, void* out, int T, int H, int G,
                             int hd, int page_tokens, int layer, int layers_in_group, float scale, int window,
                             int split_len, int max_splits, cudaStream_t stream, char* err, int err_len);
