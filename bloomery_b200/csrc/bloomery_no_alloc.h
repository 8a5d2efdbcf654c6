/* Entry points of libbloomery_cuda.so that allocate no memory at all.
 *
 * This header has no counterpart in the reference project (midagedev/bloomery): there,
 * every scratch buffer belongs to the engine that calls the kernel.  It exists for callers
 * that are not allowed to allocate device memory when they need the kernel: a process
 * whose device memory was planned and handed out in full at start-up, a latency-critical
 * loop in which cudaMalloc (which synchronises the device) is off limits, or an embedding
 * host that passes in its input and output buffers and nothing more.
 */
#ifndef BLOOMERY_NO_ALLOC_H
#define BLOOMERY_NO_ALLOC_H

#include <stdint.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Split-K decode attention over a paged f16 KV cache, exactly bl_flash_decode, except
 * that the per-segment partial results are kept in a device array that is part of the
 * library image (about 4.1 MiB on every GPU that loads the library, until exit) instead
 * of caller-provided scratch.  The caller passes only inputs and outputs.
 *
 *   q           [M, n_q, head] fp32, already scaled by 1/sqrt(head)
 *   k_cache,
 *   v_cache     [n_pages, n_kv, 64, head] f16
 *   row_pos     [M]  position of each row (the row sees keys 0..row_pos)
 *   row_seq     [M]  sequence of each row in block_table, < 0 = skip the row
 *   block_table [*, max_pages] page of positions 64 i .. 64 i + 63
 *   out         optional [M, n_q * head] fp32
 *   outq, outds q8 form of the result: int8 [M, n_q * head], {d, d*sum} fp32 per 32 values
 *   fault       optional device word lowered to (layer << 8 | site) on bad input
 *
 * Limits: head is 64 or 128 and M * n_q * n_seg <= 8192; anything larger returns -5
 * (BL_ERR_LIMIT) and launches nothing.  Returns 0, a negative contract code, or a
 * positive cudaError_t.
 *
 * The first call on each device looks up the array's device address; make that call
 * outside any stream capture.  All calls share the one array, which keeps whatever the
 * previous call left in it (nothing in it needs clearing), so calls must not overlap on
 * the GPU: issue them on one stream, or order them yourself.
 * No cudaMalloc, cudaFree or allocating library routine is called, ever.
 */
int bl_flash_decode_static(const float* q, const void* k_cache, const void* v_cache, const int* row_pos,
                           const int* row_seq, const int* block_table, int max_pages, int n_pages, int head,
                           int n_q, int n_kv, int M, int n_seg, int ctx_limit, float* out, int8_t* outq,
                           float* outds, unsigned* fault, int layer, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BLOOMERY_NO_ALLOC_H */
