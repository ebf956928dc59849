/* Allocation-free C entry point for paged GQA decode attention.
 *
 * This entry point has no counterpart in the reference (huangyibo/SkyGDR), which
 * has no paged attention and no C API at all.
 *
 * Who it is for: callers that must not, or cannot, allocate device memory at the
 * moment they need attention. Examples: a serving loop whose HBM is already owned
 * to the last byte by another allocator (a cudaMalloc there fails or evicts), code
 * that runs where an implicit device synchronisation is unacceptable (cudaMalloc
 * and cudaFree synchronise), and plug-ins written in C or another language that
 * load this library with dlopen and have no tensor library to hand out scratch.
 * The regular Python path (skygdr_b200.ops.PagedAttention) lets torch allocate the
 * split-KV scratch; this one keeps that scratch in a fixed array inside the library.
 *
 * What the scratch is: split-KV partial outputs and their softmax statistics, one
 * arrival counter per (sequence, kv head) and a small status block. It lives in a
 * file-scope device array of SKYGDR_NOALLOC_SCRATCH_BYTES bytes. Every GPU on which
 * a process loads this library holds that array until the process exits.
 *
 * Limits (a call beyond them is rejected with SKYGDR_NOALLOC_E_TOO_LARGE and a
 * message, and launches nothing):
 *     batch * q_heads * ceil(max_ctx / chunk_tokens) <= SKYGDR_NOALLOC_MAX_ROWS
 *     batch * kv_heads                               <= SKYGDR_NOALLOC_MAX_PAIRS
 *
 * First call on a device: looks up the device address of the array (once per
 * device, with that device current) before launching. Make this first call before
 * any stream capture begins on that device.
 *
 * Sharing: every call on a device uses the same array, and the array keeps what the
 * last call left. The entry point clears the parts that must start at zero (the
 * counters and the status block) on `stream` before the kernel. Two calls that
 * overlap on the GPU (different streams, no ordering between them) race on the
 * scratch and give wrong results; order them on one stream or with events.
 *
 * The function calls no cudaMalloc, cudaFree, nor any allocating library routine.
 */
#ifndef SKYGDR_PAGED_ATTN_NOALLOC_H
#define SKYGDR_PAGED_ATTN_NOALLOC_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKYGDR_NOALLOC_MAX_ROWS 16384   /* (sequence, query head, split) triples */
#define SKYGDR_NOALLOC_MAX_PAIRS 4096   /* (sequence, kv head) pairs */
/* partial outputs (128 floats per row) + two statistics per row + counters + status block */
#define SKYGDR_NOALLOC_SCRATCH_BYTES (SKYGDR_NOALLOC_MAX_ROWS * 130 * 4 + SKYGDR_NOALLOC_MAX_PAIRS * 4 + 256)

#define SKYGDR_NOALLOC_OK 0
#define SKYGDR_NOALLOC_E_TOO_LARGE -1   /* sizes beyond the limits above */
#define SKYGDR_NOALLOC_E_BAD_ARG -2     /* null pointer, unsupported geometry */
#define SKYGDR_NOALLOC_E_CUDA -3        /* a CUDA call failed; the message names it */

/* q, out: [batch][q_heads][128] bf16. kv_layer: first page of the layer in a head-major paged pool
 * (page of one head = 16 tokens x 128 bf16, contiguous); strides in elements. block_table:
 * [batch][max_blocks] int32, ctx_lens: [batch] int32, all device pointers on the current device.
 * chunk_tokens: tokens per CTA, a multiple of 64. stream: a cudaStream_t (may be 0).
 * err / err_len: optional buffer that receives a one-line message on failure.
 * Returns SKYGDR_NOALLOC_OK or a negative code. */
int skygdr_paged_attn_decode_noalloc(const void* q, const void* kv_layer, void* out, const int* block_table, const int* ctx_lens,
                                     long long block_stride, long long kv_stride, long long head_stride, int batch, int q_heads,
                                     int kv_heads, int max_blocks, int max_ctx, int chunk_tokens, float scale, void* stream,
                                     char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif
