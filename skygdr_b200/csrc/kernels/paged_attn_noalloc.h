/* Allocation-free C entry points for paged GQA decode attention.
 *
 * These entry points have no counterpart in the reference (huangyibo/SkyGDR), which
 * has no paged attention and no C API at all.
 *
 * Who they are for: callers that must not, or cannot, allocate device memory at the
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
 * file-scope device array of SKYGDR_NOALLOC_SCRATCH_BYTES bytes (about 8.5 MB).
 *
 * When that memory is taken. The CUDA runtime loads a library's device code lazily
 * (the default since CUDA 12.2): the array does not exist on a GPU until the first
 * runtime call that needs this module on that GPU. That call is the symbol lookup
 * inside skygdr_paged_attn_noalloc_init(), or inside the first
 * skygdr_paged_attn_decode_noalloc() on the device if init was not called. The
 * module load reserves the array's 8.5 MB, may synchronise the device, and can
 * fail with an out-of-memory error when no HBM is left. So a caller that is about
 * to hand all HBM to its own allocator, or that cannot tolerate a synchronisation
 * later, calls skygdr_paged_attn_noalloc_init() once per device at start-up, with
 * that device current, before the memory is given away and before any stream
 * capture. After it has returned SKYGDR_NOALLOC_OK on a device, the attention entry
 * point on that device calls no cudaMalloc, cudaFree, nor any allocating library
 * routine, and loads nothing. From then on every GPU that went through init holds
 * the array until the process exits.
 *
 * Limits (a call beyond them is rejected with SKYGDR_NOALLOC_E_TOO_LARGE and a
 * message, and launches nothing):
 *     batch * q_heads * ceil(max_ctx / chunk_tokens) <= SKYGDR_NOALLOC_MAX_ROWS
 *     batch * kv_heads                               <= SKYGDR_NOALLOC_MAX_PAIRS
 *
 * Sharing: every call on a device uses the same array, and the array keeps what the
 * last call left. The entry point clears the parts that must start at zero (the
 * counters and the status block) on `stream` before the kernel. Two calls that
 * overlap on the GPU (different streams, no ordering between them) race on the
 * scratch and give wrong results; order them on one stream or with events.
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

/* Kernel status codes reported by skygdr_paged_attn_noalloc_status (0 = the kernel ran to the end). */
#define SKYGDR_NOALLOC_KERNEL_OK 0
#define SKYGDR_NOALLOC_KERNEL_BAD_INDEX 4     /* a context length beyond max_ctx / the table row, or a block id >= num_blocks:
                                                 the value was cut or replaced (nothing outside the pool was read) and the
                                                 affected sequence's output is wrong; detail = 0x40000000 | sequence for a
                                                 length, (sequence << 16) | page for a block id */
#define SKYGDR_NOALLOC_KERNEL_TIMEOUT 5       /* a bounded wait on a copy gave up; `out` is incomplete */

/* One-time set-up on the current device: loads this library's device code there (which reserves the scratch array, see
 * "When that memory is taken" above), looks up the array's device address and prepares the kernels for the four supported
 * query-group sizes. Idempotent and thread-safe. Call it at start-up, before HBM is handed to another allocator and before
 * any stream capture; skygdr_paged_attn_decode_noalloc does the same on its first call on a device if this was skipped. */
int skygdr_paged_attn_noalloc_init(char* err, size_t err_len);

/* q, out: [batch][q_heads][128] bf16. kv_layer: first page of the layer in a head-major paged pool
 * (page of one head = 16 tokens x 128 bf16, contiguous); strides in elements. block_table:
 * [batch][max_blocks] int32, ctx_lens: [batch] int32, all device pointers on the current device.
 * q_heads / kv_heads must be 1, 2, 4 or 8. max_ctx: upper bound of ctx_lens, at most max_blocks * 16.
 * num_blocks: number of blocks in the pool counted from kv_layer's block 0; block ids in the table are checked against
 * it on the device (0 = unknown, no check). chunk_tokens: tokens per CTA, a multiple of 64. stream: a cudaStream_t (may be 0).
 * err / err_len: optional buffer that receives a one-line message on failure.
 * Returns SKYGDR_NOALLOC_OK once the work is enqueued, or a negative code (then nothing was enqueued). What the kernel
 * itself met (a bad length or block id, a wait that gave up) is read with skygdr_paged_attn_noalloc_status. */
int skygdr_paged_attn_decode_noalloc(const void* q, const void* kv_layer, void* out, const int* block_table, const int* ctx_lens,
                                     long long block_stride, long long kv_stride, long long head_stride, int batch, int q_heads,
                                     int kv_heads, int max_blocks, int num_blocks, int max_ctx, int chunk_tokens, float scale,
                                     void* stream, char* err, size_t err_len);

/* Status that the kernel of the LAST skygdr_paged_attn_decode_noalloc call on the current device left in the scratch:
 * *code is one of SKYGDR_NOALLOC_KERNEL_*, *detail is code-specific. `stream` must be the stream of that call: the status
 * is copied out behind it and the function waits for the stream, so it returns the finished call's status. code and detail
 * are host pointers (detail may be null). Allocates nothing. Returns SKYGDR_NOALLOC_OK, or a negative code if the device
 * was never initialised or a CUDA call failed. */
int skygdr_paged_attn_noalloc_status(unsigned int* code, unsigned int* detail, void* stream);

#ifdef __cplusplus
}
#endif
#endif
