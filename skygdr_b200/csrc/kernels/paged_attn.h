// Host-visible parameters of the paged GQA decode attention kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace sky {
struct LaunchStatus;

struct PagedAttnParams {
    const __nv_bfloat16* q;       // [batch][q_heads][128]
    const __nv_bfloat16* kv;      // base of this layer's pages inside the pool
    __nv_bfloat16* out;           // [batch][q_heads][128]
    const int* block_table;       // [batch][max_blocks]
    const int* ctx_lens;          // [batch]
    long long block_stride;       // elements between consecutive blocks of the pool
    long long kv_stride;          // elements from a block's K page to its V page
    long long head_stride;        // elements between kv heads inside a page (= 16*128)
    int batch, q_heads, kv_heads, head_dim, block_tokens, max_blocks;
    int num_blocks;               // blocks in the pool from `kv` on (0 = unknown: block ids are not checked by the CUDA-core kernel)
    int max_ctx;                  // upper bound of ctx_lens (sizes the grid)
    int chunk_tokens;             // tokens per CTA (multiple of 64)
    int max_splits;               // row pitch of the scratch arrays
    float scale;
    // scratch for split-KV: partial outputs and their softmax statistics, plus one counter per (seq, kv head)
    float* part_o;                // [batch][q_heads][max_splits][128]
    float* part_m;                // [batch][q_heads][max_splits]
    float* part_l;                // [batch][q_heads][max_splits]
    unsigned int* counters;       // [batch][kv_heads], zero before the first launch; the kernel re-zeroes them
    LaunchStatus* status;
};

cudaError_t launch_paged_attn_decode(const PagedAttnParams& p, cudaStream_t stream);
// Per-device set-up that the launcher otherwise does on its first call for each query-group size (1, 2, 4, 8): loads the
// kernels on the current device and raises their shared-memory limits. For callers that want it done at start-up.
cudaError_t prepare_paged_attn_decode();
// Tensor-core version (paged_attn_tc.cu). pool_rows: 128-element rows from p.kv to the end of the pool allocation;
// chunk_tokens must be a multiple of 128.
int paged_attn_tc_page_box();
cudaError_t launch_paged_attn_decode_tc(const PagedAttnParams& p, long long pool_rows, cudaStream_t stream);
}  // namespace sky
