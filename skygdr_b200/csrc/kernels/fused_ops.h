// Small fused decoder ops (all bf16 in / bf16 out, fp32 math).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace sky {

// y = rmsnorm(x) * w. With `residual`: residual += x (in place, bf16) and y = rmsnorm(residual) * w.
cudaError_t launch_rmsnorm(const __nv_bfloat16* x, __nv_bfloat16* residual, const __nv_bfloat16* w, __nv_bfloat16* y,
                           int rows, int hidden, float eps, cudaStream_t stream);

struct RopeAppendParams {
    const __nv_bfloat16* qkv;      // [tokens][(q_heads + 2*kv_heads) * 128]
    const __nv_bfloat16* q_norm;   // [128] or nullptr
    const __nv_bfloat16* k_norm;   // [128] or nullptr
    __nv_bfloat16* q_out;          // [tokens][q_heads][128]
    __nv_bfloat16* kv;             // this layer's pages: head-major paged cache
    const float* inv_freq;         // [64] rotary inverse frequencies theta^(-i/64)
    const int* block_table;        // [seqs][max_blocks]
    const int* positions;          // [tokens] position of the token inside its sequence
    const int* seq_ids;            // [tokens] row of block_table; nullptr: token i belongs to sequence i
    long long block_stride, kv_stride, head_stride, tok_stride;  // head-major: (16*128, 128); token-major: (128, heads*128)
    int tokens, q_heads, kv_heads, max_blocks, block_tokens;
    float eps;
};
// Per-head RMSNorm of q and k, rotary embedding (half-rotation form), then q -> q_out and k,v -> paged cache.
cudaError_t launch_rope_append(const RopeAppendParams& p, cudaStream_t stream);

// out[r][c] = silu(gate_up[r][c]) * gate_up[r][F + c]
cudaError_t launch_silu_mul(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int rows, int ffn, cudaStream_t stream);
// out[t] = table[ids[t]] (ids outside the table are clamped to its ends)
cudaError_t launch_embedding(const int* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int tokens, int hidden, int vocab, cudaStream_t stream);
// Greedy sampling: out[r] = argmax_c logits[r][c] (lowest index wins ties).
cudaError_t launch_argmax(const __nv_bfloat16* logits, int* out, int rows, int vocab, long long row_stride, cudaStream_t stream);
// Temperature sampling: out[r] is drawn from softmax(logits[r] / temperature) by the Gumbel-max rule, with noise from a hash
// of (seed, positions[r] or 0, r, column). Deterministic for given arguments; temperature > 0.
cudaError_t launch_sample(const __nv_bfloat16* logits, int* out, int rows, int vocab, long long row_stride, float temperature,
                          unsigned int seed, const int* positions, cudaStream_t stream);
}  // namespace sky
