// Host-visible parameters of the causal prefill attention over a paged KV pool (prefill_attn_tc.cu).
// The reference has no prefill stage (its decode stressors start from a filled cache,
// llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu:374-388); the prefill -> decode hand-off of the
// case study needs one, so that K/V exist to be transferred.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace sky {
struct LaunchStatus;

struct PrefillAttnParams {
    const __nv_bfloat16* q;      // [total_tokens][q_heads][128]: all prompts packed one after the other
    const __nv_bfloat16* kv;     // base of this layer's pages inside the pool (K and V already appended)
    __nv_bfloat16* out;          // [total_tokens][q_heads][128]
    const int* block_table;      // [n_seqs][max_blocks]; entries past a prompt's pages must name valid blocks (0 is fine)
    const int* seq_start;        // [n_seqs + 1]: token offset of every prompt (or piece of a prompt) in q / out
    long long block_stride;      // elements between consecutive blocks of the pool
    long long kv_stride;         // elements from a block's K page to its V page
    long long head_stride;       // elements between KV heads inside a page
    long long tok_stride;        // elements between tokens inside a page (128 head-major, kv_heads*128 token-major)
    int n_seqs, q_heads, kv_heads, max_blocks;
    int max_len;                 // most queries of one sequence in this launch (sizes the grid)
    int total_tokens;
    float scale;
    const int* pos0;             // [n_seqs] or nullptr: tokens of each sequence that precede its queries of this launch; their K/V are in
                                 // the pool already and every query attends to them (chunked prefill)
    LaunchStatus* status;
    int page_box;                // set by the launcher: 1 = the K/V map fetches a whole page per request (see prefill_attn_tc.cu)
};

// pool_rows: 128-element rows from p.kv to the end of the pool allocation (bounds of the tensor map).
cudaError_t launch_prefill_attn_tc(const PrefillAttnParams& p, long long pool_rows, cudaStream_t stream);
}  // namespace sky
