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
    const int* seq_start;        // [n_seqs + 1]: token offset of every prompt in q / out (prefix sums of the lengths)
    long long block_stride;      // elements between consecutive blocks of the pool
    long long kv_stride;         // elements from a block's K page to its V page
    long long head_stride;       // elements between KV heads inside a page
    long long tok_stride;        // elements between tokens inside a page (128 head-major, kv_heads*128 token-major)
    int n_seqs, q_heads, kv_heads, max_blocks;
    int max_len;                 // longest prompt (sizes the grid)
    int total_tokens;
    float scale;
    int two_tiles;               // 1: two query tiles per CTA working in alternation (prefill_attn_tc2_kernel); 0: one tile per CTA;
                                 // 2: two tiles with key steps of 64 and double-buffered scores (prefill_attn_tc3_kernel);
                                 // 3-6: the two-tile kernel with part of the exponentials on the FMA pipe and/or P kept in TMEM
                                 // (3: 1 of 4 exponentials; 4: P in TMEM; 5: both; 6: 2 of 4 exponentials and P in TMEM)
    LaunchStatus* status;
};

// pool_rows: 128-element rows from p.kv to the end of the pool allocation (bounds of the tensor map).
cudaError_t launch_prefill_attn_tc(const PrefillAttnParams& p, long long pool_rows, cudaStream_t stream);
}  // namespace sky
