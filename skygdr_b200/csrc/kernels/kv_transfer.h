// Host-visible parameters of the paged KV transfer kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "credit_page.h"

namespace sky {

struct LaunchStatus;

constexpr int KV_MAX_DST = 8;

struct KvTransferParams {
    const __nv_bfloat16* src_pool;        // token-major pages on the source GPU
    void* dst[KV_MAX_DST];                // head-major pools (local or peer-mapped)
    void* mc_dst;                         // fan-out through NVSwitch: multicast address of the destinations' pools (bf16,
                                          // replicate only); stores go out once and land in every team member's copy
    void* dst_scales[KV_MAX_DST];         // fp8 mode: one byte per 32 elements, same indexing / 32
    unsigned int* done_flag[KV_MAX_DST];  // optional: set to done_value (release, system scope) when all pages landed
    const int* src_blocks;                // [n_pairs] block ids in the source pool
    const int* dst_blocks;                // [n_pairs] block ids in the destination pool(s)
    int n_pairs, layers, heads, block_tokens, head_dim;
    int src_num_blocks, dst_num_blocks;   // pool sizes for the index check (0 = unchecked): a block id outside its pool
                                          // is skipped and reported as SKY_STATUS_BAD_INDEX with the pair's position
    long long src_block_stride, src_layer_stride, src_kv_stride;  // in source elements
    long long dst_block_stride, dst_layer_stride, dst_kv_stride;  // in destination elements
    int n_dst, heads_per_dst, replicate, fp8;
    int keep_layout;                      // 1: destination pages keep the source's token-major order (offload to host)
    int pages_per_chunk;                  // credit and scheduling granularity
    unsigned int done_value;
    const SkyCreditPage* page;            // grant half is read here; nullptr = ungated
    SkyCreditPage* usage;                 // usage half is written here at the end; may be nullptr
    unsigned long long consumed_base;     // flow's cumulative bytes before this launch
    unsigned long long max_wait_ns;       // credit wait per chunk before the kernel yields
    unsigned long long first_chunk;       // resume cursor
    LaunchStatus* status;
};

cudaError_t launch_kv_transfer(const KvTransferParams& p, int ctas, cudaStream_t stream);
// All-TMA variant for bf16 pages (kv_transfer_tma.cu). pool_elems: elements of the whole source pool allocation.
cudaError_t launch_kv_transfer_tma(const KvTransferParams& p, long long pool_elems, int ctas, cudaStream_t stream);

}  // namespace sky
