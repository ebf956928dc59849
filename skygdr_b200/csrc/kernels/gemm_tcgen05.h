// Host-visible interface of the tcgen05 GEMM.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace sky {
struct LaunchStatus;

constexpr int TP_MAX_RANKS = 8;

// Sequence number of a collective inside a replayed CUDA graph: kernels cannot carry a changing
// immediate, so they read the step counter from device memory:
//   seq = *step * uses_per_step + use_index + 1
// and wait for counters to reach seq * arrivals_per_use (counters only ever grow).
struct TpSeq {
    const unsigned int* step;     // device counter, +1 per executed step
    unsigned int uses_per_step;
    unsigned int use_index;
    unsigned int arrivals_per_use;
};

// all-gather -> GEMM: x is this GPU's gather buffer, filled row-block by row-block by the peers'
// norm kernels. The TMA producer streams weights at once and holds the x loads until every
// source's arrival counter has reached the value of this use.
struct TpAgWait {
    int n_src;                                    // 0: off
    const unsigned int* counters;                 // [n_src] in local memory
    TpSeq seq;
    unsigned long long timeout_ns;
};

// GEMM -> reduce-scatter: instead of y, token row t goes to rank t / rows_per_rank, into that rank's
// receive buffer slot [src_rank][t % rows_per_rank][N] (bf16), followed by one arrival on its counter.
// With `all` set the push is the first half of a one-shot all-reduce instead: every token row of the tile goes to EVERY rank,
// into slot [src_rank][t][N] of its buffer (rows_per_rank then holds the full number of token rows), and the consumer sums
// `world` partials per row. More bytes on the links, half as many hops per layer.
struct TpRsPush {
    int world;                                    // 0: off
    int src_rank, rows_per_rank;
    int all;
    __nv_bfloat16* dst[TP_MAX_RANKS];             // peers' receive buffers (peer-mapped)
    unsigned int* counters[TP_MAX_RANKS];         // peers' arrival counters (peer-mapped)
};

struct GemmParams {
    const __nv_bfloat16* x;   // [M][K], row pitch ldx
    const __nv_bfloat16* w;   // [N][K] (gated: [2N][K], gate rows then up rows), row pitch ldw
    __nv_bfloat16* y;         // [M][N], row pitch ldy
    int M, N, K;
    long long ldx, ldw, ldy;
    int splits;               // split-K factor (1 = none)
    int ntok;                 // token-tile width (16/32/64/128/256); 0 = smallest that covers M
    int gated;                // 1: y = silu(x*w_gate^T) * (x*w_up^T)
    float* workspace;         // split-K partials, gemm_workspace_floats() floats
    unsigned int* counters;   // split-K tile counters, gemm_counter_count() entries, zero before first use
    LaunchStatus* status;
    TpAgWait ag;
    TpRsPush rs;
    int cluster_split;        // 1 (with 2 <= splits <= 8): the splits of a tile form a thread-block cluster and reduce through distributed
                              // shared memory; workspace and counters are not used
    int persistent;           // 1: one CTA per SM walks the output tiles with two accumulators in TMEM (many-token shapes; needs
                              // splits == 1, ntok 256 or 128, neither ag nor rs); 2: the same walk over tiles of 256 rows x 256 tokens
                              // (ungated, N a multiple of 256)
};

int gemm_pick_ntok(int M, bool gated);
size_t gemm_workspace_floats(int M, int N, int splits, bool gated, int ntok = 0);
size_t gemm_counter_count(int M, int N, bool gated, int ntok = 0);
cudaError_t launch_gemm(const GemmParams& p, cudaStream_t stream);
}  // namespace sky
