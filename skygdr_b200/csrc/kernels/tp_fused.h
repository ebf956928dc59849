// Tensor-parallel glue kernels: collectives done by the compute kernels themselves over peer memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_tcgen05.h"

namespace sky {

// reduce-scatter reduce + residual add + RMSNorm + all-gather push, one CTA per local token row.
struct TpNormParams {
    const __nv_bfloat16* rs_buf;            // local receive buffer [world][rows][hidden]; nullptr: no reduce-scatter input
    const unsigned int* rs_counter;         // local arrival counter of rs_buf
    TpSeq rs_seq;
    __nv_bfloat16* resid;                   // [rows][hidden] this rank's slice of the residual stream (updated in place)
    const __nv_bfloat16* w;                 // [hidden]
    __nv_bfloat16* ag_dst[TP_MAX_RANKS];    // every rank's gather buffer [world*rows][hidden] (peer-mapped; own included)
    unsigned int* ag_counter[TP_MAX_RANKS]; // on rank j: its counter for source = this rank
    int world, rank, rows, hidden;
    // One-shot all-reduce form: `rows` is the whole batch, rs_buf holds [world][rows][hidden] full-size partials, the residual is
    // replicated, and the normed rows go to ag_n = 1 destination (a local buffer, ag_counter[0] == nullptr) at row ag_row0 = 0.
    // The reduce-scatter / all-gather form has ag_n = world and ag_row0 = rank * rows.
    int ag_n, ag_row0;
    float eps;
    unsigned long long timeout_ns;
    LaunchStatus* status;
};
cudaError_t launch_tp_norm(const TpNormParams& p, cudaStream_t stream);

// vocabulary-parallel greedy sampling: local argmax, exchange (value, index) with every rank, global argmax.
struct TpArgmaxParams {
    const __nv_bfloat16* logits;            // [rows][vocab_local]
    long long row_stride;
    int rows, vocab_local, vocab_lo, world, rank;
    unsigned long long* slots[TP_MAX_RANKS];   // on rank j: [world][rows] candidates (peer-mapped)
    unsigned int* counters[TP_MAX_RANKS];      // on rank j: its counter for source = this rank
    const unsigned long long* my_slots;
    const unsigned int* my_counters;           // [world]
    TpSeq seq;
    int* next_ids;                             // [rows]
    unsigned long long timeout_ns;
    LaunchStatus* status;
};
cudaError_t launch_tp_argmax(const TpArgmaxParams& p, cudaStream_t stream);

cudaError_t launch_step_increment(unsigned int* step, cudaStream_t stream);
}  // namespace sky
