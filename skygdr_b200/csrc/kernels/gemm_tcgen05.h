// Host-visible interface of the tcgen05 GEMM.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace sky {
struct LaunchStatus;

struct GemmParams {
    const __nv_bfloat16* x;   // [M][K], row pitch ldx
    const __nv_bfloat16* w;   // [N][K] (gated: [2N][K], gate rows then up rows), row pitch ldw
    __nv_bfloat16* y;         // [M][N], row pitch ldy
    int M, N, K;
    long long ldx, ldw, ldy;
    int splits;               // split-K factor (1 = none)
    int gated;                // 1: y = silu(x*w_gate^T) * (x*w_up^T)
    float* workspace;         // split-K partials, gemm_workspace_floats() floats
    unsigned int* counters;   // split-K tile counters, gemm_counter_count() entries, zero before first use
    LaunchStatus* status;
};

int gemm_pick_ntok(int M, bool gated);
size_t gemm_workspace_floats(int M, int N, int splits, bool gated);
size_t gemm_counter_count(int M, int N, bool gated);
cudaError_t launch_gemm(const GemmParams& p, cudaStream_t stream);
}  // namespace sky
