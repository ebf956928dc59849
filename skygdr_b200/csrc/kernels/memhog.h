// Host-visible parameters of the best-effort HBM task.
#pragma once
#include <cuda_runtime.h>

#include "credit_page.h"

namespace sky {
struct LaunchStatus;

enum MemhogOp { MEMHOG_READ = 0, MEMHOG_WRITE = 1, MEMHOG_RW = 2, MEMHOG_COPY = 3, MEMHOG_AXPY = 4 };

struct MemhogParams {
    float4* a;                      // read side (n_vec float4)
    float4* b;                      // write side (unused by READ)
    unsigned long long n_vec;
    int op;
    int iters;                      // passes over the working set; <=0: run until duration_ns
    unsigned long long duration_ns; // 0: no time limit
    unsigned long long duty_on_ns, duty_off_ns;  // off = 0: always on
    unsigned long long chunk_vec;   // float4s per scheduling chunk (per CTA)
    const SkyCreditPage* page;      // optional credit gate, checked per chunk
    SkyCreditPage* usage;
    unsigned long long consumed_base, max_wait_ns;
    float alpha;
    double* sink;                   // READ: sum lands here
    LaunchStatus* status;
};

// Bytes of HBM traffic per element for an op: the accounting of the reference's
// tasks (src/gpu_be_memhog_task.cu:273-287; decode_hbm_stress.cu:159-165 for axpy).
__host__ __device__ inline unsigned long long memhog_bytes_per_vec(int op) {
    switch (op) {
        case MEMHOG_READ: case MEMHOG_WRITE: return 16;
        case MEMHOG_RW: case MEMHOG_COPY: return 32;
        default: return 48;  // axpy reads a and b, writes b
    }
}

cudaError_t launch_memhog(const MemhogParams& p, int ctas, int threads, cudaStream_t stream);
}  // namespace sky
