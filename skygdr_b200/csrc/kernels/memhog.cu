// Best-effort HBM task: streaming read / write / read-write / copy / axpy over a
// large working set, as one persistent launch with the duty cycle, the time
// limit and the credit gate inside the kernel.
//
// It covers the reference's five memhog kernels (src/gpu_be_memhog_task.cu:58-140)
// and its decode-side stressor b += alpha*a (llm_problem_analysis/decode_hbm_stress.cu:42-60),
// which the reference drives with one launch per iteration from a host loop
// (src/gpu_be_memhog_task.cu:299-344).
#include "common.cuh"
#include "memhog.h"

namespace sky {

__device__ __forceinline__ float4 ld_stream(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(float4* p, float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int OP>
__device__ __forceinline__ void hog_chunk(const MemhogParams& p, unsigned long long v0, unsigned long long v1, float& acc, float& wv) {
    constexpr int U = 4;
    const unsigned long long stride = (unsigned long long)blockDim.x * U;
    for (unsigned long long i = v0 + threadIdx.x; i < v1; i += stride) {
        float4 x[U], y[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            unsigned long long j = i + (unsigned long long)u * blockDim.x;
            if (j < v1) {
                if (OP != MEMHOG_WRITE) x[u] = ld_stream(p.a + j);
                if (OP == MEMHOG_AXPY) y[u] = ld_stream(p.b + j);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            unsigned long long j = i + (unsigned long long)u * blockDim.x;
            if (j >= v1) continue;
            if (OP == MEMHOG_READ) acc += x[u].x + x[u].y + x[u].z + x[u].w;
            else if (OP == MEMHOG_WRITE) { st_stream(p.b + j, make_float4(wv, wv, wv, wv)); wv = wv * 1.0000001f + 1e-7f; }
            else if (OP == MEMHOG_RW) st_stream(p.b + j, make_float4(x[u].x * 1.0001f + 0.5f, x[u].y * 1.0001f + 0.5f, x[u].z * 1.0001f + 0.5f, x[u].w * 1.0001f + 0.5f));
            else if (OP == MEMHOG_COPY) st_stream(p.b + j, x[u]);
            else st_stream(p.b + j, make_float4(y[u].x + p.alpha * x[u].x, y[u].y + p.alpha * x[u].y, y[u].z + p.alpha * x[u].z, y[u].w + p.alpha * x[u].w));
        }
    }
}

__global__ void __launch_bounds__(512) memhog_kernel(const MemhogParams p) {
    __shared__ int s_go;
    __shared__ float s_red[16];
    const unsigned long long bytes_per_vec = memhog_bytes_per_vec(p.op);
    const unsigned long long chunks_per_pass = (p.n_vec + p.chunk_vec - 1) / p.chunk_vec;
    unsigned long long grant_cache = 0, stall_ns = 0, my_bytes = 0, my_chunks = 0;
    float acc = 0.f, wv = 1.0f + threadIdx.x * 1e-3f;
    unsigned long long t0 = 0;
    if (threadIdx.x == 0) {
        t0 = globaltimer_ns();
        atomicMin(&p.status->t_start_ns, t0);
    }
    // CTA c handles chunks c, c+grid, ... of each pass: a static map, so every CTA can tell its
    // own cumulative byte count for the credit gate without a shared counter.
    unsigned long long seq = 0;  // chunks this CTA has attempted
    // A CTA without a chunk of its own has nothing to do (and nothing that would ever end a timed run).
    const bool has_work = blockIdx.x < chunks_per_pass;
    for (int pass = 0; has_work && (p.iters <= 0 || pass < p.iters); ++pass) {
        bool quit = false;
        for (unsigned long long c = blockIdx.x; c < chunks_per_pass; c += gridDim.x, ++seq) {
            if (threadIdx.x == 0) {
                int go = 1;
                unsigned long long now = globaltimer_ns();
                if (p.duty_off_ns) {
                    // sleep through the OFF part of the period (bounded: one period at most)
                    unsigned long long period = p.duty_on_ns + p.duty_off_ns;
                    unsigned long long start = *(volatile unsigned long long*)&p.status->t_start_ns;
                    unsigned long long ph = (now - start) % period;
                    if (ph >= p.duty_on_ns) {
                        unsigned long long wake = now + (period - ph);
                        while (globaltimer_ns() < wake) __nanosleep(20000);
                        now = globaltimer_ns();
                    }
                }
                // The time limit counts from the first CTA's start, not this one's: with more CTAs than fit on the GPU at
                // once, the late ones must not each run a full period of their own.
                if (p.duration_ns && now - *(volatile unsigned long long*)&p.status->t_start_ns >= p.duration_ns) go = 0;
                if (go && p.page) {
                    // all CTAs advance together, so the flow has consumed about seq*grid+block chunks
                    unsigned long long need = p.consumed_base + ((seq * gridDim.x) + blockIdx.x + 1) * p.chunk_vec * bytes_per_vec;
                    bool stopped, lost;
                    if (!credit_acquire(p.page, need, &grant_cache, p.max_wait_ns, &stall_ns, &stopped, &lost)) {
                        go = 0;
                        set_status(p.status, stopped ? SKY_STATUS_STOPPED : lost ? SKY_STATUS_CONTROL_LOST : SKY_STATUS_YIELD_CREDIT, (unsigned)seq);
                    }
                }
                s_go = go;
            }
            __syncthreads();
            const int go = s_go;
            __syncthreads();
            if (!go) { quit = true; break; }
            unsigned long long v0 = c * p.chunk_vec, v1 = min(v0 + p.chunk_vec, p.n_vec);
            switch (p.op) {
                case MEMHOG_READ: hog_chunk<MEMHOG_READ>(p, v0, v1, acc, wv); break;
                case MEMHOG_WRITE: hog_chunk<MEMHOG_WRITE>(p, v0, v1, acc, wv); break;
                case MEMHOG_RW: hog_chunk<MEMHOG_RW>(p, v0, v1, acc, wv); break;
                case MEMHOG_COPY: hog_chunk<MEMHOG_COPY>(p, v0, v1, acc, wv); break;
                default: hog_chunk<MEMHOG_AXPY>(p, v0, v1, acc, wv); break;
            }
            my_bytes += (v1 - v0) * bytes_per_vec;
            ++my_chunks;
        }
        if (quit) break;
    }
    if (p.op == MEMHOG_READ && p.sink) {
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double s = 0;
            for (int w = 0; w < (blockDim.x + 31) / 32; ++w) s += s_red[w];
            atomicAdd(p.sink, s);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd(&p.status->chunks_done, my_chunks);
        atomicAdd(&p.status->bytes_done, my_bytes);
        if (stall_ns) atomicAdd(&p.status->stall_ns, stall_ns);
        __threadfence();
        unsigned prev = atomicAdd(&p.status->ctas_done, 1u);
        if (prev == gridDim.x - 1) {
            unsigned long long now = globaltimer_ns();
            p.status->t_end_ns = now;
            if (p.usage) {
                unsigned long long bytes = *(volatile unsigned long long*)&p.status->bytes_done;
                st_sys_u64((unsigned long long*)&p.usage->consumed_bytes, p.consumed_base + bytes);
                st_sys_u64((unsigned long long*)&p.usage->completed_bytes, p.consumed_base + bytes);
                st_sys_u64((unsigned long long*)&p.usage->last_ts_ns, now);
            }
        }
    }
}

cudaError_t launch_memhog(const MemhogParams& p, int ctas, int threads, cudaStream_t stream) {
    if (threads < 32 || threads > 512 || (threads & 31) || p.chunk_vec == 0 || p.n_vec == 0) return cudaErrorInvalidValue;
    if (p.iters <= 0 && p.duration_ns == 0) return cudaErrorInvalidValue;  // would never end
    const unsigned long long chunks = (p.n_vec + p.chunk_vec - 1) / p.chunk_vec;
    if ((unsigned long long)ctas > chunks) ctas = (int)chunks;
    memhog_kernel<<<ctas, threads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace sky
