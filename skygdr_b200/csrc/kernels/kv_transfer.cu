// Paged KV transfer: gather pages named by a block table out of the prefill
// GPU's cache, convert the layout token-major -> head-major (optionally pack to
// block-scaled fp8), and store them straight into one or several decode GPUs'
// paged caches through peer mappings. Every chunk passes a credit gate, so
// pacing and cooperative yield happen inside the kernel.
//
// The reference moves KV with one contiguous cudaMemcpyPeerAsync per request on
// a destination-side stream (llm_problem_analysis/kv_nvlink_transfer.cu:109-122,
// llm_problem_analysis/kv_nvlink_transfer_trace.cu:378-393) and paces a flow by
// sleeping on the host between posts (src/cpu_client.cc:875-879). This kernel
// replaces both.
//
// Source page  (block b, layer l, K|V): [T tokens][H heads][D] bf16
// Destination page                    : [Hd heads][T tokens][D]  bf16, or e4m3 + one
//                                       power-of-two scale byte per 32 elements
// With n_dst > 1 the heads are either scattered (destination g receives heads
// [g*Hd, (g+1)*Hd): tensor-parallel decode ranks) or replicated (every
// destination receives all heads: fan-out). A fan-out can also go through an
// NVLink multicast address (`mc_dst`): one `multimem.st` per 16 bytes leaves
// this GPU and NVSwitch writes it into every destination, so the source's
// link carries the payload once instead of once per destination.
#include <cuda_fp8.h>

#include "common.cuh"
#include "kv_transfer.h"

namespace sky {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// 8 bf16 -> 8 e4m3 with a shared scale 2^e chosen over 32 consecutive elements
// (4 neighbouring lanes). Returns the packed bytes; *scale_byte gets e + 127.
__device__ __forceinline__ uint2 pack_fp8_mx(uint4 v, bool valid, unsigned char* scale_byte) {
    float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y), bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(valid ? f[i] : 0.f));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // Smallest power of two 2^e with amax / 2^e <= 448 = 1.75 * 2^8, from the float's own fields so
    // that the choice is exact: amax = m * 2^k with m in [1,2)  =>  e = k - 8 + (m > 1.75).
    const uint32_t bits = __float_as_uint(amax);
    int e = (int)(bits >> 23) - 127 - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);
    if (amax == 0.f) e = -127;
    e = max(-127, min(127, e));
    float inv = exp2f((float)-e);
    *scale_byte = (unsigned char)(e + 127);
    uint2 out;
    unsigned short p0 = __nv_cvt_float2_to_fp8x2(make_float2(f[0] * inv, f[1] * inv), __NV_SATFINITE, __NV_E4M3);
    unsigned short p1 = __nv_cvt_float2_to_fp8x2(make_float2(f[2] * inv, f[3] * inv), __NV_SATFINITE, __NV_E4M3);
    unsigned short p2 = __nv_cvt_float2_to_fp8x2(make_float2(f[4] * inv, f[5] * inv), __NV_SATFINITE, __NV_E4M3);
    unsigned short p3 = __nv_cvt_float2_to_fp8x2(make_float2(f[6] * inv, f[7] * inv), __NV_SATFINITE, __NV_E4M3);
    out.x = (uint32_t)p0 | ((uint32_t)p1 << 16);
    out.y = (uint32_t)p2 | ((uint32_t)p3 << 16);
    return out;
}

template <int UNROLL>
__global__ void __launch_bounds__(256) kv_transfer_kernel(const KvTransferParams p) {
    __shared__ unsigned long long s_chunk;
    __shared__ int s_go;
    const int tid = threadIdx.x;
    const int vec_per_row = p.head_dim / 8;
    const int n_vec = p.block_tokens * p.heads * vec_per_row;
    const long long pages_per_pair = 2LL * p.layers;
    const long long n_pages = pages_per_pair * p.n_pairs;
    const long long n_chunks = (n_pages + p.pages_per_chunk - 1) / p.pages_per_chunk;
    const unsigned long long page_link_bytes =
        (p.fp8 ? (unsigned long long)n_vec * 8ull + (unsigned long long)n_vec / 4ull : (unsigned long long)n_vec * 16ull) *
        (p.replicate && !p.mc_dst ? p.n_dst : 1);     // a multicast store leaves this GPU once

    unsigned long long grant_cache = 0, stall_ns = 0, my_bytes = 0, my_chunks = 0, last_need = 0;
    if (tid == 0) {
        unsigned long long t = globaltimer_ns();
        atomicMin(&p.status->t_start_ns, t);
    }

    for (;;) {
        if (tid == 0) {
            int go = 0;
            unsigned long long k = 0;
            if (*(volatile unsigned int*)&p.status->status == SKY_STATUS_OK) {
                k = p.first_chunk + atomicAdd(&p.status->work_counter, 1u);
                if ((long long)k < n_chunks) {
                    long long last_page = min((long long)(k + 1) * p.pages_per_chunk, n_pages);
                    unsigned long long need = p.consumed_base +
                        (unsigned long long)(last_page - (long long)p.first_chunk * p.pages_per_chunk) * page_link_bytes;
                    bool stopped, lost;
                    if (credit_acquire(p.page, need, &grant_cache, p.max_wait_ns, &stall_ns, &stopped, &lost)) {
                        go = 1;
                        // Publish progress chunk by chunk (posted writes to the mapped page), so the control
                        // side sees rates inside a long transfer. Chunks are ticketed in order, so `need` is
                        // within a few chunks of the true cumulative count.
                        if (p.usage) {
                            st_sys_u64((unsigned long long*)&p.usage->consumed_bytes, need);
                            if (my_chunks) st_sys_u64((unsigned long long*)&p.usage->completed_bytes, last_need);
                        }
                        last_need = need;
                    } else {
                        atomicMin(&p.status->cursor, k);
                        set_status(p.status, stopped ? SKY_STATUS_STOPPED : lost ? SKY_STATUS_CONTROL_LOST : SKY_STATUS_YIELD_CREDIT, (unsigned)k);
                    }
                }
            }
            s_chunk = k;
            s_go = go;
        }
        __syncthreads();
        const int go = s_go;
        const long long k = (long long)s_chunk;
        __syncthreads();
        if (!go) break;

        const long long page0 = k * p.pages_per_chunk;
        const long long page1 = min(page0 + p.pages_per_chunk, n_pages);
        for (long long pg = page0; pg < page1; ++pg) {
            const int pair = (int)(pg / pages_per_pair);
            const int rem = (int)(pg - (long long)pair * pages_per_pair);
            const int layer = rem >> 1, kv = rem & 1;
            const int sb = __ldg(p.src_blocks + pair), db = __ldg(p.dst_blocks + pair);
            if ((p.src_num_blocks && (unsigned)sb >= (unsigned)p.src_num_blocks) || (p.dst_num_blocks && (unsigned)db >= (unsigned)p.dst_num_blocks)) {
                if (tid == 0) set_status(p.status, SKY_STATUS_BAD_INDEX, (unsigned)pair);    // same decision in every thread
                continue;
            }
            const __nv_bfloat16* src = p.src_pool + (long long)sb * p.src_block_stride + (long long)layer * p.src_layer_stride +
                                       (long long)kv * p.src_kv_stride;
            const long long dst_off = (long long)db * p.dst_block_stride + (long long)layer * p.dst_layer_stride +
                                      (long long)kv * p.dst_kv_stride;
            for (int base = 0; base < n_vec; base += 256 * UNROLL) {
                uint4 v[UNROLL];
                int idx[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    idx[u] = base + u * 256 + tid;
                    v[u] = idx[u] < n_vec ? ld_nc_v4(src + (long long)idx[u] * 8) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const bool valid = idx[u] < n_vec;
                    const int row = idx[u] / vec_per_row, c = idx[u] - row * vec_per_row;
                    const int t = row / p.heads, h = row - t * p.heads;
                    const int g0 = p.replicate ? 0 : h / p.heads_per_dst;
                    const int hl = p.replicate ? h : h - g0 * p.heads_per_dst;
                    const long long e = p.keep_layout ? dst_off + (long long)idx[u] * 8
                                                      : dst_off + ((long long)hl * p.block_tokens + t) * p.head_dim + c * 8;
                    if (!p.fp8) {
                        if (valid) {
                            if (p.mc_dst) {
                                multimem_st_v4((__nv_bfloat16*)p.mc_dst + e, v[u]);
                            } else if (p.replicate) {
                                for (int g = 0; g < p.n_dst; ++g) st_v4((__nv_bfloat16*)p.dst[g] + e, v[u]);
                            } else {
                                st_v4((__nv_bfloat16*)p.dst[g0] + e, v[u]);
                            }
                        }
                    } else {
                        unsigned char sb8;
                        uint2 packed = pack_fp8_mx(v[u], valid, &sb8);
                        if (valid) {
                            const int ng = p.replicate ? p.n_dst : 1;
                            for (int gi = 0; gi < ng; ++gi) {
                                const int g = p.replicate ? gi : g0;
                                *reinterpret_cast<uint2*>((unsigned char*)p.dst[g] + e) = packed;
                                if ((c & 3) == 0) ((unsigned char*)p.dst_scales[g])[e >> 5] = sb8;
                            }
                        }
                    }
                }
            }
        }
        my_bytes += (unsigned long long)(page1 - page0) * page_link_bytes;
        my_chunks += 1;
    }

    // ---- epilogue: publish progress, then (last CTA) the usage counters and the ready flags ----
    __syncthreads();
    if (tid == 0) {
        if (my_chunks) { atomicAdd(&p.status->chunks_done, my_chunks); atomicAdd(&p.status->bytes_done, my_bytes); }
        if (stall_ns) atomicAdd(&p.status->stall_ns, stall_ns);
        __threadfence_system();  // this CTA's payload stores are ordered before the counter below
        unsigned prev = atomicAdd(&p.status->ctas_done, 1u);
        if (prev == gridDim.x - 1) {
            __threadfence();
            unsigned long long now = globaltimer_ns();
            p.status->t_end_ns = now;
            unsigned long long bytes = *(volatile unsigned long long*)&p.status->bytes_done;
            bool complete = *(volatile unsigned int*)&p.status->status == SKY_STATUS_OK;
            if (p.usage) {
                SkyCreditPage* u = p.usage;
                st_sys_u64((unsigned long long*)&u->consumed_bytes, p.consumed_base + bytes);
                st_sys_u64((unsigned long long*)&u->completed_bytes, p.consumed_base + bytes);
                st_sys_u64((unsigned long long*)&u->stall_ns, u->stall_ns + *(volatile unsigned long long*)&p.status->stall_ns);
                st_sys_u64((unsigned long long*)&u->busy_ns, u->busy_ns + (now - *(volatile unsigned long long*)&p.status->t_start_ns));
                st_sys_u64((unsigned long long*)&u->chunks, u->chunks + *(volatile unsigned long long*)&p.status->chunks_done);
                st_sys_u64((unsigned long long*)&u->last_ts_ns, now);
                if (!complete) st_sys_u64((unsigned long long*)&u->yields, u->yields + 1);
            }
            if (complete) {
                __threadfence_system();
                for (int g = 0; g < p.n_dst; ++g)
                    if (p.done_flag[g]) st_release_sys_u32(p.done_flag[g], p.done_value);
            }
        }
    }
}

cudaError_t launch_kv_transfer(const KvTransferParams& p, int ctas, cudaStream_t stream) {
    if (p.head_dim % 8 != 0 || p.n_dst < 1 || p.n_dst > KV_MAX_DST || p.pages_per_chunk < 1) return cudaErrorInvalidValue;
    if (!p.replicate && p.heads_per_dst * p.n_dst != p.heads) return cudaErrorInvalidValue;
    if (p.fp8 && (p.head_dim % 32 != 0)) return cudaErrorInvalidValue;
    if (p.mc_dst && (p.fp8 || !p.replicate)) return cudaErrorInvalidValue;   // multicast stores carry whole bf16 pages to every member
    kv_transfer_kernel<8><<<ctas, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace sky
