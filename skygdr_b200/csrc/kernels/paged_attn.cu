// Paged GQA decode attention for head-major paged KV caches.
//
// One query token per sequence, G query heads per KV head, head_dim 128, bf16
// cache, pages of T tokens stored [kv_head][token][dim] so that a page of one
// head is one contiguous T*256-byte block. Split-KV: every CTA handles a fixed
// span of tokens of one (sequence, kv_head); the CTA that finishes last for
// that pair merges the partial results (log-sum-exp combine) and writes bf16.
//
// Data path: each warp streams its pages with bulk asynchronous copies
// (cp.async.bulk, the TMA engine) into a private shared-memory ring, tracked
// by mbarriers, so the bytes in flight do not occupy registers; math is fp32
// on CUDA cores with one online-softmax update per page.
//
// The workload shape is the reference's batched, tiled KV scan
// (llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu:203-278), which reads
// fp32 K/V without a block table and never merges its partials, and its
// three-pass attention (llm_problem_analysis/decode_transformer_kvcache_stress.cu:223-317).
#include "common.cuh"
#include "paged_attn.h"

namespace sky {

constexpr int ATT_WARPS = 4;
constexpr int ATT_D = 128;

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cvt8(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

// Two fp32 FMAs in one instruction (Blackwell packed-fp32 pipe): d = a * b + c on register pairs.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(*reinterpret_cast<unsigned long long*>(&d))
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return d;
}
__device__ __forceinline__ void cvt8x2(uint4 v, float2* f) {
    f[0] = make_float2(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u));
    f[1] = make_float2(__uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
    f[2] = make_float2(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u));
    f[3] = make_float2(__uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
}

// T = tokens per page (16), G = query heads per kv head, STAGES = ring depth per warp.
template <int G, int T, int STAGES>
__global__ void __launch_bounds__(ATT_WARPS * 32) paged_attn_decode_kernel(const PagedAttnParams p) {
    constexpr int PAGE_BYTES = T * ATT_D * 2;          // one of K or V
    constexpr int SLOT_BYTES = 2 * PAGE_BYTES;         // K then V
    constexpr int ITERS = T / 4;                       // 4 tokens per warp step
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t bars[ATT_WARPS * STAGES];
    __shared__ int s_last;

    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ts = lane >> 3, dl = lane & 7;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    // Lengths and block ids are device data that this kernel did not produce: a length beyond what the grid and the block
    // table cover is cut to that bound and reported, so that every split the combine counts on exists and no table entry
    // past the row is read.
    const int ctx_raw = p.ctx_lens[b];
    const int ctx = min(ctx_raw, min(p.max_ctx, p.max_blocks * T));
    if (ctx_raw > ctx && split == 0 && kvh == 0 && threadIdx.x == 0) set_status(p.status, SKY_STATUS_BAD_INDEX, 0x40000000u | (unsigned)b);
    const int tok0 = split * p.chunk_tokens;
    if (tok0 >= ctx) return;  // nothing for this CTA (uniform over the block)
    const int tok1 = min(ctx, tok0 + p.chunk_tokens);
    const int page0 = tok0 / T, page1 = (tok1 + T - 1) / T;
    const int n_splits = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;
    const int* table = p.block_table + (long long)b * p.max_blocks;
    unsigned char* ring = smem + warp * STAGES * SLOT_BYTES;
    uint64_t* bar = bars + warp * STAGES;

    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bar + s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    // q, pre-scaled by scale*log2(e): lane holds dims [dl*8, dl*8+8) and [64+dl*8, 64+dl*8+8) of each head
    float2 q[G][8];
    {
        const float qs = p.scale * 1.4426950408889634f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const __nv_bfloat16* qp = p.q + ((long long)b * p.q_heads + kvh * G + g) * ATT_D;
            uint4 a = *reinterpret_cast<const uint4*>(qp + dl * 8);
            uint4 c = *reinterpret_cast<const uint4*>(qp + 64 + dl * 8);
            cvt8x2(a, q[g]);
            cvt8x2(c, q[g] + 4);
#pragma unroll
            for (int i = 0; i < 8; ++i) { q[g][i].x *= qs; q[g][i].y *= qs; }
        }
    }

    // pages of this CTA are dealt round-robin to the warps
    const int my_first = page0 + warp;
    const int my_n = my_first < page1 ? (page1 - my_first + ATT_WARPS - 1) / ATT_WARPS : 0;
    auto issue = [&](int j) {  // lane 0 only: fetch this warp's j-th page into slot j % STAGES
        const int pg = my_first + j * ATT_WARPS;
        int blk = __ldg(table + pg);                    // pg < page1 <= max_blocks by the clamp above
        if (p.num_blocks > 0 && (unsigned)blk >= (unsigned)p.num_blocks) {
            // a block id outside the pool: report it and read block 0 instead, so that nothing outside the pool is touched
            set_status(p.status, SKY_STATUS_BAD_INDEX, ((unsigned)b << 16) | ((unsigned)pg & 0xffffu));
            blk = 0;
        }
        const __nv_bfloat16* kp = p.kv + (long long)blk * p.block_stride + (long long)kvh * p.head_stride;
        unsigned char* slot = ring + (j % STAGES) * SLOT_BYTES;
        mbar_expect_tx(bar + (j % STAGES), SLOT_BYTES);
        bulk_g2s(slot, kp, PAGE_BYTES, bar + (j % STAGES));
        bulk_g2s(slot + PAGE_BYTES, kp + p.kv_stride, PAGE_BYTES, bar + (j % STAGES));
    };
    if (lane == 0)
        for (int j = 0; j < min(STAGES, my_n); ++j) issue(j);

    float m[G], l[G];
    float2 acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = make_float2(0.f, 0.f);
    }

    bool failed = false;
    for (int j = 0; j < my_n; ++j) {
        const int s = j % STAGES;
        // warp-uniform decision: the shuffles below need every lane on the same path
        if (!__all_sync(0xffffffffu, mbar_wait(bar + s, (j / STAGES) & 1))) { failed = true; break; }
        const unsigned char* kpage = ring + s * SLOT_BYTES;
        const unsigned char* vpage = kpage + PAGE_BYTES;
        const int tbase = (my_first + j * ATT_WARPS) * T;
        // ---- scores of the page ----
        float sc[ITERS][G];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int t = it * 4 + ts;
            float2 k[8];
            cvt8x2(*reinterpret_cast<const uint4*>(kpage + t * 256 + dl * 16), k);
            cvt8x2(*reinterpret_cast<const uint4*>(kpage + t * 256 + 128 + dl * 16), k + 4);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float2 a2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) a2 = ffma2(q[g][i], k[i], a2);
                float a = a2.x + a2.y;
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                a += __shfl_xor_sync(0xffffffffu, a, 4);
                const int tok = tbase + t;
                sc[it][g] = (tok >= tok0 && tok < tok1) ? a : -INFINITY;
            }
        }
        // ---- one online-softmax update per page (warp-uniform running max) ----
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float pm = sc[0][g];
#pragma unroll
            for (int it = 1; it < ITERS; ++it) pm = fmaxf(pm, sc[it][g]);
            pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 8));
            pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 16));
            const float mn = fmaxf(m[g], pm);
            if (mn > m[g]) {
                const float r = exp2f(m[g] - mn);  // 0 when m was -inf
                l[g] *= r;
#pragma unroll
                for (int i = 0; i < 8; ++i) { acc[g][i].x *= r; acc[g][i].y *= r; }
                m[g] = mn;
            }
        }
        // ---- P*V ----
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int t = it * 4 + ts;
            float2 v[8];
            cvt8x2(*reinterpret_cast<const uint4*>(vpage + t * 256 + dl * 16), v);
            cvt8x2(*reinterpret_cast<const uint4*>(vpage + t * 256 + 128 + dl * 16), v + 4);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pr = m[g] == -INFINITY ? 0.f : exp2f(sc[it][g] - m[g]);
                l[g] += pr;
                const float2 pr2 = make_float2(pr, pr);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = ffma2(pr2, v[i], acc[g][i]);
            }
        }
        __syncwarp();
        if (lane == 0 && j + STAGES < my_n) { fence_proxy_async(); issue(j + STAGES); }
    }
    if (failed) {
        // Give copies already in flight a bounded chance to land before this CTA's smem is released.
        if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, (unsigned)blockIdx.x);
        for (int j = 0; j < my_n; ++j) mbar_wait(bar + (j % STAGES), (j / STAGES) & 1, 1000000ull);
    }

    // ---- reduce over the 4 token slots of the warp (each 8-lane group saw different tokens) ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        l[g] += __shfl_xor_sync(0xffffffffu, l[g], 8);
        l[g] += __shfl_xor_sync(0xffffffffu, l[g], 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[g][i].x += __shfl_xor_sync(0xffffffffu, acc[g][i].x, 8);
            acc[g][i].x += __shfl_xor_sync(0xffffffffu, acc[g][i].x, 16);
            acc[g][i].y += __shfl_xor_sync(0xffffffffu, acc[g][i].y, 8);
            acc[g][i].y += __shfl_xor_sync(0xffffffffu, acc[g][i].y, 16);
        }
    }
    // ---- merge the warps through shared memory (the ring is idle now) ----
    __syncthreads();
    float* sm_m = reinterpret_cast<float*>(smem);                 // [WARPS][G]
    float* sm_l = sm_m + ATT_WARPS * G;                           // [WARPS][G]
    float* sm_o = sm_l + ATT_WARPS * G;                           // [WARPS][G][128]
    if (ts == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (dl == 0) { sm_m[warp * G + g] = m[g]; sm_l[warp * G + g] = l[g]; }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sm_o[(warp * G + g) * ATT_D + dl * 8 + 2 * i] = acc[g][i].x;
                sm_o[(warp * G + g) * ATT_D + dl * 8 + 2 * i + 1] = acc[g][i].y;
                sm_o[(warp * G + g) * ATT_D + 64 + dl * 8 + 2 * i] = acc[g][4 + i].x;
                sm_o[(warp * G + g) * ATT_D + 64 + dl * 8 + 2 * i + 1] = acc[g][4 + i].y;
            }
        }
    }
    __syncthreads();
    const int d = threadIdx.x;  // 128 threads = 128 dims
    float og[G], mg[G], lg[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float mm = -INFINITY;
        for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_m[w * G + g]);
        float ll = 0.f, oo = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float mw = sm_m[w * G + g];
            const float r = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            ll += sm_l[w * G + g] * r;
            oo += sm_o[(w * G + g) * ATT_D + d] * r;
        }
        og[g] = oo; mg[g] = mm; lg[g] = ll;
    }
    if (n_splits == 1) {
#pragma unroll
        for (int g = 0; g < G; ++g)
            p.out[((long long)b * p.q_heads + kvh * G + g) * ATT_D + d] = __float2bfloat16(lg[g] > 0.f ? og[g] / lg[g] : 0.f);
        return;
    }
    // ---- split-KV: park the partial, and let the last CTA of (b, kvh) combine ----
    const long long row0 = ((long long)b * p.q_heads + kvh * G) * p.max_splits;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const long long row = row0 + (long long)g * p.max_splits + split;
        p.part_o[row * ATT_D + d] = og[g];
        if (d == 0) { p.part_m[row] = mg[g]; p.part_l[row] = lg[g]; }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ctr = p.counters + b * p.kv_heads + kvh;
        const unsigned prev = atomicAdd(ctr, 1u);
        s_last = (prev == (unsigned)n_splits - 1);
        if (s_last) *ctr = 0;  // leave the counter ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const long long row = row0 + (long long)g * p.max_splits;
        p.out[((long long)b * p.q_heads + kvh * G + g) * ATT_D + d] =
            __float2bfloat16(combine_splits(p.part_m + row, p.part_l + row, p.part_o + row * ATT_D + d, ATT_D, n_splits));
    }
}

// Per-device set-up of one instantiation (its dynamic shared memory limit); also loads the kernel's module on that device.
template <int G>
static cudaError_t prepare_g() {
    constexpr int T = 16, STAGES = 3;
    constexpr int smem_bytes = ATT_WARPS * STAGES * 2 * T * ATT_D * 2;
    static_assert(smem_bytes >= (int)((2 * ATT_WARPS * G + ATT_WARPS * G * ATT_D) * sizeof(float)), "merge area must fit in the ring");
    static unsigned long long attr_mask = 0;
    return set_max_dynamic_smem_once(reinterpret_cast<const void*>(paged_attn_decode_kernel<G, T, STAGES>), smem_bytes, &attr_mask);
}

cudaError_t prepare_paged_attn_decode() {
    if (cudaError_t e = prepare_g<1>(); e != cudaSuccess) return e;
    if (cudaError_t e = prepare_g<2>(); e != cudaSuccess) return e;
    if (cudaError_t e = prepare_g<4>(); e != cudaSuccess) return e;
    return prepare_g<8>();
}

template <int G>
static cudaError_t launch_g(const PagedAttnParams& p, cudaStream_t stream) {
    constexpr int T = 16, STAGES = 3;
    constexpr int smem_bytes = ATT_WARPS * STAGES * 2 * T * ATT_D * 2;
    auto kern = paged_attn_decode_kernel<G, T, STAGES>;
    if (cudaError_t e = prepare_g<G>(); e != cudaSuccess) return e;
    dim3 grid((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens, p.kv_heads, p.batch);
    return launch_pdl(kern, grid, dim3(ATT_WARPS * 32), (size_t)smem_bytes, stream, p);
}

cudaError_t launch_paged_attn_decode(const PagedAttnParams& p, cudaStream_t stream) {
    if (p.head_dim != ATT_D || p.block_tokens != 16 || p.kv_heads < 1 || p.q_heads % p.kv_heads) return cudaErrorInvalidValue;
    if (p.chunk_tokens % (16 * ATT_WARPS) != 0 || p.chunk_tokens <= 0) return cudaErrorInvalidValue;
    if ((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens > p.max_splits) return cudaErrorInvalidValue;
    if (p.max_blocks <= 0 || (long long)p.max_ctx > (long long)p.max_blocks * 16) return cudaErrorInvalidValue;   // the table row must cover max_ctx
    switch (p.q_heads / p.kv_heads) {
        case 1: return launch_g<1>(p, stream);
        case 2: return launch_g<2>(p, stream);
        case 4: return launch_g<4>(p, stream);
        case 8: return launch_g<8>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sky
