// Paged GQA decode attention on the 5th-generation tensor cores.
//
// Same contract as paged_attn.cu (one query token per sequence, G query heads per KV head, head_dim 128,
// bf16 head-major pages of 16 tokens, split-KV with an in-kernel last-CTA combine), different engine:
//
//   warp 4   : TMA producer. Per 128-token tile, 16 + 16 tensor-map boxes ([16 tokens] x [64 dims], 128-byte
//              swizzle; one box per page and half of head_dim) land K and V in a ring of three 32 KB units
//              (K0, V0, K1, ...), small enough for two CTAs per SM. No cluster broadcast.
//   warp 5   : MMA issuer and TMEM owner.
//                S^T[128 tok x 16] = K_tile[128 x 128] . Q^T           (A, B K-major; tokens are the MMA's M)
//                O^T[128 dim x 16] += V_tile^T[128 x 128] . P^T        (A = V as stored, MN-major; B = P^T K-major)
//              S is double-buffered in TMEM so the next tile's scores are computed while this tile's softmax runs.
//   warps 0-3: softmax. Thread t owns token t of the tile (TMEM lane t): scale, mask, tile max (shuffles + a
//              4-way exchange through shared memory), exp2, P^T written to shared memory in the swizzled layout
//              the MMA reads. The running max is only raised when a tile exceeds it by more than 8 (in log2
//              units), so the accumulator in TMEM is rescaled (tcgen05.ld/st) a handful of times per sequence.
// The epilogue reads O^T from TMEM (thread d owns dimension d), reduces the row sums, and joins the split-KV
// combine of the CUDA-core kernel.
//
// Block tables must be padded with valid block ids (e.g. 0) up to a multiple of 8 entries' worth of reads:
// a tile always fetches 8 pages; entries past the table's width are read as block 0. Page contents past a
// sequence's length must be finite (they are multiplied by exactly zero).
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "paged_attn.h"

namespace sky {

bool make_tmap_bf16_2d(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows);

namespace {

constexpr int TC_THREADS = 192;
constexpr int TILE_TOK = 128;
constexpr int TC_UNITS = 3;                         // ring of 32 KB units: K0, V0, K1, V1, ... (unit u holds tile u/2's K or V)
constexpr int HALF_BYTES = TILE_TOK * 64 * 2;       // one [128 tok][64 dim] swizzled sub-tile: 16 KB
constexpr int KV_TILE_BYTES = 2 * HALF_BYTES;       // K or V tile: 32 KB
constexpr int QP_BYTES = 2 * 16 * 128;              // [16 rows][128 cols] bf16 as two swizzled [16][64] sub-tiles: 4 KB
constexpr int TC_SMEM = TC_UNITS * KV_TILE_BYTES + 3 * QP_BYTES + 1024;    // ring + Q^T + two P^T buffers: two CTAs fit one SM
constexpr int MAX_CHUNK_PAGES = 512;                                      // chunk_tokens <= 8192
constexpr float RESCALE_THRESHOLD = 8.0f;



__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int G>
__global__ void __launch_bounds__(TC_THREADS, 2) paged_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap, const PagedAttnParams p) {
    constexpr int GL = G <= 4 ? 4 : 8;               // columns read per TMEM access
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full_bar[TC_UNITS], empty_bar[TC_UNITS], s_ready[2], p_ready[2], o_done[2];
    __shared__ uint32_t tmem_slot;
    __shared__ float xch[2][4][8];                    // tile max exchange: [parity][warp][head]
    __shared__ float lsum[4][8];
    __shared__ int s_last;
    __shared__ int s_blocks[MAX_CHUNK_PAGES];            // this CTA's slice of the block table
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_sm = smem + TC_UNITS * KV_TILE_BYTES;
    unsigned char* p_sm = q_sm + QP_BYTES;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid order: splits fastest, then KV heads, then sequences
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    // Everything up to pdl_wait() touches only this CTA's shared memory, so it may overlap the previous kernel's tail.
    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_UNITS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&s_ready[0], 1); mbar_init(&s_ready[1], 1);
        mbar_init(&p_ready[0], 128); mbar_init(&p_ready[1], 128);
        mbar_init(&o_done[0], 1); mbar_init(&o_done[1], 1);
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < 3 * QP_BYTES / 16; i += TC_THREADS) reinterpret_cast<uint4*>(q_sm)[i] = make_uint4(0, 0, 0, 0);
    pdl_wait();
    // a length beyond what the grid and the table row cover is cut to that bound and reported (see paged_attn.cu)
    const int ctx_raw = p.ctx_lens[b];
    const int ctx = min(ctx_raw, min(p.max_ctx, p.max_blocks * 16));
    if (ctx_raw > ctx && split == 0 && kvh == 0 && threadIdx.x == 0)
        set_status(p.status, SKY_STATUS_BAD_INDEX, 0x40000000u | (unsigned)b);
    const int n_splits = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;
    const int tok0 = split * p.chunk_tokens;
    const int tok1 = min(ctx, tok0 + p.chunk_tokens);
    if (tok0 >= ctx || ctx <= 0) return;
    const int n_tiles = (tok1 - tok0 + TILE_TOK - 1) / TILE_TOK;
    const int* table = p.block_table + (long long)b * p.max_blocks;

    if (warp == 5) { tmem_alloc(&tmem_slot, 64); tmem_relinquish(); }
    // Q^T and P^T operand tiles: zero everything (rows G..15 stay zero), then Q rows 0..G-1 in swizzled order
    for (int i = threadIdx.x; i < n_tiles * 8; i += TC_THREADS) {       // coalesced; entries past the table read block 0
        const int e = (tok0 >> 4) + i;
        s_blocks[i] = e < p.max_blocks ? __ldg(table + e) : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * 16; i += TC_THREADS) {        // 16-byte chunks: G rows x 16 chunks
        const int g = i >> 4, c = i & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(p.q + ((long long)b * p.q_heads + kvh * G + g) * 128 + c * 8);
        *reinterpret_cast<uint4*>(q_sm + (c >> 3) * 2048 + sw128_off(g, (c & 7) * 8)) = v;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tm_s[2] = {tmem_base, tmem_base + 16};
    const uint32_t tm_o = tmem_base + 32;

    float m_ref[GL], l_part[GL];
#pragma unroll
    for (int g = 0; g < GL; ++g) { m_ref[g] = -INFINITY; l_part[g] = 0.f; }
    bool ok = true;

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) tma_prefetch_desc(&tmap);
        const long long head_rows = (long long)kvh * (p.head_stride >> 7);
        // unit u = 2*tile + (0: K, 1: V); lanes 0-15 issue its 16 boxes (page l/2, dim half l&1)
        const int pg = lane >> 1, half = lane & 1;
        for (int u = 0; u < 2 * n_tiles; ++u) {
            const int s = u % TC_UNITS;
            if (u >= TC_UNITS && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((u / TC_UNITS) - 1) & 1))) {
                if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 11);
                break;
            }
            unsigned char* st = smem + s * KV_TILE_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[s], KV_TILE_BYTES);
            __syncwarp();
            if (lane < 16) {
                const int blk = s_blocks[(u >> 1) * 8 + pg];
                const long long row = ((long long)blk * p.block_stride >> 7) + head_rows + ((u & 1) ? (p.kv_stride >> 7) : 0);
                tma_load_2d(st + half * HALF_BYTES + pg * 2048, &tmap, half * 64, (int)row, &full_bar[s]);
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 16);                      // K-major x K-major
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, 16) | (1u << 15);         // A is MN-major
            const uint32_t q_addr = smem_u32(q_sm), p_addr = smem_u32(p_sm);
            auto issue_s = [&](int i) -> bool {
                const int u = 2 * i, s = u % TC_UNITS;
                if (!mbar_wait(&full_bar[s], (u / TC_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 12); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t a = umma_desc_k_sw128(k_addr + (j >> 2) * HALF_BYTES + (j & 3) * 32);
                    const uint64_t bq = umma_desc_k_sw128(q_addr + (j >> 2) * 2048 + (j & 3) * 32);
                    tc_mma_f16(tm_s[i & 1], a, bq, idesc_s, j ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);     // K of this tile is free once the scores are done
                tc_commit(&s_ready[i & 1]);
                return true;
            };
            bool good = issue_s(0);
            for (int i = 0; i < n_tiles && good; ++i) {
                if (i + 1 < n_tiles) good = issue_s(i + 1);
                if (!good) break;
                if (!mbar_wait(&p_ready[i & 1], (i >> 1) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 13); break; }
                const int u = 2 * i + 1, s = u % TC_UNITS;
                if (!mbar_wait(&full_bar[s], (u / TC_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 17); break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t a = umma_desc_mn_sw128(v_addr + j * 2048, HALF_BYTES, 1024);
                    const uint64_t bp = umma_desc_k_sw128(p_addr + (i & 1) * QP_BYTES + (j >> 2) * 2048 + (j & 3) * 32);
                    tc_mma_f16(tm_o, a, bp, idesc_o, (i | j) ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);     // V of this tile is free again
                tc_commit(&o_done[i & 1]);    // this tile's P buffer is free again; the accumulator may be touched
            }
        }
    } else {
        // ---------------- softmax warps: thread t <-> token t of the tile ----------------
        const int t = threadIdx.x;                                   // 0..127
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float qs = p.scale * 1.4426950408889634f;
        for (int i = 0; i < n_tiles; ++i) {
            if (!mbar_wait(&s_ready[i & 1], (i >> 1) & 1)) { if (t == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 14); ok = false; break; }
            tc_fence_after();
            uint32_t raw[GL];
            if (GL == 4) tmem_ld_x4(tm_s[i & 1] + lane_off, raw); else tmem_ld_x8(tm_s[i & 1] + lane_off, raw);
            tc_wait_ld();
            const int tok = tok0 + i * TILE_TOK + t;
            const bool valid = tok < tok1;
            float sc[GL], tmax[GL];
#pragma unroll
            for (int g = 0; g < GL; ++g) {
                sc[g] = (valid && g < G) ? __uint_as_float(raw[g]) * qs : -INFINITY;
                tmax[g] = sc[g];
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
                for (int o = 16; o; o >>= 1) tmax[g] = fmaxf(tmax[g], __shfl_xor_sync(0xffffffffu, tmax[g], o));
            if (lane == 0)
#pragma unroll
                for (int g = 0; g < G; ++g) xch[i & 1][warp][g] = tmax[g];
            softmax_bar();
            float alpha[GL];
            bool rescale = false;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float tm = fmaxf(fmaxf(xch[i & 1][0][g], xch[i & 1][1][g]), fmaxf(xch[i & 1][2][g], xch[i & 1][3][g]));
                alpha[g] = 1.0f;
                if (tm > m_ref[g] + RESCALE_THRESHOLD || m_ref[g] == -INFINITY) {      // same decision in every thread
                    alpha[g] = m_ref[g] == -INFINITY ? 0.f : exp2f(m_ref[g] - tm);
                    m_ref[g] = tm;
                    rescale = true;
                }
            }
            float pr[GL];
#pragma unroll
            for (int g = 0; g < GL; ++g) {
                pr[g] = (g < G && valid) ? exp2f(sc[g] - m_ref[g]) : 0.f;
                if (g < G) l_part[g] = l_part[g] * alpha[g] + pr[g];
            }
            // P^T is double-buffered: buffer i&1 was last read by tile i-2's P.V. A rescale of the accumulator has to
            // wait for tile i-1's P.V too (which, issued in order, also covers tile i-2). o_done[k] completes once per
            // tile of parity k, so tile j is completion number j>>1 of o_done[j&1].
            if (rescale && i > 0) {
                if (!mbar_wait(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1)) { if (t == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 15); ok = false; break; }
            } else if (i > 1) {
                if (!mbar_wait(&o_done[i & 1], ((i - 2) >> 1) & 1)) { if (t == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 15); ok = false; break; }
            }
            if (rescale && i > 0) {
                tc_fence_after();
                uint32_t o[GL];
                if (GL == 4) tmem_ld_x4(tm_o + lane_off, o); else tmem_ld_x8(tm_o + lane_off, o);
                tc_wait_ld();
#pragma unroll
                for (int g = 0; g < GL; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * (g < G ? alpha[g] : 1.0f));
                if (GL == 4) tmem_st_x4(tm_o + lane_off, o); else tmem_st_x8(tm_o + lane_off, o);
                tc_wait_st();
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
                *reinterpret_cast<__nv_bfloat16*>(p_sm + (i & 1) * QP_BYTES + (t >> 6) * 2048 + sw128_off(g, t & 63)) = __float2bfloat16(pr[g]);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_ready[i & 1]);     // one barrier per P buffer: the softmax may run a tile ahead of the MMA thread
        }
        // the last P.V
        if (ok && !mbar_wait(&o_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1)) { if (t == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 16); ok = false; }
        tc_fence_after();
    }

    // ---------------- epilogue: thread d owns dimension d ----------------
    float og[G], lg[G];
    if (warp < 4) {
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        uint32_t o[GL];
        if (GL == 4) tmem_ld_x4(tm_o + lane_off, o); else tmem_ld_x8(tm_o + lane_off, o);
        tc_wait_ld();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            og[g] = ok ? __uint_as_float(o[g]) : 0.f;
            float l = l_part[g];
            for (int of = 16; of; of >>= 1) l += __shfl_xor_sync(0xffffffffu, l, of);
            if (lane == 0) lsum[warp][g] = l;
        }
        softmax_bar();
#pragma unroll
        for (int g = 0; g < G; ++g) lg[g] = lsum[0][g] + lsum[1][g] + lsum[2][g] + lsum[3][g];
        const int d = threadIdx.x;
        if (n_splits == 1) {
#pragma unroll
            for (int g = 0; g < G; ++g)
                p.out[((long long)b * p.q_heads + kvh * G + g) * 128 + d] = __float2bfloat16(lg[g] > 0.f ? og[g] / lg[g] : 0.f);
        } else {
            const long long row0 = ((long long)b * p.q_heads + kvh * G) * p.max_splits;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const long long row = row0 + (long long)g * p.max_splits + split;
                p.part_o[row * 128 + d] = og[g];
                if (d == 0) { p.part_m[row] = m_ref[g]; p.part_l[row] = lg[g]; }
            }
            __threadfence();
            softmax_bar();
            if (threadIdx.x == 0) {
                unsigned* ctr = p.counters + b * p.kv_heads + kvh;
                const unsigned prev = atomicAdd(ctr, 1u);
                s_last = (prev == (unsigned)n_splits - 1);
                if (s_last) *ctr = 0;
            }
            softmax_bar();
            if (s_last) {
                __threadfence();
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const long long row = row0 + (long long)g * p.max_splits;
                    p.out[((long long)b * p.q_heads + kvh * G + g) * 128 + d] =
                        __float2bfloat16(combine_splits(p.part_m + row, p.part_l + row, p.part_o + row * 128 + d, 128, n_splits));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, 64);
}

template <int G>
cudaError_t launch_tc_g(const PagedAttnParams& p, const CUtensorMap& tm, cudaStream_t stream) {
    auto kern = paged_attn_tc_kernel<G>;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kern), TC_SMEM, &attr_mask); e != cudaSuccess) return e;
    const dim3 grid((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens, p.kv_heads, p.batch);
    return launch_pdl(kern, grid, dim3(TC_THREADS), (size_t)TC_SMEM, stream, tm, p);
}

}  // namespace

// `pool_rows`: number of 128-element rows from p.kv (the layer's first page) to the end of the pool allocation.
cudaError_t launch_paged_attn_decode_tc(const PagedAttnParams& p, long long pool_rows, cudaStream_t stream) {
    if (p.head_dim != 128 || p.block_tokens != 16 || p.kv_heads < 1 || p.q_heads % p.kv_heads) return cudaErrorInvalidValue;
    if (p.chunk_tokens % TILE_TOK != 0 || p.chunk_tokens <= 0) return cudaErrorInvalidValue;
    if ((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens > p.max_splits) return cudaErrorInvalidValue;
    if (p.max_blocks <= 0 || (long long)p.max_ctx > (long long)p.max_blocks * 16) return cudaErrorInvalidValue;   // the table row must cover max_ctx
    if ((p.block_stride | p.kv_stride | p.head_stride) & 127) return cudaErrorInvalidValue;   // rows of 128 elements
    if (pool_rows <= 0 || pool_rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    CUtensorMap tm;
    if (!make_tmap_bf16_2d(&tm, p.kv, pool_rows, 128, 128, 16)) return cudaErrorInvalidValue;
    switch (p.q_heads / p.kv_heads) {
        case 1: return launch_tc_g<1>(p, tm, stream);
        case 2: return launch_tc_g<2>(p, tm, stream);
        case 4: return launch_tc_g<4>(p, tm, stream);
        case 8: return launch_tc_g<8>(p, tm, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sky
