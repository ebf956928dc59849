// Paged GQA decode attention on the 5th-generation tensor cores.
//
// Same contract as paged_attn.cu (one query token per sequence, G query heads per KV head, head_dim 128,
// bf16 head-major pages of 16 tokens, split-KV with an in-kernel last-CTA combine), different engine:
//
//   warp 4   : TMA producer. K and V tiles of 128 tokens land in a ring of three 32 KB units (K0, V0, K1, ...), small
//              enough for two CTAs per SM. No cluster broadcast. One tensor-map box per page: the SM's TMA unit takes
//              a request about every 37 ns whatever its size (measured with timestamps in this kernel: a unit of 16
//              two-kilobyte boxes took 0.6 us to issue and 2.3-3.4 us to arrive on an idle GPU), so the request
//              count, not the bytes, bounded what one CTA could keep in flight. A page [16 tokens][128 dims] is
//              4 KB contiguous; a five-dimensional map (64 dims, 8 tokens, 2 halves of head_dim, 2 token groups,
//              page) brings it in one request and lays it down as [token group][half][8 tokens][128 bytes], which
//              both MMAs address with plain strides (8-token groups 2 KB apart, halves 1 KB apart). Where the
//              driver does not take that map, two boxes per page ([16 tokens] x [64 dims]) as before.
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

// Pages of [16 tokens][128 dims] bf16 (4 KB, contiguous) as a five-dimensional tensor: (64 dims, 8 tokens, 2 halves of the
// head dimension, 2 groups of 8 tokens, page slot); the box is one whole page. In shared memory the page becomes
// [token group][half][8 tokens][64 dims] with the 128-byte swizzle: 1 KB atoms of 8 rows, as the MMA descriptors expect.
static bool make_tmap_kv_pages(CUtensorMap* m, const void* base, long long n_slots) {
    typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                           const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Fn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) ptr = nullptr;
        return reinterpret_cast<Fn>(ptr);
    }();
    if (!fn || n_slots <= 0 || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
    cuuint64_t dims[5] = {64, 8, 2, 2, (cuuint64_t)n_slots};
    cuuint64_t strides[4] = {256, 128, 2048, 4096};          // bytes, for dimensions 1..4
    cuuint32_t box[5] = {64, 8, 2, 2, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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

template <int G, bool PAGE_BOX>
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
    if (threadIdx.x == 4 * 32) tma_prefetch_desc(&tmap);
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
    // The producer warp needs the block list only: it starts the first loads now, while the other warps bring in Q.
    if (warp != 4) {
        const int tid = warp < 4 ? threadIdx.x : threadIdx.x - 32;      // 0..159 over the warps that meet below
        for (int i = tid; i < G * 16; i += TC_THREADS - 32) {           // 16-byte chunks: G rows x 16 chunks
            const int g = i >> 4, c = i & 15;
            const uint4 v = *reinterpret_cast<const uint4*>(p.q + ((long long)b * p.q_heads + kvh * G + g) * 128 + c * 8);
            *reinterpret_cast<uint4*>(q_sm + (c >> 3) * 2048 + sw128_off(g, (c & 7) * 8)) = v;
        }
        fence_proxy_async();
        tc_fence_before();
        asm volatile("bar.sync 2, 160;" ::: "memory");
        tc_fence_after();
    }
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tm_s[2] = {tmem_base, tmem_base + 16};
    const uint32_t tm_o = tmem_base + 32;

    float m_ref[GL], l_part[GL];
#pragma unroll
    for (int g = 0; g < GL; ++g) { m_ref[g] = -INFINITY; l_part[g] = 0.f; }
    bool ok = true;

    if (warp == 4) {
        // ---------------- TMA producer ----------------
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
            if (PAGE_BOX) {
                if (lane < 8) {                       // one request per page
                    const int blk = s_blocks[(u >> 1) * 8 + lane];
                    const long long row = ((long long)blk * p.block_stride >> 7) + head_rows + ((u & 1) ? (p.kv_stride >> 7) : 0);
                    tma_load_5d(st + lane * 4096, &tmap, 0, 0, 0, 0, (int)(row >> 4), &full_bar[s]);
                }
            } else if (lane < 16) {
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
            // Two kinds of work, each ready at its own time: the scores of tile i (needs K_i in its unit, and the score
            // buffer i & 1 free: the softmax of tile i - 2 has handed in its P), and P.V of tile i (needs P_i and V_i). They are
            // issued in whichever order they become ready. Waiting for K_{i+1} before P.V of tile i, as a fixed order would,
            // held back the release of V_i's unit, and with it the next load, by the whole latency of a load (timestamps in
            // this kernel on an idle GPU: P_0 written at 3.8 us, its P.V issued at 5.8 us, after K_1 had arrived).
            auto issue_s = [&](int i) {
                const int u = 2 * i, s = u % TC_UNITS;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t a = PAGE_BOX ? umma_desc_k_sw128_sbo(k_addr + (j >> 2) * 1024 + (j & 3) * 32, 2048)
                                                : umma_desc_k_sw128(k_addr + (j >> 2) * HALF_BYTES + (j & 3) * 32);
                    const uint64_t bq = umma_desc_k_sw128(q_addr + (j >> 2) * 2048 + (j & 3) * 32);
                    tc_mma_f16(tm_s[i & 1], a, bq, idesc_s, j ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);     // K of this tile is free once the scores are done
                tc_commit(&s_ready[i & 1]);
            };
            auto issue_pv = [&](int i) {
                const int u = 2 * i + 1, s = u % TC_UNITS;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint64_t a = PAGE_BOX ? umma_desc_mn_sw128(v_addr + j * 4096, 1024, 2048) : umma_desc_mn_sw128(v_addr + j * 2048, HALF_BYTES, 1024);
                    const uint64_t bp = umma_desc_k_sw128(p_addr + (i & 1) * QP_BYTES + (j >> 2) * 2048 + (j & 3) * 32);
                    tc_mma_f16(tm_o, a, bp, idesc_o, (i | j) ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);     // V of this tile is free again
                tc_commit(&o_done[i & 1]);    // this tile's P buffer is free again; the accumulator may be touched
            };
            int next_s = 0, next_pv = 0;
            unsigned idle = 0;
            unsigned long long t_idle = 0;
            while (next_pv < n_tiles) {
                bool did = false;
                if (next_s < n_tiles && next_s <= next_pv + 1) {
                    const int u = 2 * next_s;
                    if (mbar_try_wait(&full_bar[u % TC_UNITS], (u / TC_UNITS) & 1)) { issue_s(next_s); ++next_s; did = true; }
                }
                if (next_pv < next_s) {
                    const int u = 2 * next_pv + 1;
                    if (mbar_try_wait(&p_ready[next_pv & 1], (next_pv >> 1) & 1) && mbar_try_wait(&full_bar[u % TC_UNITS], (u / TC_UNITS) & 1)) {
                        issue_pv(next_pv);
                        ++next_pv;
                        did = true;
                    }
                }
                if (did) { idle = 0; continue; }
                // nothing was ready: bounded, as every wait in this kernel (200 ms without progress)
                if (++idle == 64) t_idle = globaltimer_ns();
                else if (idle > 64 && (idle & 63) == 0 && globaltimer_ns() - t_idle > 200000000ull) {
                    set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, next_pv < next_s ? 13 : 12);
                    break;
                }
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
                // all heads' partials are loaded before the first store: a store between two combines would keep the compiler
                // from moving the next head's loads above it, and every combine is two or three dependent L2 round trips
                float res[G];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const long long row = row0 + (long long)g * p.max_splits;
                    res[g] = combine_splits(p.part_m + row, p.part_l + row, p.part_o + row * 128 + d, 128, n_splits);
                }
#pragma unroll
                for (int g = 0; g < G; ++g) p.out[((long long)b * p.q_heads + kvh * G + g) * 128 + d] = __float2bfloat16(res[g]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, 64);
}

template <int G, bool PAGE_BOX>
cudaError_t launch_tc_g(const PagedAttnParams& p, const CUtensorMap& tm, cudaStream_t stream) {
    auto kern = paged_attn_tc_kernel<G, PAGE_BOX>;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kern), TC_SMEM, &attr_mask); e != cudaSuccess) return e;
    const dim3 grid((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens, p.kv_heads, p.batch);
    return launch_pdl(kern, grid, dim3(TC_THREADS), (size_t)TC_SMEM, stream, tm, p);
}

}  // namespace

static int g_page_box = -1;
// 1 if the last launch fetched whole pages (one request per page), 0 if it fell back to two boxes per page, -1 before any launch.
int paged_attn_tc_page_box() { return g_page_box; }

// `pool_rows`: number of 128-element rows from p.kv (the layer's first page) to the end of the pool allocation.
cudaError_t launch_paged_attn_decode_tc(const PagedAttnParams& p, long long pool_rows, cudaStream_t stream) {
    if (p.head_dim != 128 || p.block_tokens != 16 || p.kv_heads < 1 || p.q_heads % p.kv_heads) return cudaErrorInvalidValue;
    if (p.chunk_tokens % TILE_TOK != 0 || p.chunk_tokens <= 0) return cudaErrorInvalidValue;
    if ((p.max_ctx + p.chunk_tokens - 1) / p.chunk_tokens > p.max_splits) return cudaErrorInvalidValue;
    if (p.max_blocks <= 0 || (long long)p.max_ctx > (long long)p.max_blocks * 16) return cudaErrorInvalidValue;   // the table row must cover max_ctx
    if ((p.block_stride | p.kv_stride | p.head_stride) & 127) return cudaErrorInvalidValue;   // rows of 128 elements
    if (pool_rows <= 0 || pool_rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    CUtensorMap tm;
    // one box per page needs every page on a 4 KB boundary from p.kv (head-major pools are) and a driver that takes the map
    const bool aligned = ((p.block_stride | p.kv_stride | p.head_stride) & 2047) == 0;
    // SKYGDR_ATTN_TWO_BOXES=1 keeps the two-boxes-per-page fetch (the switch the two were measured against each other with:
    // 167.6 against 171.3 us at batch 16, 540 against 553 us at batch 64, contexts 8k-16k)
    static const bool two_boxes = [] { const char* v = getenv("SKYGDR_ATTN_TWO_BOXES"); return v && v[0] == '1'; }();
    if (aligned && !two_boxes && make_tmap_kv_pages(&tm, p.kv, pool_rows / 16)) {
        g_page_box = 1;
        switch (p.q_heads / p.kv_heads) {
            case 1: return launch_tc_g<1, true>(p, tm, stream);
            case 2: return launch_tc_g<2, true>(p, tm, stream);
            case 4: return launch_tc_g<4, true>(p, tm, stream);
            case 8: return launch_tc_g<8, true>(p, tm, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    if (!make_tmap_bf16_2d(&tm, p.kv, pool_rows, 128, 128, 16)) return cudaErrorInvalidValue;
    g_page_box = 0;
    switch (p.q_heads / p.kv_heads) {
        case 1: return launch_tc_g<1, false>(p, tm, stream);
        case 2: return launch_tc_g<2, false>(p, tm, stream);
        case 4: return launch_tc_g<4, false>(p, tm, stream);
        case 8: return launch_tc_g<8, false>(p, tm, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sky
