// Causal prefill attention on the 5th-generation tensor cores, reading K and V straight from the paged pool.
//
// One CTA per (query tile of 128 tokens, query head, prompt). Query rows are the MMA's M, so TMEM lane t holds query
// row t and the softmax of a row lives in one thread: no shuffles, no exchange through shared memory.
//
//   warp 8   : TMA producer. Q tile once (two boxes of [128 tokens] x [64 dims]); then per key tile of 128 tokens
//              K and V, each as 8 pages x 2 dim halves of [16 tokens] x [64 dims], 128-byte swizzle, into a ring of
//              three 32 KB units (K0, V0, K1, ...). The pool is addressed through one 3-D tensor map
//              {128 dims, rows between tokens, token rows}, which covers head-major and token-major pages alike.
//   warp 9   : MMA issuer and TMEM owner (512 columns: two score buffers of 128 and the output accumulator of 128).
//                S[128 q x 128 keys]  = Q[128 x 128] . K_tile^T          (A, B K-major)
//                O[128 q x 128 dims] += P[128 x 128] . V_tile             (A = P K-major, B = V as stored, MN-major)
//              The next tile's scores are issued before this tile's P.V, so the softmax of tile j+1 can start while the
//              tensor core works on tile j.
//   warps 0-7: softmax, two warpgroups. Query row r belongs to thread r of each warpgroup; warpgroup 0 owns key columns
//              0-63 of the tile (and output dims 0-63), warpgroup 1 columns 64-127. A thread reads its 64 scores from
//              TMEM in one go, the two halves of a row exchange their maxima through shared memory, then each thread
//              masks (diagonal tile only), exponentiates, writes its half of the P row as bf16 into the swizzled operand
//              layout and keeps a partial row sum. The running maximum is raised lazily (only when a tile exceeds it by 8
//              in log2 units) and then the accumulator row is rescaled in TMEM. The epilogue divides by the row sum and
//              writes bf16 rows.
// Causality skips key tiles above the diagonal, so a query tile at position qt does qt + 1 key tiles; CTAs are
// launched heaviest first. The four query heads of a KV head run next to one another (head is the fastest grid
// dimension) and find each other's K/V tiles in L2.
#include <cuda.h>

#include "common.cuh"
#include "prefill_attn.h"

namespace sky {
namespace {

constexpr int PF_THREADS = 320;
constexpr int PF_TILE = 128;
constexpr int PF_UNITS = 4;                        // K(j), V(j), K(j+1), V(j+1): the next tile loads while this one is computed
constexpr int PF_HALF = PF_TILE * 64 * 2;          // [128 rows][64 cols] bf16, swizzled: 16 KB
constexpr int PF_TILE_BYTES = 2 * PF_HALF;         // 32 KB: Q tile, K tile, V tile, P tile
constexpr int PF_TILES_BYTES = PF_TILE_BYTES * (1 + PF_UNITS + 2);       // Q, the ring, two P buffers: 224 KB
constexpr int PF_SMEM = PF_TILES_BYTES + 2 * 2 * PF_TILE * 4 + 256;       // + maxima exchange + barriers; no static shared memory
constexpr float PF_RESCALE = 8.0f;

__device__ __forceinline__ void pf_softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(PF_THREADS, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                         const __grid_constant__ CUtensorMap tmap_kv, const PrefillAttnParams p) {
    // Everything lives in dynamic shared memory (224 KB of tiles leave no room for a static part and an alignment slack): the
    // tiles first, since the 128-byte swizzle wants them on 1024-byte boundaries, then the exchange array and the barriers.
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* q_sm = smem;
    unsigned char* ring = smem + PF_TILE_BYTES;
    unsigned char* p_sm = ring + PF_UNITS * PF_TILE_BYTES;
    float (*xch)[2][PF_TILE] = reinterpret_cast<float (*)[2][PF_TILE]>(smem + PF_TILES_BYTES);      // [tile parity][warpgroup][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PF_TILES_BYTES + 2 * 2 * PF_TILE * 4);
    uint64_t* full_bar = bars;                        // [PF_UNITS]
    uint64_t* empty_bar = bars + PF_UNITS;            // [PF_UNITS]
    uint64_t* s_ready = bars + 2 * PF_UNITS;          // [2]
    uint64_t* p_ready = s_ready + 2;                  // [2]
    uint64_t* o_done = p_ready + 2;                   // [2]
    uint64_t& q_full = *(o_done + 2);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(o_done + 3);
    if (smem_u32(smem) & 1023) {                      // the swizzled tiles would be misread: report instead of computing garbage
        if (threadIdx.x == 0) set_status(p.status, SKY_STATUS_BAD_INDEX, 49);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.z;
    const int tok_base = p.seq_start[seq];
    const int n = p.seq_start[seq + 1] - tok_base;                       // prompt length
    const int q_tiles = (n + PF_TILE - 1) / PF_TILE;
    const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;                 // heaviest query tiles first
    if (qt >= q_tiles) return;                                           // whole CTA leaves together, before any barrier
    const int n_kt = qt + 1;                                             // key tiles 0..qt (causal)
    const int kvh = head / (p.q_heads / p.kv_heads);
    const int* table = p.block_table + (long long)seq * p.max_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_UNITS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&q_full, 1);
        mbar_init(&s_ready[0], 1); mbar_init(&s_ready[1], 1);
        mbar_init(&p_ready[0], 256); mbar_init(&p_ready[1], 256);
        mbar_init(&o_done[0], 1); mbar_init(&o_done[1], 1);
        fence_barrier_init();
    }
    if (warp == 9) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tm_s[2] = {tmem_base, tmem_base + 128};
    const uint32_t tm_o = tmem_base + 256;

    if (warp == 8) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_kv);
            mbar_expect_tx(&q_full, PF_TILE_BYTES);
            tma_load_3d(q_sm, &tmap_q, 0, head, tok_base + qt * PF_TILE, &q_full);
            tma_load_3d(q_sm + PF_HALF, &tmap_q, 64, head, tok_base + qt * PF_TILE, &q_full);
        }
        const int ts_rows = (int)(p.tok_stride >> 7);                    // 128-element rows between two tokens of a page
        const long long head_row = (long long)kvh * (p.head_stride >> 7);
        const int pg = lane >> 1, half = lane & 1;                       // lanes 0-15: page pg, dim half
        for (int u = 0; u < 2 * n_kt; ++u) {
            const int s = u % PF_UNITS;
            if (u >= PF_UNITS && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (uint32_t)((u / PF_UNITS) - 1) & 1))) {
                if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 41);
                break;
            }
            unsigned char* st = ring + s * PF_TILE_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[s], PF_TILE_BYTES);
            __syncwarp();
            if (lane < 16) {
                const int e = (u >> 1) * 8 + pg;
                const int blk = e < p.max_blocks ? __ldg(table + e) : 0;
                const long long row0 = ((long long)blk * p.block_stride >> 7) + ((u & 1) ? (p.kv_stride >> 7) : 0) + head_row;
                tma_load_3d(st + half * PF_HALF + pg * 2048, &tmap_kv, half * 64, (int)(row0 % ts_rows), (int)(row0 / ts_rows), &full_bar[s]);
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128);                     // Q K-major x K K-major
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);        // P K-major x V MN-major
            const uint32_t q_addr = smem_u32(q_sm), p_addr = smem_u32(p_sm);
            bool good = mbar_wait(&q_full, 0);
            if (!good) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 42);
            auto issue_s = [&](int j) -> bool {
                const int u = 2 * j, s = u % PF_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 43); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(ring + s * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {                                        // 8 steps of 16 dims
                    const uint64_t a = umma_desc_k_sw128(q_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    const uint64_t b = umma_desc_k_sw128(k_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    tc_mma_f16(tm_s[j & 1], a, b, idesc_s, k ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);        // the K tile is free once the scores are done
                tc_commit(&s_ready[j & 1]);
                return true;
            };
            if (good) good = issue_s(0);
            for (int j = 0; j < n_kt && good; ++j) {
                if (j + 1 < n_kt) good = issue_s(j + 1);
                if (!good) break;
                if (!mbar_wait(&p_ready[j & 1], (uint32_t)(j >> 1) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 44); break; }
                const int u = 2 * j + 1, s = u % PF_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 45); break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(ring + s * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {                                        // 8 steps of 16 keys
                    const uint64_t a = umma_desc_k_sw128(p_addr + (j & 1) * PF_TILE_BYTES + (k >> 2) * PF_HALF + (k & 3) * 32);
                    const uint64_t b = umma_desc_mn_sw128(v_addr + k * 2048, PF_HALF, 1024);
                    tc_mma_f16(tm_o, a, b, idesc_o, (j | k) ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);        // the V tile is free again
                tc_commit(&o_done[j & 1]);       // this tile's P buffer is free; the accumulator may be touched
            }
        }
    } else {
        // ---------------- softmax warpgroups: thread (wg, r) <-> half of query row r ----------------
        const int wg = warp >> 2;                                        // 0: key columns / output dims 0-63, 1: 64-127
        const int r = threadIdx.x & 127;                                 // query row of the tile = TMEM lane
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;     // a warp reaches the TMEM lanes of its rank in the warpgroup
        const int col0 = wg * 64;
        const float qs = p.scale * 1.4426950408889634f;
        const int qpos_raw = qt * PF_TILE + r;
        const bool row_valid = qpos_raw < n;
        const int qpos = row_valid ? qpos_raw : n - 1;                   // rows past the prompt compute something finite, unused
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kt; ++j) {
            const int par = j & 1;
            // A wait that runs out does not leave the loop: the thread keeps taking part in the named barrier and the P
            // arrivals (so that nobody waits for it without a bound) and only stops waiting itself.
            if (ok && !mbar_wait(&s_ready[par], (uint32_t)(j >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 46); ok = false; }
            tc_fence_after();
            uint32_t sc[64];
            tmem_ld_x32(tm_s[par] + lane_off + col0, sc);
            tmem_ld_x32(tm_s[par] + lane_off + col0 + 32, sc + 32);
            tc_wait_ld();
            const bool diag = j == qt;
            const int kbase = j * PF_TILE + col0;
            // Maximum of the raw scores (the scale is positive, so it commutes); masked entries of the diagonal tile become -inf.
            float tmax = -INFINITY;
            if (diag) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int kpos = kbase + i;
                    if (kpos > qpos || kpos >= n) sc[i] = 0xff800000u;      // -inf
                    tmax = fmaxf(tmax, __uint_as_float(sc[i]));
                }
            } else {
                float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    t0 = fmaxf(t0, __uint_as_float(sc[i]));
                    t1 = fmaxf(t1, __uint_as_float(sc[i + 1]));
                    t2 = fmaxf(t2, __uint_as_float(sc[i + 2]));
                    t3 = fmaxf(t3, __uint_as_float(sc[i + 3]));
                }
                tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
            }
            tmax *= qs;
            xch[par][wg][r] = tmax;
            pf_softmax_bar();                                            // both halves of every row have posted their maxima
            tmax = fmaxf(tmax, xch[par][wg ^ 1][r]);
            float alpha = 1.0f;
            const bool raise = tmax > m_ref + PF_RESCALE || m_ref == -INFINITY;        // same decision in both threads of a row
            if (raise) {
                alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - tmax);
                m_ref = tmax;
            }
            const bool any_raise = __any_sync(0xffffffffu, raise) && j > 0;      // tcgen05.ld/st are warp-wide: decide per warp
            // P buffer `par` was last read by the P.V of tile j-2; a rescale waits for tile j-1 (in-order completion covers j-2).
            if (any_raise) {
                if (ok && !mbar_wait(&o_done[(j - 1) & 1], (uint32_t)((j - 1) >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 47); ok = false; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 16) {                   // this thread's half of the accumulator row
                    uint32_t o[16];
                    tmem_ld_x16(tm_o + lane_off + col0 + c0, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_x16(tm_o + lane_off + col0 + c0, o);
                }
                tc_wait_st();
            } else if (j > 1) {
                if (ok && !mbar_wait(&o_done[par], (uint32_t)((j - 2) >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 47); ok = false; }
            }
            l_sum *= alpha;
            // exponentials -> this thread's 64 keys of the P row (bf16, swizzled operand layout), partial row sum
            unsigned char* prow = p_sm + par * PF_TILE_BYTES + wg * PF_HALF;
            const float neg_m = -m_ref;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = exp2f(fmaf(__uint_as_float(sc[c + i]), qs, neg_m));      // masked scores are -inf: 0
                s0 += e[0] + e[4]; s1 += e[1] + e[5]; s2 += e[2] + e[6]; s3 += e[3] + e[7];
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(e[i], e[i + 1]);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(prow + sw128_off(r, c)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            l_sum += (s0 + s1) + (s2 + s3);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_ready[par]);
        }
        if (ok && !mbar_wait(&o_done[(n_kt - 1) & 1], (uint32_t)((n_kt - 1) >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 48); ok = false; }
        tc_fence_after();
        // ---------------- epilogue: this thread's 64 dims of output row r ----------------
        pf_softmax_bar();                                                // every thread is past its last read of xch
        xch[0][wg][r] = l_sum;
        pf_softmax_bar();
        const float l_row = l_sum + xch[0][wg ^ 1][r];
        const float inv = (ok && l_row > 0.f) ? 1.0f / l_row : 0.f;
        __nv_bfloat16* orow = p.out + ((long long)(tok_base + qpos_raw) * p.q_heads + head) * 128 + col0;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t o[16];
            tmem_ld_x16(tm_o + lane_off + col0 + c0, o);
            tc_wait_ld();
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
            }
            if (row_valid) {
                *reinterpret_cast<uint4*>(orow + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA. Tiles A = 2c and B = 2c + 1 of a prompt (256 consecutive queries) share every K/V tile that
// the CTA loads, and their softmax warpgroups work in alternation with the tensor core: while warpgroup A turns its
// scores of key tile j into P, the tensor core runs P.V of tile B and the next scores of B, and the other way round.
// One warpgroup per query tile, one thread per query row (all 128 scores of a row in registers, no exchange between
// threads). TMEM: scores of A and B (single-buffered, 128 columns each) and the two accumulators: 512 columns.
// Shared memory: Q_A, Q_B, a ring of three K/V units, P_A, P_B (single-buffered): 224 KB.
constexpr int PF2_TILES_BYTES = PF_TILE_BYTES * 7;
constexpr int PF2_SMEM = PF2_TILES_BYTES + 256;

// exp2 on the FMA and integer pipes instead of the special-function unit: floor by a round-down add of 1.5 * 2^23, a cubic
// for 2^frac (largest relative error 1.0e-4, far below bf16's 3.9e-3), the integer part added to the exponent field.
// Arguments below -126 return 2^-126 (about 1e-38) instead of 0, which vanishes in a bf16 P and in the row sum.
__device__ __forceinline__ float pf_exp2_poly(float x) {
    x = fmaxf(x, -126.0f);
    float t;
    asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(t) : "f"(x), "f"(12582912.0f));
    const float f = x - (t - 12582912.0f);
    const float pl = fmaf(fmaf(fmaf(0.07826747000217438f, f, 0.22630836069583893f), f, 0.6954241991043091f), f, 1.0f);
    return __uint_as_float(__float_as_uint(pl) + (__float_as_uint(t) << 23));
}

// POLY: how many of every four exponentials take pf_exp2_poly (0 = all on the special-function unit, as measured).
// PTMEM: P is written as packed bf16 over the first 64 columns of its own score buffer in TMEM (lane = query row, two
// keys per column) and the P.V MMA takes its A operand from there; the 64 KB of P tiles in shared memory become two more
// ring units. Neither option has run on a GPU yet; <0, false> is the measured kernel.
template <int POLY, bool PTMEM>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_attn_tc2_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                          const __grid_constant__ CUtensorMap tmap_kv, const PrefillAttnParams p) {
    constexpr int PF2_UNITS = PTMEM ? 5 : 3;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* q_sm = smem;                                        // Q_A, Q_B
    unsigned char* ring = smem + 2 * PF_TILE_BYTES;
    unsigned char* p_sm = ring + PF2_UNITS * PF_TILE_BYTES;            // P_A, P_B (not used with PTMEM: the ring ends where the barriers start)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PF2_TILES_BYTES);
    uint64_t* full_bar = bars;                        // [PF2_UNITS]
    uint64_t* empty_bar = bars + PF2_UNITS;           // [PF2_UNITS]
    uint64_t* s_ready = bars + 2 * PF2_UNITS;         // [2]: per query tile, one completion per key tile
    uint64_t* p_ready = s_ready + 2;                  // [2]
    uint64_t* o_done = p_ready + 2;                   // [2]
    uint64_t& q_full = *(o_done + 2);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(o_done + 3);
    if (smem_u32(smem) & 1023) {
        if (threadIdx.x == 0) set_status(p.status, SKY_STATUS_BAD_INDEX, 59);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.z;
    const int tok_base = p.seq_start[seq];
    const int n = p.seq_start[seq + 1] - tok_base;
    const int q_tiles = (n + PF_TILE - 1) / PF_TILE;
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;               // heaviest pairs first
    if (2 * pair >= q_tiles) return;
    const int qt_x[2] = {2 * pair, 2 * pair + 1};
    const int nkt_x[2] = {qt_x[0] + 1, qt_x[1] < q_tiles ? qt_x[1] + 1 : 0};      // key tiles each query tile needs (0: tile B is past the prompt)
    const int n_kt = max(nkt_x[0], nkt_x[1]);
    const int kvh = head / (p.q_heads / p.kv_heads);
    const int* table = p.block_table + (long long)seq * p.max_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF2_UNITS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&q_full, 1);
        for (int x = 0; x < 2; ++x) { mbar_init(&s_ready[x], 1); mbar_init(&p_ready[x], 128); mbar_init(&o_done[x], 1); }
        fence_barrier_init();
    }
    if (warp == 9) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 8) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_kv);
            mbar_expect_tx(&q_full, 2 * PF_TILE_BYTES);                  // tile B is fetched even when it is past the prompt (zero fill or unused rows)
            for (int x = 0; x < 2; ++x) {
                tma_load_3d(q_sm + x * PF_TILE_BYTES, &tmap_q, 0, head, tok_base + qt_x[x] * PF_TILE, &q_full);
                tma_load_3d(q_sm + x * PF_TILE_BYTES + PF_HALF, &tmap_q, 64, head, tok_base + qt_x[x] * PF_TILE, &q_full);
            }
        }
        const int ts_rows = (int)(p.tok_stride >> 7);
        const long long head_row = (long long)kvh * (p.head_stride >> 7);
        const int pg = lane >> 1, half = lane & 1;
        for (int u = 0; u < 2 * n_kt; ++u) {
            const int s = u % PF2_UNITS;
            if (u >= PF2_UNITS && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (uint32_t)((u / PF2_UNITS) - 1) & 1))) {
                if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 51);
                break;
            }
            unsigned char* st = ring + s * PF_TILE_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[s], PF_TILE_BYTES);
            __syncwarp();
            if (lane < 16) {
                const int e = (u >> 1) * 8 + pg;
                const int blk = e < p.max_blocks ? __ldg(table + e) : 0;
                const long long row0 = ((long long)blk * p.block_stride >> 7) + ((u & 1) ? (p.kv_stride >> 7) : 0) + head_row;
                tma_load_3d(st + half * PF_HALF + pg * 2048, &tmap_kv, half * 64, (int)(row0 % ts_rows), (int)(row0 / ts_rows), &full_bar[s]);
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128);
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);
            bool good = mbar_wait(&q_full, 0);
            if (!good) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 52);
            // scores of query tile x against key tile j; the K unit is released after the last tile that uses it
            auto issue_s = [&](int x, int j) -> bool {
                const int u = 2 * j, s = u % PF2_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF2_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 53); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(ring + s * PF_TILE_BYTES), q_addr = smem_u32(q_sm + x * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t a = umma_desc_k_sw128(q_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    const uint64_t b = umma_desc_k_sw128(k_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    tc_mma_f16(tmem_base + x * 128, a, b, idesc_s, k ? 1u : 0u);
                }
                const bool last_user = x == 1 || j >= nkt_x[1];
                if (last_user) tc_commit(&empty_bar[s]);
                tc_commit(&s_ready[x]);
                return true;
            };
            auto issue_pv = [&](int x, int j) -> bool {
                if (!mbar_wait(&p_ready[x], (uint32_t)j & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 54); return false; }
                const int u = 2 * j + 1, s = u % PF2_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF2_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 55); return false; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(ring + s * PF_TILE_BYTES), p_addr = smem_u32(p_sm + x * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t b = umma_desc_mn_sw128(v_addr + k * 2048, PF_HALF, 1024);
                    if constexpr (PTMEM) {                              // 16 keys of P = 8 columns of packed bf16 in the score buffer
                        tc_mma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + k * 8, b, idesc_o, (j | k) ? 1u : 0u);
                    } else {
                        const uint64_t a = umma_desc_k_sw128(p_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                        tc_mma_f16(tmem_base + 256 + x * 128, a, b, idesc_o, (j | k) ? 1u : 0u);
                    }
                }
                const bool last_user = x == 1 || j >= nkt_x[1];
                if (last_user) tc_commit(&empty_bar[s]);
                tc_commit(&o_done[x]);
                return true;
            };
            if (good) good = issue_s(0, 0);
            if (good && nkt_x[1] > 0) good = issue_s(1, 0);
            for (int j = 0; j < n_kt && good; ++j) {
                for (int x = 0; x < 2 && good; ++x) {
                    if (j >= nkt_x[x]) continue;
                    good = issue_pv(x, j);
                    if (good && j + 1 < nkt_x[x]) good = issue_s(x, j + 1);     // its score buffer is free: the P of tile j has been written
                }
            }
        }
    } else {
        // ---------------- softmax warpgroups: warpgroup x <-> query tile x, thread r <-> query row r ----------------
        const int x = warp >> 2;
        const int r = threadIdx.x & 127;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_s = tmem_base + x * 128, tm_o = tmem_base + 256 + x * 128;
        const int qt = qt_x[x], my_kt = nkt_x[x];
        const float qs = p.scale * 1.4426950408889634f;
        const int qpos_raw = qt * PF_TILE + r;
        const bool row_valid = my_kt > 0 && qpos_raw < n;
        const int qpos = qpos_raw < n ? qpos_raw : n - 1;
        unsigned char* prow = p_sm + x * PF_TILE_BYTES;
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < my_kt; ++j) {
            // A wait that runs out does not leave the loop: the thread keeps arriving, so that nobody waits for it without a bound.
            if (ok && !mbar_wait(&s_ready[x], (uint32_t)j & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 56); ok = false; }
            tc_fence_after();
            uint32_t sc[128];
            tmem_ld_x32(tm_s + lane_off, sc);
            tmem_ld_x32(tm_s + lane_off + 32, sc + 32);
            tmem_ld_x32(tm_s + lane_off + 64, sc + 64);
            tmem_ld_x32(tm_s + lane_off + 96, sc + 96);
            tc_wait_ld();
            const int kbase = j * PF_TILE;
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
            if (j == qt) {                                                 // the diagonal tile: causal mask and the prompt's end
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    const int kpos = kbase + i;
                    if (kpos > qpos || kpos >= n) sc[i] = 0xff800000u;     // -inf
                }
            }
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                t0 = fmaxf(t0, __uint_as_float(sc[i]));
                t1 = fmaxf(t1, __uint_as_float(sc[i + 1]));
                t2 = fmaxf(t2, __uint_as_float(sc[i + 2]));
                t3 = fmaxf(t3, __uint_as_float(sc[i + 3]));
            }
            const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * qs;
            float alpha = 1.0f;
            const bool raise = tmax > m_ref + PF_RESCALE || m_ref == -INFINITY;
            if (raise) {
                alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - tmax);
                m_ref = tmax;
            }
            // P_x is single-buffered and the accumulator may only be touched between two P.V: wait for the P.V of tile j-1.
            if (j > 0 && ok && !mbar_wait(&o_done[x], (uint32_t)(j - 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 57); ok = false; }
            if (j > 0 && __any_sync(0xffffffffu, raise)) {                 // tcgen05.ld/st are warp-wide: decide per warp
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 16) {
                    uint32_t o[16];
                    tmem_ld_x16(tm_o + lane_off + c0, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_x16(tm_o + lane_off + c0, o);
                }
                tc_wait_st();
            }
            l_sum *= alpha;
            const float neg_m = -m_ref;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            if constexpr (!PTMEM) {
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = fmaf(__uint_as_float(sc[c + i]), qs, neg_m);
                        e[i] = (i & 3) < POLY ? pf_exp2_poly(a) : exp2f(a);
                    }
                    s0 += e[0] + e[4]; s1 += e[1] + e[5]; s2 += e[2] + e[6]; s3 += e[3] + e[7];
                    uint32_t packed[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const __nv_bfloat162 b2 = __floats2bfloat162_rn(e[i], e[i + 1]);
                        packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
                    }
                    *reinterpret_cast<uint4*>(prow + (c >> 6) * PF_HALF + sw128_off(r, c & 63)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
                l_sum += (s0 + s1) + (s2 + s3);
                fence_proxy_async();
            } else {
                // every lane of the warp has its 128 scores in registers (the load above was warp-wide and waited for), and the
                // next score MMA of this tile is issued only after the P.V that reads these columns: the buffer is ours
#pragma unroll
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t pk[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float e[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float a = fmaf(__uint_as_float(sc[c0 + c + i]), qs, neg_m);
                            e[i] = i < POLY ? pf_exp2_poly(a) : exp2f(a);
                        }
                        s0 += e[0]; s1 += e[1]; s2 += e[2]; s3 += e[3];
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(e[0], e[1]), hi = __floats2bfloat162_rn(e[2], e[3]);
                        pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&lo);
                        pk[(c >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&hi);
                    }
                    tmem_st_x16(tm_s + lane_off + (c0 >> 1), pk);
                }
                l_sum += (s0 + s1) + (s2 + s3);
                tc_wait_st();
            }
            tc_fence_before();
            mbar_arrive(&p_ready[x]);
        }
        if (my_kt > 0) {
            if (ok && !mbar_wait(&o_done[x], (uint32_t)(my_kt - 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 58); ok = false; }
            tc_fence_after();
            const float inv = (ok && l_sum > 0.f) ? 1.0f / l_sum : 0.f;
            __nv_bfloat16* orow = p.out + ((long long)(tok_base + qpos_raw) * p.q_heads + head) * 128;
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t o[16];
                tmem_ld_x16(tm_o + lane_off + c0, o);
                tc_wait_ld();
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                if (row_valid) {
                    *reinterpret_cast<uint4*>(orow + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA with key steps of 64. Same roles, rings and tiles as the kernel above, but every 128-token
// K/V tile is consumed as two steps of 64 keys, so that each query tile can keep TWO score buffers in TMEM
// (2 tiles x 2 buffers x 64 columns + 2 accumulators x 128 columns = 512 columns): the scores of step t+1 are computed
// while the warpgroup still works on step t, and a softmax warpgroup never waits for its own score MMA. P is
// double-buffered the same way (2 x 16 KB per query tile, the space of one 32 KB buffer).
// Barriers per query tile x: s_ready[x][t&1], p_ready[x][t&1], o_done[x][t&1], one completion each per step of that parity.
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_attn_tc3_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                          const __grid_constant__ CUtensorMap tmap_kv, const PrefillAttnParams p) {
    constexpr int PF2_UNITS = 3;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* q_sm = smem;                                        // Q_A, Q_B
    unsigned char* ring = smem + 2 * PF_TILE_BYTES;
    unsigned char* p_sm = ring + PF2_UNITS * PF_TILE_BYTES;            // P_A[2], P_B[2]: four [128 q][64 keys] halves
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PF2_TILES_BYTES);
    uint64_t* full_bar = bars;                        // [PF2_UNITS]
    uint64_t* empty_bar = bars + PF2_UNITS;           // [PF2_UNITS]
    uint64_t* s_ready = bars + 2 * PF2_UNITS;         // [2 tiles][2 parities]
    uint64_t* p_ready = s_ready + 4;                  // [2][2]
    uint64_t* o_done = p_ready + 4;                   // [2][2]
    uint64_t& q_full = *(o_done + 4);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(o_done + 5);
    if (smem_u32(smem) & 1023) {
        if (threadIdx.x == 0) set_status(p.status, SKY_STATUS_BAD_INDEX, 69);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, seq = blockIdx.z;
    const int tok_base = p.seq_start[seq];
    const int n = p.seq_start[seq + 1] - tok_base;
    const int q_tiles = (n + PF_TILE - 1) / PF_TILE;
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;
    if (2 * pair >= q_tiles) return;
    const int qt_x[2] = {2 * pair, 2 * pair + 1};
    const int nkt_x[2] = {qt_x[0] + 1, qt_x[1] < q_tiles ? qt_x[1] + 1 : 0};      // 128-token key tiles per query tile
    const int n_kt = max(nkt_x[0], nkt_x[1]);
    const int kvh = head / (p.q_heads / p.kv_heads);
    const int* table = p.block_table + (long long)seq * p.max_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF2_UNITS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&q_full, 1);
        for (int i = 0; i < 4; ++i) { mbar_init(&s_ready[i], 1); mbar_init(&p_ready[i], 128); mbar_init(&o_done[i], 1); }
        fence_barrier_init();
    }
    if (warp == 9) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;                               // scores: x * 128 + buffer * 64; accumulators: 256 + x * 128

    if (warp == 8) {
        // ---------------- TMA producer (as in the kernel above) ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_kv);
            mbar_expect_tx(&q_full, 2 * PF_TILE_BYTES);
            for (int x = 0; x < 2; ++x) {
                tma_load_3d(q_sm + x * PF_TILE_BYTES, &tmap_q, 0, head, tok_base + qt_x[x] * PF_TILE, &q_full);
                tma_load_3d(q_sm + x * PF_TILE_BYTES + PF_HALF, &tmap_q, 64, head, tok_base + qt_x[x] * PF_TILE, &q_full);
            }
        }
        const int ts_rows = (int)(p.tok_stride >> 7);
        const long long head_row = (long long)kvh * (p.head_stride >> 7);
        const int pg = lane >> 1, half = lane & 1;
        for (int u = 0; u < 2 * n_kt; ++u) {
            const int s = u % PF2_UNITS;
            if (u >= PF2_UNITS && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (uint32_t)((u / PF2_UNITS) - 1) & 1))) {
                if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 61);
                break;
            }
            unsigned char* st = ring + s * PF_TILE_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[s], PF_TILE_BYTES);
            __syncwarp();
            if (lane < 16) {
                const int e = (u >> 1) * 8 + pg;
                const int blk = e < p.max_blocks ? __ldg(table + e) : 0;
                const long long row0 = ((long long)blk * p.block_stride >> 7) + ((u & 1) ? (p.kv_stride >> 7) : 0) + head_row;
                tma_load_3d(st + half * PF_HALF + pg * 2048, &tmap_kv, half * 64, (int)(row0 % ts_rows), (int)(row0 / ts_rows), &full_bar[s]);
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer: steps of 64 keys; step t of a query tile uses key tile t >> 1, half t & 1 ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64);
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);
            bool good = mbar_wait(&q_full, 0);
            if (!good) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 62);
            auto issue_s = [&](int x, int t) -> bool {
                const int j = t >> 1, hb = t & 1, u = 2 * j, s = u % PF2_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF2_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 63); return false; }
                tc_fence_after();
                // rows hb * 64 .. + 63 of the K tile: 64 rows x 128 bytes further into each dim half
                const uint32_t k_addr = smem_u32(ring + s * PF_TILE_BYTES) + hb * 64 * 128, q_addr = smem_u32(q_sm + x * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t a = umma_desc_k_sw128(q_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    const uint64_t b = umma_desc_k_sw128(k_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    tc_mma_f16(tmem_base + x * 128 + (t & 1) * 64, a, b, idesc_s, k ? 1u : 0u);
                }
                const bool last_user = hb == 1 && (x == 1 || j >= nkt_x[1]);
                if (last_user) tc_commit(&empty_bar[s]);
                tc_commit(&s_ready[x * 2 + (t & 1)]);
                return true;
            };
            auto issue_pv = [&](int x, int t) -> bool {
                const int j = t >> 1, hb = t & 1;
                if (!mbar_wait(&p_ready[x * 2 + (t & 1)], (uint32_t)(t >> 1) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 64); return false; }
                const int u = 2 * j + 1, s = u % PF2_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF2_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 65); return false; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(ring + s * PF_TILE_BYTES) + hb * 64 * 128;
                const uint32_t p_addr = smem_u32(p_sm + x * PF_TILE_BYTES + (t & 1) * PF_HALF);
#pragma unroll
                for (int k = 0; k < 4; ++k) {                          // 4 steps of 16 keys
                    const uint64_t a = umma_desc_k_sw128(p_addr + k * 32);
                    const uint64_t b = umma_desc_mn_sw128(v_addr + k * 2048, PF_HALF, 1024);
                    tc_mma_f16(tmem_base + 256 + x * 128, a, b, idesc_o, (t | k) ? 1u : 0u);
                }
                const bool last_user = hb == 1 && (x == 1 || j >= nkt_x[1]);
                if (last_user) tc_commit(&empty_bar[s]);
                tc_commit(&o_done[x * 2 + (t & 1)]);
                return true;
            };
            const int steps_x[2] = {2 * nkt_x[0], 2 * nkt_x[1]};
            const int steps = max(steps_x[0], steps_x[1]);
            for (int t = 0; t < 2 && good; ++t)                        // both score buffers of both tiles
                for (int x = 0; x < 2 && good; ++x)
                    if (t < steps_x[x]) good = issue_s(x, t);
            for (int t = 0; t < steps && good; ++t) {
                for (int x = 0; x < 2 && good; ++x) {
                    if (t >= steps_x[x]) continue;
                    good = issue_pv(x, t);
                    if (good && t + 2 < steps_x[x]) good = issue_s(x, t + 2);      // its buffer is free: the P of step t has been written
                }
            }
        }
    } else {
        // ---------------- softmax warpgroups: warpgroup x <-> query tile x, thread r <-> query row r ----------------
        const int x = warp >> 2;
        const int r = threadIdx.x & 127;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tm_o = tmem_base + 256 + x * 128;
        const int qt = qt_x[x], my_steps = 2 * nkt_x[x];
        const float qs = p.scale * 1.4426950408889634f;
        const int qpos_raw = qt * PF_TILE + r;
        const bool row_valid = my_steps > 0 && qpos_raw < n;
        const int qpos = qpos_raw < n ? qpos_raw : n - 1;
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int t = 0; t < my_steps; ++t) {
            const int par = t & 1, bi = x * 2 + par;
            if (ok && !mbar_wait(&s_ready[bi], (uint32_t)(t >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 66); ok = false; }
            tc_fence_after();
            uint32_t sc[64];
            tmem_ld_x32(tmem_base + x * 128 + par * 64 + lane_off, sc);
            tmem_ld_x32(tmem_base + x * 128 + par * 64 + lane_off + 32, sc + 32);
            tc_wait_ld();
            const int kbase = t * 64;                                    // first key of this step
            if ((t >> 1) == qt) {                                        // the diagonal key tile: causal mask and the prompt's end
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int kpos = kbase + i;
                    if (kpos > qpos || kpos >= n) sc[i] = 0xff800000u;     // -inf
                }
            }
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
                t0 = fmaxf(t0, __uint_as_float(sc[i]));
                t1 = fmaxf(t1, __uint_as_float(sc[i + 1]));
                t2 = fmaxf(t2, __uint_as_float(sc[i + 2]));
                t3 = fmaxf(t3, __uint_as_float(sc[i + 3]));
            }
            const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * qs;      // -inf when the whole step is masked (upper half of a diagonal tile)
            float alpha = 1.0f;
            const bool raise = tmax > m_ref + PF_RESCALE || (m_ref == -INFINITY && tmax > -INFINITY);
            if (raise) {
                alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - tmax);
                m_ref = tmax;
            }
            const bool any_raise = __any_sync(0xffffffffu, raise) && t > 0;
            // P buffer `par` was last read by the P.V of step t-2; a rescale of the accumulator waits for step t-1 as well.
            if (any_raise) {
                if (ok && !mbar_wait(&o_done[x * 2 + ((t - 1) & 1)], (uint32_t)((t - 1) >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 67); ok = false; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 16) {
                    uint32_t o[16];
                    tmem_ld_x16(tm_o + lane_off + c0, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_x16(tm_o + lane_off + c0, o);
                }
                tc_wait_st();
            } else if (t > 1) {
                if (ok && !mbar_wait(&o_done[bi], (uint32_t)((t - 2) >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 67); ok = false; }
            }
            l_sum *= alpha;
            unsigned char* prow = p_sm + x * PF_TILE_BYTES + par * PF_HALF;
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;       // nothing seen yet: every score of this step is -inf, exp2 gives 0
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = exp2f(fmaf(__uint_as_float(sc[c + i]), qs, neg_m));
                s0 += e[0] + e[4]; s1 += e[1] + e[5]; s2 += e[2] + e[6]; s3 += e[3] + e[7];
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(e[i], e[i + 1]);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(prow + sw128_off(r, c)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            l_sum += (s0 + s1) + (s2 + s3);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_ready[bi]);
        }
        if (my_steps > 0) {
            const int tl = my_steps - 1;
            if (ok && !mbar_wait(&o_done[x * 2 + (tl & 1)], (uint32_t)(tl >> 1) & 1)) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 68); ok = false; }
            tc_fence_after();
            const float inv = (ok && l_sum > 0.f) ? 1.0f / l_sum : 0.f;
            __nv_bfloat16* orow = p.out + ((long long)(tok_base + qpos_raw) * p.q_heads + head) * 128;
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t o[16];
                tmem_ld_x16(tm_o + lane_off + c0, o);
                tc_wait_ld();
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                if (row_valid) {
                    *reinterpret_cast<uint4*>(orow + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 512);
}

typedef CUresult (*PfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D bf16 map {128, mid, outer} with box {64, 1, box_outer}, 128-byte swizzle, zero fill outside.
bool pf_make_tmap(CUtensorMap* m, const void* base, long long mid, long long outer, int box_outer) {
    static PfEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return false;
        fn = reinterpret_cast<PfEncodeFn>(ptr);
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || mid < 1 || outer < 1) return false;
    const cuuint64_t dims[3] = {128, (cuuint64_t)mid, (cuuint64_t)outer};
    const cuuint64_t strides[2] = {256, (cuuint64_t)mid * 256};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_outer};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int POLY, bool PTMEM>
cudaError_t pf_launch_tc2(dim3 grid, const CUtensorMap& tq, const CUtensorMap& tkv, const PrefillAttnParams& p, cudaStream_t stream) {
    static unsigned long long attr_mask = 0;             // one per instantiation
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(prefill_attn_tc2_kernel<POLY, PTMEM>), PF2_SMEM, &attr_mask); e != cudaSuccess) return e;
    prefill_attn_tc2_kernel<POLY, PTMEM><<<grid, PF_THREADS, PF2_SMEM, stream>>>(tq, tkv, p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_attn_tc(const PrefillAttnParams& p, long long pool_rows, cudaStream_t stream) {
    if (p.n_seqs < 1 || p.q_heads < 1 || p.kv_heads < 1 || p.q_heads % p.kv_heads || p.max_len < 1 || p.total_tokens < 1) return cudaErrorInvalidValue;
    if ((p.block_stride | p.kv_stride | p.head_stride | p.tok_stride) & 127) return cudaErrorInvalidValue;        // whole rows of 128 elements
    const long long ts_rows = p.tok_stride >> 7;
    if (ts_rows < 1 || pool_rows < ts_rows || pool_rows / ts_rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    // a page's 16 tokens must sit on one middle coordinate: its first row and the head offset may not cross a token row group
    if ((p.block_stride >> 7) % ts_rows || (p.kv_stride >> 7) % ts_rows) return cudaErrorInvalidValue;
    if ((long long)p.kv_heads * (p.head_stride >> 7) > ts_rows && ts_rows != 1) return cudaErrorInvalidValue;
    CUtensorMap tq, tkv;
    if (!pf_make_tmap(&tq, p.q, p.q_heads, p.total_tokens, PF_TILE)) return cudaErrorInvalidValue;
    if (!pf_make_tmap(&tkv, p.kv, ts_rows, pool_rows / ts_rows, 16)) return cudaErrorInvalidValue;
    if (p.two_tiles == 2) {                              // key steps of 64, double-buffered scores (not yet run on a GPU)
        static unsigned long long attr_mask3 = 0;
        if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(prefill_attn_tc3_kernel), PF2_SMEM, &attr_mask3); e != cudaSuccess) return e;
        const int q_tiles = (p.max_len + PF_TILE - 1) / PF_TILE;
        dim3 grid(p.q_heads, (q_tiles + 1) / 2, p.n_seqs);
        prefill_attn_tc3_kernel<<<grid, PF_THREADS, PF2_SMEM, stream>>>(tq, tkv, p);
        return cudaGetLastError();
    }
    if (p.two_tiles) {
        const int q_tiles = (p.max_len + PF_TILE - 1) / PF_TILE;
        const dim3 grid(p.q_heads, (q_tiles + 1) / 2, p.n_seqs);
        switch (p.two_tiles) {                           // 1 is the measured kernel; 3-6 have not run on a GPU yet
            case 1: return pf_launch_tc2<0, false>(grid, tq, tkv, p, stream);
            case 3: return pf_launch_tc2<1, false>(grid, tq, tkv, p, stream);
            case 4: return pf_launch_tc2<0, true>(grid, tq, tkv, p, stream);
            case 5: return pf_launch_tc2<1, true>(grid, tq, tkv, p, stream);
            case 6: return pf_launch_tc2<2, true>(grid, tq, tkv, p, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(prefill_attn_tc_kernel), PF_SMEM, &attr_mask); e != cudaSuccess) return e;
    dim3 grid(p.q_heads, (p.max_len + PF_TILE - 1) / PF_TILE, p.n_seqs);
    prefill_attn_tc_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(tq, tkv, p);
    return cudaGetLastError();
}

}  // namespace sky
