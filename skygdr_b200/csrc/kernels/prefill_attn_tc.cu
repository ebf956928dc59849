// Causal prefill attention on the 5th-generation tensor cores, reading K and V straight from the paged pool.
//
// One CTA per (pair of query tiles of 128 tokens, query head, prompt). Query rows are the MMA's M, so TMEM lane t holds
// query row t and the softmax of a row lives in one thread: no shuffles, no exchange through shared memory. Tiles
// A = 2c and B = 2c + 1 of a prompt (256 consecutive queries) share every K/V tile that the CTA loads, and their softmax
// warpgroups work in alternation with the tensor core: while warpgroup A turns its scores of key tile j into P, the
// tensor core runs P.V of tile B and the next scores of B, and the other way round.
//
//   warp 8   : TMA producer. Q_A and Q_B once (two boxes of [128 tokens] x [64 dims] each); then per key tile of 128 tokens
//              K and V, each as 8 pages x 2 dim halves of [16 tokens] x [64 dims], 128-byte swizzle, into a ring of
//              five 32 KB units (K0, V0, K1, ...). The pool is addressed through one 3-D tensor map
//              {128 dims, rows between tokens, token rows}, which covers head-major and token-major pages alike.
//   warp 9   : MMA issuer and TMEM owner (512 columns: scores of A and B, 128 each, and the two output accumulators).
//                S[128 q x 128 keys]  = Q[128 x 128] . K_tile^T          (A, B K-major, both from shared memory)
//                O[128 q x 128 dims] += P[128 x 128] . V_tile             (A = P from TMEM, B = V as stored, MN-major)
//   warps 0-7: softmax, one warpgroup per query tile, one thread per query row: all 128 scores of the row in registers,
//              masked on the diagonal tiles, exponentiated, and written back as packed bf16 over the first 64 columns of
//              the row's own score buffer in TMEM (lane = query row, two keys per column), from where the P.V MMA takes
//              its A operand: P never passes through shared memory. The running maximum is raised lazily (only when a
//              tile exceeds it by 8 in log2 units) and then the accumulator row is rescaled in TMEM. The epilogue divides
//              by the row sum and writes bf16 rows.
// Causality skips key tiles above the diagonal; CTAs are launched heaviest first. The four query heads of a KV head run
// next to one another (head is the fastest grid dimension) and find each other's K/V tiles in L2.
// Chunked prefill: with pos0[seq] > 0 the queries of a launch are the next piece of a longer prompt; the K/V of the
// earlier pieces are in the pool already and every query attends to all of them.
//
// Measured on B200, 32 / 8 heads, one prompt of 16384 tokens: 1107 TFLOP/s causal. Forms that were tried and measured slower
// on the same case and removed: P through shared memory (1032), one query tile per CTA with two softmax warpgroups (591),
// key steps of 64 with double-buffered scores (665), one or two of every four exponentials as a cubic on the FMA pipe
// (1001-1006 and 967).
#include <cuda.h>

#include "common.cuh"
#include "prefill_attn.h"

namespace sky {
namespace {

constexpr int PF_THREADS = 320;
constexpr int PF_TILE = 128;
constexpr int PF_UNITS = 5;                        // ring units of one K or V tile each
constexpr int PF_HALF = PF_TILE * 64 * 2;          // [128 rows][64 cols] bf16, swizzled: 16 KB
constexpr int PF_TILE_BYTES = 2 * PF_HALF;         // 32 KB: a Q, K or V tile
constexpr int PF_TILES_BYTES = PF_TILE_BYTES * (2 + PF_UNITS);           // Q_A, Q_B and the ring: 224 KB
constexpr int PF_SMEM = PF_TILES_BYTES + 256;                            // + barriers; no static shared memory
constexpr float PF_RESCALE = 8.0f;

__global__ void __launch_bounds__(PF_THREADS, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                                                         const __grid_constant__ CUtensorMap tmap_kv, const PrefillAttnParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* q_sm = smem;                                        // Q_A, Q_B
    unsigned char* ring = smem + 2 * PF_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PF_TILES_BYTES);
    uint64_t* full_bar = bars;                        // [PF_UNITS]
    uint64_t* empty_bar = bars + PF_UNITS;           // [PF_UNITS]
    uint64_t* s_ready = bars + 2 * PF_UNITS;         // [2]: per query tile, one completion per key tile
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
    const int n_q = p.seq_start[seq + 1] - tok_base;                     // queries of this sequence in this launch
    const int pos0 = p.pos0 ? p.pos0[seq] : 0;                           // tokens of the sequence before them (K/V already in the pool)
    const int n = pos0 + n_q;                                            // keys the last query sees
    const int q_tiles = (n_q + PF_TILE - 1) / PF_TILE;
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;               // heaviest pairs first
    if (2 * pair >= q_tiles) return;
    const int qt_x[2] = {2 * pair, 2 * pair + 1};
    // key tiles each query tile needs: up to the tile that holds its last query's position (0: tile B is past the prompt);
    // from key tile mask_x on, some key of the tile lies after some query of the query tile, so the causal mask applies
    int nkt_x[2], mask_x[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int g0 = pos0 + qt_x[x] * PF_TILE;
        nkt_x[x] = qt_x[x] < q_tiles ? (min(g0 + PF_TILE - 1, n - 1) >> 7) + 1 : 0;
        mask_x[x] = g0 >> 7;
    }
    const int n_kt = max(nkt_x[0], nkt_x[1]);
    const int kvh = head / (p.q_heads / p.kv_heads);
    const int* table = p.block_table + (long long)seq * p.max_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_UNITS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
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
            const int s = u % PF_UNITS;
            if (u >= PF_UNITS && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (uint32_t)((u / PF_UNITS) - 1) & 1))) {
                if (lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 51);
                break;
            }
            unsigned char* st = ring + s * PF_TILE_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[s], PF_TILE_BYTES);
            __syncwarp();
            if (p.page_box) {
                // One request per page: the five-dimensional map (64 dims, 8 tokens, 2 halves of head_dim, 2 token groups, 256-byte
                // row of the pool) lays a page down as [token group][half][8 tokens][128 bytes]. The SM's TMA unit takes a request
                // about every 37 ns whatever its size; 32 boxes per key tile took as long to issue as the tile takes to compute.
                if (lane < 8) {
                    const int e = (u >> 1) * 8 + lane;
                    const int blk = e < p.max_blocks ? __ldg(table + e) : 0;
                    const long long row0 = ((long long)blk * p.block_stride >> 7) + ((u & 1) ? (p.kv_stride >> 7) : 0) + head_row;
                    tma_load_5d(st + lane * 4096, &tmap_kv, 0, 0, 0, 0, (int)row0, &full_bar[s]);
                }
            } else if (lane < 16) {
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
                const int u = 2 * j, s = u % PF_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 53); return false; }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(ring + s * PF_TILE_BYTES), q_addr = smem_u32(q_sm + x * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t a = umma_desc_k_sw128(q_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    const uint64_t b = p.page_box ? umma_desc_k_sw128_sbo(k_addr + (k >> 2) * 1024 + (k & 3) * 32, 2048)
                                                  : umma_desc_k_sw128(k_addr + (k >> 2) * PF_HALF + (k & 3) * 32);
                    tc_mma_f16(tmem_base + x * 128, a, b, idesc_s, k ? 1u : 0u);
                }
                const bool last_user = x == 1 || j >= nkt_x[1];
                if (last_user) tc_commit(&empty_bar[s]);
                tc_commit(&s_ready[x]);
                return true;
            };
            auto issue_pv = [&](int x, int j) -> bool {
                if (!mbar_wait(&p_ready[x], (uint32_t)j & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 54); return false; }
                const int u = 2 * j + 1, s = u % PF_UNITS;
                if (!mbar_wait(&full_bar[s], (uint32_t)(u / PF_UNITS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 55); return false; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(ring + s * PF_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 8; ++k) {                           // 16 keys of P = 8 columns of packed bf16 in the score buffer
                    const uint64_t b = p.page_box ? umma_desc_mn_sw128(v_addr + k * 4096, 1024, 2048) : umma_desc_mn_sw128(v_addr + k * 2048, PF_HALF, 1024);
                    tc_mma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + k * 8, b, idesc_o, (j | k) ? 1u : 0u);
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
        const int qt = qt_x[x], my_kt = nkt_x[x], mask_from = mask_x[x];
        const float qs = p.scale * 1.4426950408889634f;
        const int q_local = qt * PF_TILE + r;                              // row of q / out inside this sequence's piece
        const bool row_valid = my_kt > 0 && q_local < n_q;
        const int qpos = q_local < n_q ? pos0 + q_local : n - 1;           // position in the sequence (rows past the piece: harmless values)
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
            if (j >= mask_from) {                                          // tiles on the diagonal: causal mask and the prompt's end
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
            {
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
                            e[i] = exp2f(a);
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
            __nv_bfloat16* orow = p.out + ((long long)(tok_base + q_local) * p.q_heads + head) * 128;
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

// Pages of 16 tokens x 128 dims as one box: dimensions (64 dims, 8 tokens at the token pitch, 2 halves of head_dim, 2 groups of 8
// tokens, 256-byte row of the pool from which the page starts). The last dimension steps by one pool row, so any page start
// (block, K or V, head) is a coordinate; the dimensions overlap in memory, which the address arithmetic does not mind.
bool pf_make_tmap_pages(CUtensorMap* m, const void* base, long long tok_pitch_bytes, long long pool_rows) {
    static PfEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return false;
        fn = reinterpret_cast<PfEncodeFn>(ptr);
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || pool_rows < 16 || pool_rows > 0x7fffffffLL) return false;
    const cuuint64_t dims[5] = {64, 8, 2, 2, (cuuint64_t)pool_rows};
    const cuuint64_t strides[4] = {(cuuint64_t)tok_pitch_bytes, 128, (cuuint64_t)(8 * tok_pitch_bytes), 256};
    const cuuint32_t box[5] = {64, 8, 2, 2, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
    PrefillAttnParams q = p;
    // SKYGDR_ATTN_TWO_BOXES=1 keeps two boxes per page (measured against each other: 1088 against 1060 TFLOP/s at 16k tokens)
    static const bool two_boxes = [] { const char* v = getenv("SKYGDR_ATTN_TWO_BOXES"); return v && v[0] == '1'; }();
    // the last page may not reach past the allocation: its last token row starts 15 token pitches after its first
    q.page_box = (!two_boxes && pf_make_tmap_pages(&tkv, p.kv, ts_rows * 256, pool_rows - 15 * ts_rows)) ? 1 : 0;
    if (!q.page_box && !pf_make_tmap(&tkv, p.kv, ts_rows, pool_rows / ts_rows, 16)) return cudaErrorInvalidValue;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(prefill_attn_tc_kernel), PF_SMEM, &attr_mask); e != cudaSuccess) return e;
    const int q_tiles = (p.max_len + PF_TILE - 1) / PF_TILE;
    const dim3 grid(p.q_heads, (q_tiles + 1) / 2, p.n_seqs);
    prefill_attn_tc_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(tq, tkv, q);
    return cudaGetLastError();
}

}  // namespace sky
