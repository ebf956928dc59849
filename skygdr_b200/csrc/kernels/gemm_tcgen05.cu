// bf16 GEMM on the 5th-generation tensor cores: y[M][N] = x[M][K] * w[N][K]^T.
//
// Built for decode, where M (tokens) is small and the weight stream is the
// bound: the 128-row MMA dimension is given to the WEIGHT rows and the tokens
// are the MMA's N dimension (16..256), so a 16-token batch wastes nothing.
//   warp 0   : TMA producer   (cp.async.bulk.tensor, 128-byte swizzle, no cluster broadcast)
//   warp 1   : MMA issuer     (tcgen05.mma, accumulators in TMEM) and TMEM owner
//   warps 2-5: epilogue       (tcgen05.ld -> registers -> bf16 / split-K partials)
// Options: split-K with an in-kernel last-CTA reduction through an fp32
// scratch buffer, and a gated mode that keeps two accumulators (gate and up
// rows of the same tile) and stores silu(gate)*up.
//
// The reference has no GEMM at all; its decode model stands in for the MLP
// with a streaming pass over two small arrays
// (llm_problem_analysis/decode_transformer_kvcache_stress.cu:323-356).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace sky {

bool pdl_enabled() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("SKYGDR_PDL"); on = (e && e[0] == '0') ? 0 : 1; }
    return on == 1;
}

// Writes a chunk of 16 token rows x 128 columns. Thread r (0..127 of the epilogue warps) holds column n0+r of the 16
// rows. The values are staged through shared memory so that each row leaves as 16-byte pieces, 256 contiguous bytes
// per row, instead of one 2-byte store per element: that matters most when the destination is a peer over NVLink.
// Only the first `count` rows are stored (the cluster form hands a CTA fewer than 16 token columns at a time).
__device__ __forceinline__ void store_chunk16(const GemmParams& p, __nv_bfloat16* stage, int t_base, int n0, int r, float* vals, int count = 16,
                                              int bar = 3) {
#pragma unroll
    for (int j = 0; j < 16; ++j) stage[j * 128 + r] = __float2bfloat16(vals[j]);
    asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = r + 128 * k, j = idx >> 4, ch = idx & 15;
        const int t = t_base + j, n = n0 + ch * 8;
        if (j < count && t < p.M && n < p.N) {
            __nv_bfloat16* dst;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + j * 128 + ch * 8);
            if (p.rs.world > 0 && p.rs.all) {                       // one-shot all-reduce: the same row to every rank
                const long long off = ((long long)p.rs.src_rank * p.rs.rows_per_rank + t) * p.N + n;
                if (n + 8 <= p.N) {
                    for (int d = 0; d < p.rs.world; ++d) st_v4(p.rs.dst[d] + off, v);
                } else {
                    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
                    for (int d = 0; d < p.rs.world; ++d)
                        for (int q = 0; q < 8 && n + q < p.N; ++q) p.rs.dst[d][off + q] = e[q];
                }
                continue;
            }
            if (p.rs.world == 0) dst = p.y + (long long)t * p.ldy + n;
            else {
                const int d = t / p.rs.rows_per_rank, lr = t - d * p.rs.rows_per_rank;
                dst = p.rs.dst[d] + ((long long)(p.rs.src_rank * p.rs.rows_per_rank + lr)) * p.N + n;
            }
            if (n + 8 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) st_v4(dst, v);
            else {
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
                for (int q = 0; q < 8 && n + q < p.N; ++q) dst[q] = e[q];
            }
        }
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
}

// Thread-block cluster pieces of the split-K form below: the CTAs of one output tile (one per K range) form a cluster and
// reduce their partial accumulators through each other's shared memory instead of through global memory.
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta_rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_smem_addr), "r"(cta_rank));
    return a;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

constexpr int GEMM_THREADS = 192;
constexpr int BM = 128;   // weight rows per tile (MMA M)
constexpr int BK = 64;    // K per stage: 64 bf16 = 128 bytes = one swizzle row

// DEEP: one CTA per SM with the deepest pipeline that fits (up to 8 stages). The GEMMs that wait for an all-gather use it: their
// producer streams weight tiles while the CTA waits for its arrivals, so every extra stage is weight traffic hidden behind
// the wait (measured: TP 2 decode 8.82 ms per step with 8 stages, 9.13-9.16 ms with the 5 stages of the shared layout).
template <int NTOK, bool GATED, bool DEEP = false>
struct GemmSmem {
    static constexpr int W_BYTES = BM * BK * 2;
    static constexpr int X_BYTES = NTOK * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES * (GATED ? 2 : 1) + X_BYTES;
    // Two CTAs per SM where three stages fit in half an SM's shared memory: while one CTA is in its prologue or
    // epilogue the other keeps the SM's share of the weight stream going.
    static constexpr bool TWO_PER_SM = !DEEP && 3 * STAGE_BYTES <= 104 * 1024;
    static constexpr int BUDGET = TWO_PER_SM ? 104 * 1024 : 200 * 1024;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024;  // + alignment slack
    static constexpr int ACC_COLS = NTOK * (GATED ? 2 : 1);
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;
};

// CSPLIT: split-K inside a thread-block cluster. The `splits` CTAs of an output tile are launched as one cluster (cluster
// dimension z); each leaves its fp32 partial accumulator in its own shared memory (over the pipeline stages, which are idle by
// then), the cluster synchronises, and CTA s sums and stores the token columns [s * NTOK / splits, (s + 1) * NTOK / splits) of the
// tile, reading all partials through distributed shared memory. No workspace in global memory, no counters, no last CTA that
// re-reads every partial on its own: that is what made splits of 128-token tiles too expensive to use.
template <int NTOK, bool GATED, bool DEEP, bool CSPLIT>
__global__ void __launch_bounds__(GEMM_THREADS, (GemmSmem<NTOK, GATED, DEEP>::TWO_PER_SM ? 2 : 1))
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using S = GemmSmem<NTOK, GATED, DEEP>;
    static_assert(!CSPLIT || S::ACC_COLS * BM * 4 <= S::STAGES * S::STAGE_BYTES, "the partial accumulator must fit over the pipeline stages");
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full_bar[8], empty_bar[8], acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_last;
    __shared__ __align__(16) __nv_bfloat16 stage[16 * 128];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    pdl_trigger();     // the next kernel may start its own prologue while this one streams
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
    const int n0 = tile_n * BM, t0 = tile_m * NTOK;
    const int kb_total = p.K / BK;
    const int kb_per = (kb_total + p.splits - 1) / p.splits;
    const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
    const int nkb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(&tmem_slot, S::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // With an all-gather in front, the producer may wait for peers up to its own deadline; the consumers of its
    // barriers must outlast that, or a late peer would look like a broken pipeline.
    const unsigned long long bar_timeout = p.ag.n_src > 0 ? p.ag.timeout_ns + 1000000000ull : 200000000ull;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmap_w);
            tma_prefetch_desc(&tmap_x);
            // Weights do not depend on any peer: start streaming them, then wait for the gathered
            // activations, then add the x tiles to the stages already in flight.
            const int pre = min(nkb, S::STAGES);
            for (int i = 0; i < pre; ++i) {
                unsigned char* st = smem + i * S::STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], S::STAGE_BYTES);
                const int kx = (kb0 + i) * BK;
                tma_load_2d(st, &tmap_w, kx, n0, &full_bar[i]);
                if (GATED) tma_load_2d(st + S::W_BYTES, &tmap_w, kx, p.N + n0, &full_bar[i]);
            }
            // Weights are constants, so the loads above ran ahead of the previous kernel; x is that kernel's output.
            pdl_wait();
            if (p.ag.n_src > 0 && *(volatile unsigned int*)&p.status->status == SKY_STATUS_OK) {
                const unsigned seq = *p.ag.seq.step * p.ag.seq.uses_per_step + p.ag.seq.use_index + 1;
                const unsigned want = seq * p.ag.seq.arrivals_per_use;
                for (int r = 0; r < p.ag.n_src; ++r)
                    if (!wait_flag_ge(p.ag.counters + r, want, p.ag.timeout_ns)) {
                        set_status(p.status, SKY_STATUS_TIMEOUT_FLAG, (unsigned)r);
                        break;
                    }
                // peers wrote x with ordinary stores; the loads below go through the async proxy
                asm volatile("fence.proxy.async;" ::: "memory");
            }
            for (int i = 0; i < pre; ++i)
                tma_load_2d(smem + i * S::STAGE_BYTES + S::W_BYTES * (GATED ? 2 : 1), &tmap_x, (kb0 + i) * BK, t0, &full_bar[i]);
            for (int i = pre; i < nkb; ++i) {
                const int s = i % S::STAGES;
                if (!mbar_wait(&empty_bar[s], ((i / S::STAGES) - 1) & 1)) {
                    set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 1);
                    break;
                }
                unsigned char* st = smem + s * S::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
                const int kx = (kb0 + i) * BK;
                tma_load_2d(st, &tmap_w, kx, n0, &full_bar[s]);
                if (GATED) tma_load_2d(st + S::W_BYTES, &tmap_w, kx, p.N + n0, &full_bar[s]);
                tma_load_2d(st + S::W_BYTES * (GATED ? 2 : 1), &tmap_x, kx, t0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, NTOK);
            bool ok = true;
            // The first stage cannot fill before the producer's own pdl_wait() has returned. Waiting here as well keeps the bounded
            // waits below from counting time that the previous kernel spent waiting for a peer (they would give up first).
            pdl_wait();
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % S::STAGES;
                if (!mbar_wait(&full_bar[s], (i / S::STAGES) & 1, bar_timeout)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 2); ok = false; break; }
                tc_fence_after();
                const uint32_t st = smem_u32(smem + s * S::STAGE_BYTES);
                const uint64_t a0 = umma_desc_k_sw128(st);
                const uint64_t a1 = umma_desc_k_sw128(st + S::W_BYTES);
                const uint64_t b = umma_desc_k_sw128(st + S::W_BYTES * (GATED ? 2 : 1));
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t accum = (i | k) ? 1u : 0u;
                    tc_mma_f16(tmem_base, a0 + 2 * k, b + 2 * k, idesc, accum);
                    if (GATED) tc_mma_f16(tmem_base + NTOK, a1 + 2 * k, b + 2 * k, idesc, accum);
                }
                tc_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
            }
            tc_commit(&acc_bar);           // accumulators complete
        }
    } else {
        // ---- epilogue warps: TMEM lanes 32*(warp%4) .. +31 ----
        const int slice = warp & 3;
        const int r = slice * 32 + lane;           // weight row inside the tile
        bool ok = true;
        pdl_wait();     // nothing is written before the previous kernel has finished reading its inputs
        if (nkb > 0) ok = mbar_wait(&acc_bar, 0, bar_timeout);
        if (!ok && lane == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 3);
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(slice * 32) << 16);
        const bool direct = p.splits == 1;
        float* ws = nullptr;
        if constexpr (CSPLIT) {
            ws = reinterpret_cast<float*>(smem);                   // [ACC_COLS][128] floats of this CTA, read by the cluster below
        } else if (!direct) {
            const long long tile_id = (long long)tile_m * gridDim.x + tile_n;
            ws = p.workspace + ((tile_id * p.splits + split) * S::ACC_COLS) * BM;
        }
#pragma unroll 1
        for (int c = 0; c < NTOK; c += 16) {
            uint32_t v[16], u[16];
            if (ok && nkb > 0) {
                tmem_ld_x16(taddr + c, v);
                if (GATED) tmem_ld_x16(taddr + NTOK + c, u);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) { v[i] = 0; u[i] = 0; }
            }
            if (direct && !CSPLIT) {
                float vals[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float val = __uint_as_float(v[i]);
                    if (GATED) { const float up = __uint_as_float(u[i]); val = val / (1.0f + __expf(-val)) * up; }
                    vals[i] = val;
                }
                store_chunk16(p, stage, t0 + c, n0, r, vals);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    ws[(c + i) * BM + r] = __uint_as_float(v[i]);
                    if (GATED) ws[(NTOK + c + i) * BM + r] = __uint_as_float(u[i]);
                }
            }
        }
        if (!direct && !CSPLIT) {
            // last-arriving split of this tile sums all partials
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
                unsigned* ctr = p.counters + tile_m * gridDim.x + tile_n;
                const unsigned prev = atomicAdd(ctr, 1u);
                s_last = prev == (unsigned)p.splits - 1;
                if (s_last) *ctr = 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (s_last) {
                __threadfence();
                const long long tile_id = (long long)tile_m * gridDim.x + tile_n;
                const float* base = p.workspace + (tile_id * p.splits) * S::ACC_COLS * BM;
                // 16 token columns at a time: all their partial loads are in flight together
#pragma unroll 1
                for (int c0 = 0; c0 < NTOK; c0 += 16) {
                    float g[16], up[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) { g[j] = 0.f; up[j] = 0.f; }
                    if (t0 + c0 < p.M) {
                        for (int s2 = 0; s2 < p.splits; ++s2) {
                            float a[16], b[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                a[j] = __ldcg(base + ((long long)s2 * S::ACC_COLS + c0 + j) * BM + r);
                                if (GATED) b[j] = __ldcg(base + ((long long)s2 * S::ACC_COLS + NTOK + c0 + j) * BM + r);
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) { g[j] += a[j]; if (GATED) up[j] += b[j]; }
                        }
                        if (GATED) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * up[j];
                        }
                    }
                    store_chunk16(p, stage, t0 + c0, n0, r, g);     // rows past M are skipped inside
                }
            }
        }
    }
    if constexpr (CSPLIT) {
        tc_fence_before();
        cluster_sync_all();                                        // every CTA's partial is in its shared memory
        const uint32_t crank = cluster_ctarank();
        if (warp >= 2) {
            const int r = (warp & 3) * 32 + lane;
            const int c_lo = (int)(crank * NTOK / p.splits), c_hi = (int)((crank + 1) * NTOK / p.splits);
            const uint32_t part = smem_u32(smem);
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
                const int cnt = min(16, c_hi - c0);
                float g[16], up[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) { g[j] = 0.f; up[j] = 0.f; }
                if (t0 + c0 < p.M) {
                    for (int s2 = 0; s2 < p.splits; ++s2) {
                        const uint32_t base = dsmem_addr(part, (uint32_t)s2) + (uint32_t)(c0 * BM + r) * 4u;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (j < cnt) {
                                g[j] += ld_dsmem_f32(base + (uint32_t)(j * BM) * 4u);
                                if (GATED) up[j] += ld_dsmem_f32(base + (uint32_t)((NTOK + j) * BM) * 4u);
                            }
                        }
                    }
                    if (GATED) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * up[j];
                    }
                }
                store_chunk16(p, stage, t0 + c0, n0, r, g, cnt);
            }
        }
        // nobody leaves while a peer may still read its partial; and every CTA's stores come before rank 0's fence below
        cluster_sync_all();
        if (p.rs.world > 0 && crank == 0 && threadIdx.x == 64) {   // one arrival per destination and output tile, as without splits
            __threadfence_system();
            for (int j = 0; j < p.rs.world; ++j) red_relaxed_sys_add_u32(p.rs.counters[j], 1u);
        }
    } else if (p.rs.world > 0 && warp >= 2) {
        // one arrival per destination from the CTA that wrote this tile's rows (with split-K: the last split)
        const bool wrote = p.splits == 1 || s_last;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (wrote && threadIdx.x == 64) {
            __threadfence_system();
            for (int j = 0; j < p.rs.world; ++j) red_relaxed_sys_add_u32(p.rs.counters[j], 1u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Persistent form for many-token (prefill) shapes: one CTA per SM walks the output tiles, and the accumulator is double
// buffered in TMEM, so the epilogue of tile i (TMEM -> registers -> shared memory -> global) runs while the tensor core
// already works on tile i + 1. The shared-memory ring runs across tile boundaries, so the loads of the next tile are in
// flight during the last MMAs of the current one. Same roles and the same operand layout as the kernel above (weight rows
// on the MMA's M, tokens on N); no split-K, no tensor-parallel hooks: this is the plain projection of a prefill step.
// Tiles are numbered token tile fastest, so the CTAs that run side by side share a few weight panels and the x tiles
// stay in L2. Measured on B200 against the one-tile-per-CTA kernel above: 1118 against 790 TFLOP/s at 2048 x 4096 x 4096,
// 1244 against 889 at 8192 x 12288 x 4096 gated. The tensor pipe is busy 69-75 % of the active cycles: the ring holds three to
// five stages in flight, about what a load from L2 takes under this traffic. Asking for every k-block into L2 a ring's depth
// ahead of its load (cp.async.bulk.prefetch.tensor) was measured and made it slower (849 against 1082 TFLOP/s at
// 2048 x 4096 x 4096, 1013 against 1335 at 8192 x 4096 x 4096), so the producer issues loads only.
template <int NTOK, bool GATED>
struct GemmPersistSmem {
    static constexpr int W_BYTES = BM * BK * 2;
    static constexpr int X_BYTES = NTOK * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES * (GATED ? 2 : 1) + X_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024;
    static constexpr int ACC_COLS = NTOK * (GATED ? 2 : 1);     // one accumulator
    static constexpr int TMEM_COLS = 2 * ACC_COLS;              // two of them
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32, "two accumulators must fit TMEM");
};

template <int NTOK, bool GATED>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using S = GemmPersistSmem<NTOK, GATED>;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) __nv_bfloat16 stage[16 * 128];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + NTOK - 1) / NTOK, tiles_n = (p.N + BM - 1) / BM;
    const int n_tiles = tiles_m * tiles_n;
    const int nkb = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 1); }
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(&tmem_slot, S::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmap_w);
            tma_prefetch_desc(&tmap_x);
            pdl_wait();                                    // x is the previous kernel's output
            long long it = 0;                              // k-blocks issued so far, over all tiles of this CTA
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int n0 = (tile / tiles_m) * BM, t0 = (tile % tiles_m) * NTOK;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    if (it >= S::STAGES && !mbar_wait(&empty_bar[s], (uint32_t)((it / S::STAGES) - 1) & 1)) {
                        set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 61);
                        ok = false;
                        break;
                    }
                    unsigned char* st = smem + s * S::STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
                    tma_load_2d(st, &tmap_w, kb * BK, n0, &full_bar[s]);
                    if (GATED) tma_load_2d(st + S::W_BYTES, &tmap_w, kb * BK, p.N + n0, &full_bar[s]);
                    tma_load_2d(st + S::W_BYTES * (GATED ? 2 : 1), &tmap_x, kb * BK, t0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, NTOK);
            long long it = 0;
            int j = 0;                                     // tiles of this CTA so far
            bool ok = true;
            pdl_wait();                                    // as the producer: bounded waits start when the previous kernel is done
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
                const int buf = j & 1;
                // the epilogue must have drained this accumulator (used two tiles ago) before it is overwritten
                if (j >= 2 && !mbar_wait(&acc_empty[buf], (uint32_t)((j >> 1) - 1) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 62); break; }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * S::ACC_COLS);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    if (!mbar_wait(&full_bar[s], (uint32_t)(it / S::STAGES) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 63); ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + s * S::STAGE_BYTES);
                    const uint64_t a0 = umma_desc_k_sw128(st);
                    const uint64_t a1 = umma_desc_k_sw128(st + S::W_BYTES);
                    const uint64_t b = umma_desc_k_sw128(st + S::W_BYTES * (GATED ? 2 : 1));
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t accum = (kb | k) ? 1u : 0u;
                        tc_mma_f16(acc, a0 + 2 * k, b + 2 * k, idesc, accum);
                        if (GATED) tc_mma_f16(acc + NTOK, a1 + 2 * k, b + 2 * k, idesc, accum);
                    }
                    tc_commit(&empty_bar[s]);
                }
                if (ok) tc_commit(&acc_full[buf]);         // this tile's accumulator is complete
            }
        }
    } else {
        // ---- epilogue warps: TMEM lanes 32*(warp%4) .. +31 ----
        const int slice = warp & 3;
        const int r = slice * 32 + lane;
        pdl_wait();
        int j = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
            const int buf = j & 1;
            const int n0 = (tile / tiles_m) * BM, t0 = (tile % tiles_m) * NTOK;
            // All 128 epilogue threads take the same way out: they meet at named barriers below, so a wait that gave up in
            // some of them only (the deadline is per thread) must end the loop for all of them.
            const uint32_t mine = mbar_wait(&acc_full[buf], (uint32_t)(j >> 1) & 1) ? 1u : 0u;
            uint32_t n_ok;
            asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.popc.u32 %0, 3, 128, q;\n\t}" : "=r"(n_ok) : "r"(mine) : "memory");
            if (n_ok != 128u) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 64); break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t)(buf * S::ACC_COLS) + ((uint32_t)(slice * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < NTOK; c += 16) {
                if (t0 + c >= p.M) break;                  // uniform over the 128 threads: rows past M are never stored
                uint32_t v[16], u[16];
                tmem_ld_x16(taddr + c, v);
                if (GATED) tmem_ld_x16(taddr + NTOK + c, u);
                tc_wait_ld();
                float vals[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float val = __uint_as_float(v[i]);
                    if (GATED) { const float up = __uint_as_float(u[i]); val = val / (1.0f + __expf(-val)) * up; }
                    vals[i] = val;
                }
                store_chunk16(p, stage, t0 + c, n0, r, vals);   // ends with a barrier of the 128 epilogue threads
            }
            // every thread's TMEM loads are complete (tc_wait_ld above); hand the accumulator back to the MMA warp
            tc_fence_before();
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (r == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Persistent form with a tile of 256 weight rows x 256 tokens per CTA: two 128-row MMAs per k-block share one token operand, so
// a stage of 64 KB feeds 1024 tensor-core cycles (64 bytes per cycle and SM from L2 instead of 96) and the three stages that
// fit cover the load latency that bounds the kernel above. The two accumulators fill all 512 TMEM columns, so a tile's
// epilogue is not overlapped with the next tile's MMAs (its loads are: the producer runs on); two groups of four epilogue
// warps keep it short. Ungated (256 weight rows per tile, N a multiple of 256) or gated (a gate block and an up block per tile,
// 128 output rows). Measured on B200 against the kernel above (TFLOP/s):
// 1220 / 1137 at 2048 x 4096 x 4096, 1420 / 1333 at 8192 x 4096 x 12288, 1362 / 1391 at 8192 x 4096 x 4096 (half as many tiles
// leave the last wave emptier there); gated 1463 / 1236 at 8192 x 12288 x 4096, 1505 / 1335 at 4096 tokens, 1418 / 1270 at 2048.
// ops.gemm.wide_tiles_pay chooses between the two per shape.
struct GemmWideSmem {
    static constexpr int W_BYTES = BM * BK * 2;                 // one 128-row weight block
    static constexpr int X_BYTES = 256 * BK * 2;
    static constexpr int STAGE_BYTES = 2 * W_BYTES + X_BYTES;   // 64 KB
    static constexpr int STAGES = 3;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024;
    static constexpr int THREADS = 64 + 256;                    // producer warp, MMA warp, two epilogue groups of four warps
};

template <bool GATED>
__global__ void __launch_bounds__(GemmWideSmem::THREADS, 1)
gemm_persistent_wide_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using S = GemmWideSmem;
    constexpr int NTOK = 256;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full_bar[S::STAGES], empty_bar[S::STAGES], acc_full, acc_empty;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) __nv_bfloat16 stage[2][16 * 128];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // output rows per tile: 256 (two weight blocks), or 128 when gated (a gate block and an up block give one block of outputs)
    constexpr int ROWS = GATED ? BM : 2 * BM;
    const int tiles_m = (p.M + NTOK - 1) / NTOK, tiles_n = (p.N + ROWS - 1) / ROWS;
    const int n_tiles = tiles_m * tiles_n;
    const int nkb = p.K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, 2);                          // one arrival per epilogue group
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmap_w);
            tma_prefetch_desc(&tmap_x);
            pdl_wait();                                    // x is the previous kernel's output
            long long it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int n0 = (tile / tiles_m) * ROWS, t0 = (tile % tiles_m) * NTOK;
                const int n1 = GATED ? p.N + n0 : n0 + BM;             // second weight block: the up rows, or the next 128 rows
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    if (it >= S::STAGES && !mbar_wait(&empty_bar[s], (uint32_t)((it / S::STAGES) - 1) & 1)) {
                        set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 71);
                        ok = false;
                        break;
                    }
                    unsigned char* st = smem + s * S::STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
                    tma_load_2d(st, &tmap_w, kb * BK, n0, &full_bar[s]);
                    tma_load_2d(st + S::W_BYTES, &tmap_w, kb * BK, n1, &full_bar[s]);
                    tma_load_2d(st + 2 * S::W_BYTES, &tmap_x, kb * BK, t0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, NTOK);
            long long it = 0;
            int j = 0;
            bool ok = true;
            pdl_wait();                                    // bounded waits start when the previous kernel is done
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
                // both epilogue groups must have drained the accumulators of the previous tile
                if (j >= 1 && !mbar_wait(&acc_empty, (uint32_t)(j - 1) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 72); break; }
                tc_fence_after();
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    if (!mbar_wait(&full_bar[s], (uint32_t)(it / S::STAGES) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 73); ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + s * S::STAGE_BYTES);
                    const uint64_t a0 = umma_desc_k_sw128(st);
                    const uint64_t a1 = umma_desc_k_sw128(st + S::W_BYTES);
                    const uint64_t b = umma_desc_k_sw128(st + 2 * S::W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t accum = (kb | k) ? 1u : 0u;
                        tc_mma_f16(tmem_base, a0 + 2 * k, b + 2 * k, idesc, accum);
                        tc_mma_f16(tmem_base + NTOK, a1 + 2 * k, b + 2 * k, idesc, accum);
                    }
                    tc_commit(&empty_bar[s]);
                }
                if (ok) tc_commit(&acc_full);
            }
        }
    } else {
        // ---- epilogue: two groups of four warps; warp w reads TMEM lanes 32 (w % 4) .. +31. Ungated: group g drains accumulator g
        // (weight rows n0 + 128 g ..). Gated: both accumulators hold the same 128 output rows (gate and up), and group g takes
        // the token columns 128 g .. 128 g + 127 of both. ----
        const int g = (warp - 2) >> 2;
        const int slice = warp & 3;
        const int r = slice * 32 + lane;
        const int bar = 3 + g;
        pdl_wait();
        int j = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
            const int n0 = (tile / tiles_m) * ROWS + (GATED ? 0 : g * BM), t0 = (tile % tiles_m) * NTOK;
            const uint32_t mine = mbar_wait(&acc_full, (uint32_t)j & 1) ? 1u : 0u;
            uint32_t n_ok;
            asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.popc.u32 %0, %2, 128, q;\n\t}" : "=r"(n_ok) : "r"(mine), "r"(bar) : "memory");
            if (n_ok != 128u) { if (r == 0) set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 74); break; }
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(slice * 32) << 16);
            const int c_lo = GATED ? g * (NTOK / 2) : 0, c_hi = GATED ? c_lo + NTOK / 2 : NTOK;
#pragma unroll 1
            for (int c = c_lo; c < c_hi; c += 16) {
                if (t0 + c >= p.M) break;                  // uniform over the group: rows past M are never stored
                uint32_t v[16], u[16];
                tmem_ld_x16(lane_addr + (uint32_t)((GATED ? 0 : g * NTOK) + c), v);
                if (GATED) tmem_ld_x16(lane_addr + (uint32_t)(NTOK + c), u);
                tc_wait_ld();
                float vals[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float val = __uint_as_float(v[i]);
                    if (GATED) { const float up = __uint_as_float(u[i]); val = val / (1.0f + __expf(-val)) * up; }
                    vals[i] = val;
                }
                store_chunk16(p, stage[g], t0 + c, n0, r, vals, 16, bar);
            }
            tc_fence_before();
            asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
            if (r == 0) mbar_arrive(&acc_empty);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and dispatch.

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D bf16 row-major [rows][cols] with row pitch `ld` elements; box = 64 columns x box_rows rows, 128-byte swizzle.
bool make_tmap_bf16_2d(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NTOK, bool GATED, bool DEEP, bool CSPLIT = false>
static cudaError_t launch_t(const GemmParams& p, const CUtensorMap& tw, const CUtensorMap& tx, cudaStream_t stream) {
    using S = GemmSmem<NTOK, GATED, DEEP>;
    auto kern = gemm_tcgen05_kernel<NTOK, GATED, DEEP, CSPLIT>;
    // SKYGDR_GEMM_ONE_PER_SM=1 pads the request of the small-stage kernels so that only one CTA fits on an SM (a switch for
    // measuring what co-residency is worth; the kernel itself does not change).
    static const bool one_per_sm = [] { const char* v = getenv("SKYGDR_GEMM_ONE_PER_SM"); return v && v[0] == '1'; }();
    const int dyn = (S::TWO_PER_SM && one_per_sm) ? (S::TOTAL > 120 * 1024 ? S::TOTAL : 120 * 1024) : S::TOTAL;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kern), dyn, &attr_mask); e != cudaSuccess) return e;
    dim3 grid((p.N + BM - 1) / BM, (p.M + NTOK - 1) / NTOK, p.splits);
    return launch_pdl_cluster(kern, grid, dim3(GEMM_THREADS), (size_t)dyn, stream, CSPLIT ? p.splits : 0, tw, tx, p);
}

template <int NTOK, bool GATED>
static cudaError_t launch_persistent_t(const GemmParams& p, const CUtensorMap& tw, const CUtensorMap& tx, cudaStream_t stream) {
    using S = GemmPersistSmem<NTOK, GATED>;
    auto kern = gemm_persistent_kernel<NTOK, GATED>;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kern), S::TOTAL, &attr_mask); e != cudaSuccess) return e;
    int dev = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); e != cudaSuccess) return e;
    const long long tiles = (long long)((p.N + BM - 1) / BM) * ((p.M + NTOK - 1) / NTOK);
    const int ctas = (int)std::min<long long>(tiles, sms > 0 ? sms : 1);     // one CTA per SM, each walks tiles cta, cta + ctas, ...
    return launch_pdl(kern, dim3(ctas), dim3(GEMM_THREADS), (size_t)S::TOTAL, stream, tw, tx, p);
}

template <bool GATED>
static cudaError_t launch_persistent_wide(const GemmParams& p, const CUtensorMap& tw, const CUtensorMap& tx, cudaStream_t stream) {
    using S = GemmWideSmem;
    auto kern = gemm_persistent_wide_kernel<GATED>;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kern), S::TOTAL, &attr_mask); e != cudaSuccess) return e;
    int dev = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); e != cudaSuccess) return e;
    const int rows = GATED ? BM : 2 * BM;
    const long long tiles = (long long)((p.N + rows - 1) / rows) * ((p.M + 255) / 256);
    const int ctas = (int)std::min<long long>(tiles, sms > 0 ? sms : 1);
    return launch_pdl(kern, dim3(ctas), dim3(S::THREADS), (size_t)S::TOTAL, stream, tw, tx, p);
}

int gemm_pick_ntok(int M, bool gated) {
    if (M <= 16) return 16;
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    if (M <= 128 || gated) return 128;  // gated keeps two accumulators: 2 x 128 columns
    return 256;
}

size_t gemm_workspace_floats(int M, int N, int splits, bool gated, int ntok) {
    if (splits <= 1) return 0;
    if (ntok <= 0) ntok = gemm_pick_ntok(M, gated);
    const long long tiles = (long long)((N + BM - 1) / BM) * ((M + ntok - 1) / ntok);
    return (size_t)(tiles * splits * ntok * (gated ? 2 : 1) * BM);
}
size_t gemm_counter_count(int M, int N, bool gated, int ntok) {
    if (ntok <= 0) ntok = gemm_pick_ntok(M, gated);
    return (size_t)((N + BM - 1) / BM) * ((M + ntok - 1) / ntok);
}

cudaError_t launch_gemm(const GemmParams& p, cudaStream_t stream) {
    if (p.K % BK || p.M <= 0 || p.N <= 0 || p.splits < 1 || p.splits > p.K / BK) return cudaErrorInvalidValue;
    const bool csplit = p.cluster_split && p.splits > 1;
    if (csplit && (p.splits > 8 || p.ag.n_src > 0)) return cudaErrorInvalidValue;        // a portable cluster holds at most 8 CTAs
    if (p.splits > 1 && !csplit && (!p.workspace || !p.counters)) return cudaErrorInvalidValue;
    // the form with two weight blocks per token operand always takes 256 tokens (its x box and its stage size are built on that)
    const int ntok = p.persistent == 2 ? 256 : (p.ntok > 0 ? p.ntok : gemm_pick_ntok(p.M, p.gated != 0));
    if (ntok != 16 && ntok != 32 && ntok != 64 && ntok != 128 && ntok != 256) return cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    const long long w_rows = p.gated ? 2LL * p.N : p.N;
    if (!make_tmap_bf16_2d(&tw, p.w, w_rows, p.K, p.ldw, BM)) return cudaErrorInvalidValue;
    if (!make_tmap_bf16_2d(&tx, p.x, p.M, p.K, p.ldx, ntok)) return cudaErrorInvalidValue;
    if (p.persistent) {
        // the persistent form is the plain projection at many-token shapes: 256-token tiles (128 when gated or asked for)
        if (p.splits != 1 || p.ag.n_src > 0 || p.rs.world > 0) return cudaErrorInvalidValue;
        if (p.persistent == 2) {                           // two weight blocks per 256-token operand
            if (p.gated) return launch_persistent_wide<true>(p, tw, tx, stream);
            if (p.N % (2 * BM)) return cudaErrorInvalidValue;
            return launch_persistent_wide<false>(p, tw, tx, stream);
        }
        if (ntok == 256 && !p.gated) return launch_persistent_t<256, false>(p, tw, tx, stream);
        if (ntok == 128) return p.gated ? launch_persistent_t<128, true>(p, tw, tx, stream) : launch_persistent_t<128, false>(p, tw, tx, stream);
        return cudaErrorInvalidValue;
    }
    // A GEMM that waits for an all-gather runs one CTA per SM with the deepest pipeline (more weight traffic hidden behind the
    // wait). Everything else, the GEMMs that only push their tiles to peers included, keeps the small pipeline: two CTAs per
    // SM, which also leaves room on the SM for the next kernel's CTAs to start early (measured in a chain of launches inside
    // a CUDA graph, every decode GEMM shape at TP 1 / 2 / 4 / 8 and every tile and split: the deep layout was never faster, and
    // slower by 1 - 2 us per launch for most).
    const bool deep = p.ag.n_src > 0;
#define SKY_GEMM_CLUSTER_CASE(NT) \
    case NT: return p.gated ? launch_t<NT, true, false, true>(p, tw, tx, stream) : launch_t<NT, false, false, true>(p, tw, tx, stream);
    if (csplit) {
        switch (ntok) {
            SKY_GEMM_CLUSTER_CASE(16)
            SKY_GEMM_CLUSTER_CASE(32)
            SKY_GEMM_CLUSTER_CASE(64)
            SKY_GEMM_CLUSTER_CASE(128)
            default: return p.gated ? cudaErrorInvalidValue : launch_t<256, false, false, true>(p, tw, tx, stream);
        }
    }
#undef SKY_GEMM_CLUSTER_CASE
#define SKY_GEMM_CASE(NT)                                                                   \
    case NT: return deep ? (p.gated ? launch_t<NT, true, true>(p, tw, tx, stream) : launch_t<NT, false, true>(p, tw, tx, stream))   \
                         : (p.gated ? launch_t<NT, true, false>(p, tw, tx, stream) : launch_t<NT, false, false>(p, tw, tx, stream));
    switch (ntok) {
        SKY_GEMM_CASE(16)
        SKY_GEMM_CASE(32)
        SKY_GEMM_CASE(64)
        SKY_GEMM_CASE(128)
        default: return p.gated ? cudaErrorInvalidValue : launch_t<256, false, false>(p, tw, tx, stream);
    }
#undef SKY_GEMM_CASE
}

}  // namespace sky
