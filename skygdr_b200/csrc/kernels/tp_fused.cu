// Tensor-parallel glue kernels. The collectives of a tensor-parallel decoder
// layer are not separate library calls here: the GEMM epilogue stores its
// partial rows straight into the owning rank's receive buffer (reduce-scatter),
// this norm kernel sums them, adds the residual, normalises and stores the
// result into every rank's gather buffer (all-gather), and the next GEMM's TMA
// producer waits for those rows while its weight tiles are already streaming.
// Arrival counters with release/acquire at system scope order the traffic; they
// only grow, and every wait has a deadline.
//
// The reference has no tensor parallelism and no collective of any kind (its
// only multi-GPU traffic is cudaMemcpyPeerAsync, llm_problem_analysis/kv_nvlink_transfer.cu:122).
#include "common.cuh"
#include "tp_fused.h"

namespace sky {

__device__ __forceinline__ void unpack8f(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2f(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8f(const float* f) {
    return make_uint4(pack2f(f[0], f[1]), pack2f(f[2], f[3]), pack2f(f[4], f[5]), pack2f(f[6], f[7]));
}
__device__ __forceinline__ unsigned tp_seq(const TpSeq& s) { return *s.step * s.uses_per_step + s.use_index + 1; }

__global__ void __launch_bounds__(256) tp_norm_kernel(const TpNormParams p) {
    __shared__ float red[8];
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int nvec = p.hidden / 8;
    // The residual row (written by the previous launch of this kernel, complete after pdl_wait) and the norm weights do not
    // depend on the arrivals: their loads are in flight while thread 0 waits.
    uint4 res_raw[4], w_raw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nvec) {
            res_raw[k] = *reinterpret_cast<const uint4*>(p.resid + (long long)row * p.hidden + v * 8);
            w_raw[k] = __ldg(reinterpret_cast<const uint4*>(p.w + v * 8));
        }
    }
    if (threadIdx.x == 0) {
        int ok = 1;
        if (p.rs_buf && *(volatile unsigned int*)&p.status->status == SKY_STATUS_OK) {
            const unsigned want = tp_seq(p.rs_seq) * p.rs_seq.arrivals_per_use;
            if (!wait_flag_ge(p.rs_counter, want, p.timeout_ns)) {
                set_status(p.status, SKY_STATUS_TIMEOUT_FLAG, 100u + (unsigned)row);
                ok = 0;
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    float vals[4][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nvec) {
            unpack8f(res_raw[k], vals[k]);
            if (p.rs_buf) {
                // all partials of this piece are requested before the first one is used: one L2 round trip, not `world` of them
                uint4 raw[TP_MAX_RANKS];
#pragma unroll
                for (int s = 0; s < TP_MAX_RANKS; ++s)
                    if (s < p.world) raw[s] = __ldcg(reinterpret_cast<const uint4*>(p.rs_buf + ((long long)(s * p.rows + row)) * p.hidden + v * 8));
#pragma unroll
                for (int s = 0; s < TP_MAX_RANKS; ++s) {
                    if (s < p.world) {
                        float part[8];
                        unpack8f(raw[s], part);
#pragma unroll
                        for (int i = 0; i < 8; ++i) vals[k][i] += part[i];
                    }
                }
                const uint4 packed = pack8f(vals[k]);
                *reinterpret_cast<uint4*>(p.resid + (long long)row * p.hidden + v * 8) = packed;
                unpack8f(packed, vals[k]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += vals[k][i] * vals[k][i];
        }
    }
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = rsqrtf(tot / p.hidden + p.eps);
    const long long grow = (long long)(p.ag_row0 + row) * p.hidden;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nvec) {
            float g[8], o[8];
            unpack8f(w_raw[k], g);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = vals[k][i] * inv * g[i];
            const uint4 packed = pack8f(o);
            for (int j = 0; j < p.ag_n; ++j) st_v4(p.ag_dst[j] + grow + v * 8, packed);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.ag_counter[0] != nullptr) {            // a purely local destination needs no arrival
        __threadfence_system();
        for (int j = 0; j < p.ag_n; ++j) red_relaxed_sys_add_u32(p.ag_counter[j], 1u);
    }
}

cudaError_t launch_tp_norm(const TpNormParams& p, cudaStream_t stream) {
    if (p.hidden % 8 || p.hidden > 8192 || p.rows <= 0 || p.world < 1 || p.world > TP_MAX_RANKS) return cudaErrorInvalidValue;
    if (p.ag_n < 1 || p.ag_n > TP_MAX_RANKS) return cudaErrorInvalidValue;
    return launch_pdl(tp_norm_kernel, dim3(p.rows), dim3(256), 0, stream, p);
}

// Orders floats as unsigned integers: larger float <=> larger key.
__device__ __forceinline__ unsigned float_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(256) tp_argmax_kernel(const TpArgmaxParams p) {
    __shared__ unsigned long long best_s[8];
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const __nv_bfloat16* lg = p.logits + (long long)row * p.row_stride;
    // candidate = (ordered value, inverted global index): the maximum prefers the larger value, then the lower index
    unsigned long long best = 0;
    for (int c = threadIdx.x; c < p.vocab_local; c += 256) {
        const unsigned long long cand = ((unsigned long long)float_key(__bfloat162float(lg[c])) << 32) |
                                        (unsigned long long)(0xffffffffu - (unsigned)(p.vocab_lo + c));
        best = cand > best ? cand : best;
    }
    for (int o = 16; o; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = best_s[w] > best ? best_s[w] : best;
        for (int j = 0; j < p.world; ++j) p.slots[j][(long long)p.rank * p.rows + row] = best;
        __threadfence_system();
        for (int j = 0; j < p.world; ++j) red_relaxed_sys_add_u32(p.counters[j], 1u);
        int ok = 1;
        if (*(volatile unsigned int*)&p.status->status == SKY_STATUS_OK) {
            const unsigned want = tp_seq(p.seq) * p.seq.arrivals_per_use;
            for (int r = 0; r < p.world && ok; ++r)
                if (!wait_flag_ge(p.my_counters + r, want, p.timeout_ns)) {
                    set_status(p.status, SKY_STATUS_TIMEOUT_FLAG, 200u + (unsigned)r);
                    ok = 0;
                }
        }
        unsigned long long g = 0;
        for (int r = 0; r < p.world; ++r) {
            const unsigned long long c = __ldcg(p.my_slots + (long long)r * p.rows + row);
            g = c > g ? c : g;
        }
        p.next_ids[row] = (int)(0xffffffffu - (unsigned)(g & 0xffffffffull));
        s_ok = ok;
    }
}

cudaError_t launch_tp_argmax(const TpArgmaxParams& p, cudaStream_t stream) {
    if (p.rows <= 0 || p.world < 1 || p.world > TP_MAX_RANKS) return cudaErrorInvalidValue;
    return launch_pdl(tp_argmax_kernel, dim3(p.rows), dim3(256), 0, stream, p);
}

__global__ void step_increment_kernel(unsigned int* step) { pdl_wait(); *step += 1; }
cudaError_t launch_step_increment(unsigned int* step, cudaStream_t stream) {
    return launch_pdl(step_increment_kernel, dim3(1), dim3(1), 0, stream, step);
}

}  // namespace sky
