// Small fused decoder ops: RMSNorm (+ residual add), per-head QK-norm + RoPE +
// KV append into the paged cache, SiLU*mul, embedding gather, argmax.
//
// The reference's decode stressors only append raw K/V rows
// (llm_problem_analysis/decode_transformer_kvcache_stress.cu:360-391,
// llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu:284-328) and model the MLP
// as a streaming pass (decode_transformer_kvcache_stress.cu:323-356); these are the
// real ops of a Qwen3 decoder layer.
#include "common.cuh"
#include "fused_ops.h"

namespace sky {

__device__ __forceinline__ void unpack8(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];
    __syncthreads();
    return t;
}

// One CTA per row; each thread owns up to 4 vectors of 8 elements (hidden <= 256*8*4 = 8192).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                                                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                       int hidden, float eps) {
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const long long row = blockIdx.x;
    const int nvec = hidden / 8;
    float vals[4][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nvec) {
            unpack8(*reinterpret_cast<const uint4*>(x + row * hidden + v * 8), vals[k]);
            if (residual) {
                float r[8];
                unpack8(*reinterpret_cast<const uint4*>(residual + row * hidden + v * 8), r);
#pragma unroll
                for (int i = 0; i < 8; ++i) vals[k][i] += r[i];
                uint4 packed = pack8(vals[k]);
                *reinterpret_cast<uint4*>(residual + row * hidden + v * 8) = packed;
                unpack8(packed, vals[k]);  // normalise what was stored (bf16-rounded), as a two-kernel version would
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += vals[k][i] * vals[k][i];
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / hidden + eps);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nvec) {
            float g[8], o[8];
            unpack8(*reinterpret_cast<const uint4*>(w + v * 8), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = vals[k][i] * inv * g[i];
            *reinterpret_cast<uint4*>(y + row * hidden + v * 8) = pack8(o);
        }
    }
}

cudaError_t launch_rmsnorm(const __nv_bfloat16* x, __nv_bfloat16* residual, const __nv_bfloat16* w, __nv_bfloat16* y,
                           int rows, int hidden, float eps, cudaStream_t stream) {
    if (hidden % 8 || hidden > 8192 || rows <= 0) return cudaErrorInvalidValue;
    return launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, stream, x, residual, w, y, hidden, eps);
}

// One warp per (token, head) over q heads, k heads and v heads; lane owns dims [4*lane, 4*lane+4).
// Rotation pairs dim i with dim i+64, i.e. lane L with lane L^16.
__global__ void __launch_bounds__(128) rope_append_kernel(const RopeAppendParams p) {
    pdl_trigger();
    pdl_wait();
    const int heads_total = p.q_heads + 2 * p.kv_heads;
    const long long gw = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (gw >= (long long)p.tokens * heads_total) return;
    const int tok = (int)(gw / heads_total), h = (int)(gw % heads_total);
    const int lane = threadIdx.x & 31;
    const __nv_bfloat16* src = p.qkv + ((long long)tok * heads_total + h) * 128 + lane * 4;
    uint2 raw = *reinterpret_cast<const uint2*>(src);
    float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                  __uint_as_float(raw.y & 0xffff0000u)};
    const bool is_q = h < p.q_heads, is_k = !is_q && h < p.q_heads + p.kv_heads;
    const int pos = p.positions[tok];
    if (is_q || is_k) {
        const __nv_bfloat16* nw = is_q ? p.q_norm : p.k_norm;
        if (nw) {
            float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
            uint2 wr = *reinterpret_cast<const uint2*>(nw + lane * 4);
            float g[4] = {__uint_as_float(wr.x << 16), __uint_as_float(wr.x & 0xffff0000u), __uint_as_float(wr.y << 16),
                          __uint_as_float(wr.y & 0xffff0000u)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // round to bf16 like a separate norm kernel would, so results match a layer-by-layer reference
                x[i] = __bfloat162float(__float2bfloat16(x[i] * inv * g[i]));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int dim = (lane & 15) * 4 + i;  // frequency index 0..63
            // angle in fp32 as the usual eager implementation forms it, then an exact reduction to
            // [0, 2pi) in double so that the fast sincos stays accurate at positions of tens of thousands
            const float ang = __fmul_rn((float)pos, __ldg(p.inv_freq + dim));
            const double two_pi = 6.283185307179586476925;
            const double red = (double)ang - two_pi * floor((double)ang * (1.0 / two_pi));
            float sn, cs;
            __sincosf((float)red, &sn, &cs);
            const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
            x[i] = lane < 16 ? x[i] * cs - other * sn : x[i] * cs + other * sn;
        }
    }
    uint2 outv = make_uint2(pack2(x[0], x[1]), pack2(x[2], x[3]));
    if (is_q) {
        *reinterpret_cast<uint2*>(p.q_out + ((long long)tok * p.q_heads + h) * 128 + lane * 4) = outv;
    } else {
        const int kvh = is_k ? h - p.q_heads : h - p.q_heads - p.kv_heads;
        const int seq = p.seq_ids ? p.seq_ids[tok] : tok;
        const int blk = p.block_table[(long long)seq * p.max_blocks + pos / p.block_tokens];
        const int slot = pos % p.block_tokens;
        __nv_bfloat16* dst = p.kv + (long long)blk * p.block_stride + (is_k ? 0 : p.kv_stride) + (long long)kvh * p.head_stride +
                             (long long)slot * p.tok_stride + lane * 4;
        *reinterpret_cast<uint2*>(dst) = outv;
    }
}

cudaError_t launch_rope_append(const RopeAppendParams& p, cudaStream_t stream) {
    if (p.tokens <= 0) return cudaErrorInvalidValue;
    const long long warps = (long long)p.tokens * (p.q_heads + 2 * p.kv_heads);
    return launch_pdl(rope_append_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, p);
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                                        long long n_vec, int ffn_vec) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n_vec) return;
    const long long r = i / ffn_vec;
    const int c = (int)(i - r * ffn_vec);
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + (r * 2 * ffn_vec + c) * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + (r * 2 * ffn_vec + ffn_vec + c) * 8), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
    *reinterpret_cast<uint4*>(out + i * 8) = pack8(o);
}

cudaError_t launch_silu_mul(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int rows, int ffn, cudaStream_t stream) {
    if (ffn % 8 || rows <= 0) return cudaErrorInvalidValue;
    const long long n_vec = (long long)rows * (ffn / 8);
    silu_mul_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, stream>>>(gate_up, out, n_vec, ffn / 8);
    return cudaGetLastError();
}

__global__ void __launch_bounds__(128) embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                                         __nv_bfloat16* __restrict__ out, int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int tok = blockIdx.x;
    int id = ids[tok];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int v = threadIdx.x; v < hidden / 8; v += 128)
        *reinterpret_cast<uint4*>(out + (long long)tok * hidden + v * 8) = *reinterpret_cast<const uint4*>(table + (long long)id * hidden + v * 8);
}

cudaError_t launch_embedding(const int* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int tokens, int hidden, int vocab,
                             cudaStream_t stream) {
    if (hidden % 8 || tokens <= 0) return cudaErrorInvalidValue;
    return launch_pdl(embedding_kernel, dim3(tokens), dim3(128), 0, stream, ids, table, out, hidden, vocab);
}

__global__ void __launch_bounds__(1024) argmax_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int vocab,
                                                       long long row_stride) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    const __nv_bfloat16* row = logits + (long long)blockIdx.x * row_stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < vocab; c += 1024) {
        const float v = __bfloat162float(row[c]);
        if (v > best || (v == best && c < bi)) { best = v; bi = c; }
    }
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x]; bi = si[threadIdx.x];
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi;
    }
}

// Temperature sampling without a normalisation pass (Gumbel-max): argmax_c (logit_c / T + g_c) with g_c = -log(-log(u_c)) and
// u_c uniform in (0, 1) picks column c with probability softmax(logits / T)_c. u_c comes from a counter-based hash of
// (seed, position of the row's sequence, row, column), so a replayed CUDA graph draws fresh noise every step (the position
// advances) and a given (seed, position) always draws the same token. The hash is restated in skygdr_b200/ops/small.py.
__device__ __forceinline__ unsigned int sample_hash(unsigned int seed, unsigned int pos, unsigned int row, unsigned int col) {
    unsigned int h = seed * 0x9E3779B1u ^ (pos + 0x7F4A7C15u) * 0x85EBCA77u ^ (row + 0x165667B1u) * 0xC2B2AE3Du ^ (col + 0x27D4EB2Fu) * 0x9E3779B1u;
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;      // murmur3 finaliser
    return h;
}

__global__ void __launch_bounds__(1024) sample_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int vocab,
                                                       long long row_stride, float inv_temperature, unsigned int seed,
                                                       const int* __restrict__ positions) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    const __nv_bfloat16* row = logits + (long long)blockIdx.x * row_stride;
    const unsigned int pos = positions ? (unsigned int)positions[blockIdx.x] : 0u;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < vocab; c += 1024) {
        const float u = ((float)(sample_hash(seed, pos, blockIdx.x, (unsigned int)c) >> 8) + 0.5f) * (1.0f / 16777216.0f);
        const float v = __bfloat162float(row[c]) * inv_temperature - logf(-logf(u));
        if (v > best || (v == best && c < bi)) { best = v; bi = c; }
    }
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x]; bi = si[threadIdx.x];
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi;
    }
}

cudaError_t launch_sample(const __nv_bfloat16* logits, int* out, int rows, int vocab, long long row_stride, float temperature,
                          unsigned int seed, const int* positions, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0 || !(temperature > 0.f)) return cudaErrorInvalidValue;
    return launch_pdl(sample_kernel, dim3(rows), dim3(1024), 0, stream, logits, out, vocab, row_stride, 1.0f / temperature, seed, positions);
}

cudaError_t launch_argmax(const __nv_bfloat16* logits, int* out, int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return cudaErrorInvalidValue;
    return launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, stream, logits, out, vocab, row_stride);
}

}  // namespace sky
