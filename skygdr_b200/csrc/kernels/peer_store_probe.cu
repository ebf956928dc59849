// Store-only probe: what SM-originated writes into another GPU's memory can reach, with nothing else in the way.
//
// The paged transfer kernels (kv_transfer.cu, kv_transfer_tma.cu) gather, convert the layout and write to a peer; their
// link rate is bounded by what the SMs' write path over NVLink sustains. This kernel only writes: no loads, no gather,
// no credit gate. It gives that bound for the store forms the transfer kernels can choose from:
//   mode 0: st.global.v4 from registers, one 16-byte store per thread per step (what kv_transfer.cu issues)
//   mode 1: cp.async.bulk shared -> global of `store_bytes` per copy, `inflight` bulk groups outstanding per CTA before
//           the issuing thread waits (what kv_transfer_tma.cu issues)
//   mode 2: multimem.st through an NVLink multicast address (mode 0's store, delivered by the switch to every bound GPU)
// Every CTA writes its own contiguous span of `dst`, again and again for `iters` rounds.
//
// The reference measures the copy engine only (cudaMemcpyPeerAsync, llm_problem_analysis/kv_nvlink_transfer.cu:109-137).
#include "common.cuh"
#include "peer_store_probe.h"

namespace sky {
namespace {

constexpr int PROBE_THREADS = 256;
constexpr int PROBE_SMEM = 64 * 1024;

__global__ void __launch_bounds__(PROBE_THREADS) peer_store_probe_kernel(unsigned char* dst, unsigned long long span_bytes, int mode,
                                                                          unsigned store_bytes, int inflight, int iters) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* mine = dst + (unsigned long long)blockIdx.x * span_bytes;
    if (mode == 1) {
        for (int i = threadIdx.x; i < PROBE_SMEM / 16; i += PROBE_THREADS)
            reinterpret_cast<uint4*>(smem)[i] = make_uint4(i, blockIdx.x, 0x5a5a5a5au, 0xa5a5a5a5u);
        fence_proxy_async();
        __syncthreads();
        if (threadIdx.x != 0) return;
        const unsigned long long n = span_bytes / store_bytes;
        for (int it = 0; it < iters; ++it) {
            for (unsigned long long i = 0; i < n; ++i) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(mine + i * store_bytes), "r"(smem_u32(smem + (i % (PROBE_SMEM / store_bytes)) * store_bytes)), "r"(store_bytes) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                // at most `inflight` groups outstanding (the instruction takes an immediate: pick the nearest form)
                if (inflight <= 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                else if (inflight <= 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                else if (inflight <= 4) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
                else asm volatile("cp.async.bulk.wait_group.read 7;" ::: "memory");
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        return;
    }
    const uint4 v = make_uint4(threadIdx.x, blockIdx.x, 0x5a5a5a5au, 0xa5a5a5a5u);
    const unsigned long long n = span_bytes / 16;
    for (int it = 0; it < iters; ++it) {
        if (mode == 0) {
#pragma unroll 4
            for (unsigned long long i = threadIdx.x; i < n; i += PROBE_THREADS) st_v4(mine + i * 16, v);
        } else {
#pragma unroll 4
            for (unsigned long long i = threadIdx.x; i < n; i += PROBE_THREADS) multimem_st_v4(mine + i * 16, v);
        }
    }
}

}  // namespace

cudaError_t launch_peer_store_probe(void* dst, unsigned long long total_bytes, int mode, unsigned store_bytes, int inflight, int ctas,
                                    int iters, cudaStream_t stream) {
    if (!dst || ctas < 1 || iters < 1 || mode < 0 || mode > 2) return cudaErrorInvalidValue;
    if (mode == 1 && (store_bytes < 16 || store_bytes % 16 || store_bytes > PROBE_SMEM || PROBE_SMEM % store_bytes)) return cudaErrorInvalidValue;
    const unsigned long long unit = mode == 1 ? store_bytes : 16ull * PROBE_THREADS;
    const unsigned long long span = total_bytes / (unsigned long long)ctas / unit * unit;
    if (span == 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return cudaErrorInvalidValue;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(peer_store_probe_kernel), PROBE_SMEM, &attr_mask); e != cudaSuccess) return e;
    peer_store_probe_kernel<<<ctas, PROBE_THREADS, PROBE_SMEM, stream>>>(static_cast<unsigned char*>(dst), span, mode, store_bytes, inflight, iters);
    return cudaGetLastError();
}

}  // namespace sky
