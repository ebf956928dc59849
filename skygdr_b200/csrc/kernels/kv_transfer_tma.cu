// Paged KV transfer, all-TMA variant for bf16 pages: the gather, the token-major -> head-major conversion and the
// peer write are done by the copy hardware of the SM; one thread per CTA drives it.
//
//   load : 3-D tensor map over the source pool viewed as [token][head][dim]; one box {128 dims, 1 head, 16 tokens}
//          per head lands that head's [16][128] tile at head*4 KB of a shared-memory slot, so the slot holds the page
//          in destination (head-major) order. Loads complete on an mbarrier. No cluster broadcast.
//   store: cp.async.bulk shared -> global of the slot (32 KB, or one piece per destination when heads are scattered or
//          the page is replicated) straight into the peer's pool: long contiguous writes for NVLink.
// Loads run LOOKAHEAD pages ahead of stores in a ring of SLOTS slots; a slot is reused once the store that read it
// has finished reading (bulk-group accounting). Chunks are ticketed and credit-gated exactly like the register
// variant (kv_transfer.cu), with which it shares parameters, status block and completion protocol; that one remains
// for fp8 packing and for layouts this one does not cover.
//
// Same reference counterpart: one contiguous cudaMemcpyPeerAsync per request
// (llm_problem_analysis/kv_nvlink_transfer.cu:109-122, llm_problem_analysis/kv_nvlink_transfer_trace.cu:378-393).
#include <cuda.h>

#include "common.cuh"
#include "kv_transfer.h"

namespace sky {
namespace {

constexpr int SLOTS = 6;
constexpr int LOOKAHEAD = 3;
constexpr int SLOT_BYTES = 32768;                 // 8 heads x 16 tokens x 128 x bf16
constexpr int TMA_THREADS = 32;

__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(TMA_THREADS) kv_transfer_tma_kernel(const __grid_constant__ CUtensorMap tmap, const KvTransferParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t full[SLOTS];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    if (threadIdx.x != 0) return;                  // one thread drives the copy hardware

    const long long pages_per_pair = 2LL * p.layers;
    const long long n_pages = pages_per_pair * p.n_pairs;
    const long long n_chunks = (n_pages + p.pages_per_chunk - 1) / p.pages_per_chunk;
    const uint32_t page_bytes = (uint32_t)p.heads * p.block_tokens * p.head_dim * 2;
    const unsigned long long page_link_bytes = (unsigned long long)page_bytes * (p.replicate ? p.n_dst : 1);
    const uint32_t piece = p.replicate ? page_bytes : (uint32_t)p.heads_per_dst * p.block_tokens * p.head_dim * 2;

    for (int s = 0; s < SLOTS; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmap);
    atomicMin(&p.status->t_start_ns, globaltimer_ns());

    unsigned long long grant_cache = 0, stall_ns = 0, my_bytes = 0, my_chunks = 0, last_need = 0;
    long long issued = 0, stored = 0;             // pages of this CTA whose loads / stores have been issued
    long long dst_off[SLOTS];                     // destination element offset of the page in each slot
    bool failed = false;

    auto store_page = [&](long long j) {           // j-th page of this CTA: wait for its loads, write it out
        const int s = (int)(j % SLOTS);
        if (!mbar_wait(&full[s], (uint32_t)(j / SLOTS) & 1)) { set_status(p.status, SKY_STATUS_TIMEOUT_MBAR, 21); failed = true; return; }
        const unsigned char* slot = smem + s * SLOT_BYTES;
        if (p.replicate) {
            for (int g = 0; g < p.n_dst; ++g) bulk_s2g((__nv_bfloat16*)p.dst[g] + dst_off[s], slot, page_bytes);
        } else {
            for (int g = 0; g < p.n_dst; ++g) bulk_s2g((__nv_bfloat16*)p.dst[g] + dst_off[s], slot + (size_t)g * piece, piece);
        }
        bulk_commit();
    };

    for (;;) {
        if (failed || *(volatile unsigned int*)&p.status->status != SKY_STATUS_OK) break;
        const unsigned long long k = p.first_chunk + atomicAdd(&p.status->work_counter, 1u);
        if ((long long)k >= n_chunks) break;
        const long long page0 = (long long)k * p.pages_per_chunk, page1 = min(page0 + p.pages_per_chunk, n_pages);
        const unsigned long long need = p.consumed_base + (unsigned long long)(page1 - (long long)p.first_chunk * p.pages_per_chunk) * page_link_bytes;
        bool stopped, lost;
        if (!credit_acquire(p.page, need, &grant_cache, p.max_wait_ns, &stall_ns, &stopped, &lost)) {
            atomicMin(&p.status->cursor, k);
            set_status(p.status, stopped ? SKY_STATUS_STOPPED : lost ? SKY_STATUS_CONTROL_LOST : SKY_STATUS_YIELD_CREDIT, (unsigned)k);
            break;
        }
        if (p.usage) {
            st_sys_u64((unsigned long long*)&p.usage->consumed_bytes, need);
            if (my_chunks) st_sys_u64((unsigned long long*)&p.usage->completed_bytes, last_need);
        }
        last_need = need;
        for (long long pg = page0; pg < page1 && !failed; ++pg) {
            const int pair = (int)(pg / pages_per_pair);
            const int rem = (int)(pg - (long long)pair * pages_per_pair);
            const int layer = rem >> 1, kv = rem & 1;
            const int sb = __ldg(p.src_blocks + pair), db = __ldg(p.dst_blocks + pair);
            if ((p.src_num_blocks && (unsigned)sb >= (unsigned)p.src_num_blocks) || (p.dst_num_blocks && (unsigned)db >= (unsigned)p.dst_num_blocks)) {
                set_status(p.status, SKY_STATUS_BAD_INDEX, (unsigned)pair);    // nothing is loaded or stored for this page
                continue;
            }
            // the slot about to be loaded was last read by the store of page (issued - SLOTS)
            bulk_wait_read<SLOTS - LOOKAHEAD - 1>();
            const int s = (int)(issued % SLOTS);
            const long long src_elem = (long long)sb * p.src_block_stride + (long long)layer * p.src_layer_stride + (long long)kv * p.src_kv_stride;
            const int tok_row = (int)(src_elem / ((long long)p.heads * p.head_dim));       // global token row of the page's first token
            dst_off[s] = (long long)db * p.dst_block_stride + (long long)layer * p.dst_layer_stride + (long long)kv * p.dst_kv_stride;
            mbar_expect_tx(&full[s], page_bytes);
            for (int h = 0; h < p.heads; ++h)
                tma_load_3d(smem + s * SLOT_BYTES + h * (p.block_tokens * p.head_dim * 2), &tmap, 0, h, tok_row, &full[s]);
            ++issued;
            if (issued - stored > LOOKAHEAD) { store_page(stored); ++stored; }
        }
        my_bytes += (unsigned long long)(page1 - page0) * page_link_bytes;
        ++my_chunks;
    }
    while (stored < issued && !failed) { store_page(stored); ++stored; }
    if (failed) {
        // loads already in flight must land before this CTA's shared memory goes away (bounded)
        for (long long j = stored; j < issued; ++j) mbar_wait(&full[j % SLOTS], (uint32_t)(j / SLOTS) & 1, 1000000ull);
    }
    bulk_wait_all();                               // every write of this CTA has completed

    if (my_chunks) { atomicAdd(&p.status->chunks_done, my_chunks); atomicAdd(&p.status->bytes_done, my_bytes); }
    if (stall_ns) atomicAdd(&p.status->stall_ns, stall_ns);
    asm volatile("fence.proxy.async;" ::: "memory");   // order the bulk writes (async proxy) before the generic-proxy signals below
    __threadfence_system();
    const unsigned prev = atomicAdd(&p.status->ctas_done, 1u);
    if (prev == gridDim.x - 1) {
        __threadfence();
        const unsigned long long now = globaltimer_ns();
        p.status->t_end_ns = now;
        const unsigned long long bytes = *(volatile unsigned long long*)&p.status->bytes_done;
        const bool complete = *(volatile unsigned int*)&p.status->status == SKY_STATUS_OK;
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// The source pool must be one contiguous token-major allocation: page (block, layer, kv) at
// block*src_block_stride + layer*src_layer_stride + kv*src_kv_stride, each [16 tokens][heads][128].
cudaError_t launch_kv_transfer_tma(const KvTransferParams& p, long long pool_elems, int ctas, cudaStream_t stream) {
    if (p.fp8 || p.keep_layout || p.head_dim != 128 || p.block_tokens != 16 || p.heads < 1 || p.heads > 8) return cudaErrorInvalidValue;
    if (p.n_dst < 1 || p.n_dst > KV_MAX_DST || p.pages_per_chunk < 1) return cudaErrorInvalidValue;
    if (!p.replicate && p.heads_per_dst * p.n_dst != p.heads) return cudaErrorInvalidValue;
    const long long row = (long long)p.heads * p.head_dim;                   // elements per token row
    if (p.src_block_stride % row || p.src_layer_stride % row || p.src_kv_stride % row || pool_elems % row) return cudaErrorInvalidValue;
    if ((p.dst_block_stride | p.dst_layer_stride | p.dst_kv_stride) & 7) return cudaErrorInvalidValue;   // 16-byte aligned pieces
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return cudaErrorNotSupported;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    CUtensorMap tm;
    const cuuint64_t dims[3] = {128, (cuuint64_t)p.heads, (cuuint64_t)(pool_elems / row)};
    const cuuint64_t strides[2] = {256, (cuuint64_t)row * 2};
    const cuuint32_t box[3] = {128, 1, 16};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(p.src_pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    constexpr int smem_bytes = SLOTS * SLOT_BYTES + 128;
    static unsigned long long attr_mask = 0;
    if (cudaError_t e = set_max_dynamic_smem_once(reinterpret_cast<const void*>(kv_transfer_tma_kernel), smem_bytes, &attr_mask); e != cudaSuccess) return e;
    kv_transfer_tma_kernel<<<ctas, TMA_THREADS, smem_bytes, stream>>>(tm, p);
    return cudaGetLastError();
}

}  // namespace sky
