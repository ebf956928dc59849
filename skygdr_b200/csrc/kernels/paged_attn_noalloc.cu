// Allocation-free entry point for paged GQA decode attention: the split-KV scratch is a fixed
// device array of this file instead of caller- or torch-allocated memory. See paged_attn_noalloc.h
// for who needs this, the limits, and the sharing rules.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "common_host.h"
#include "paged_attn.h"
#include "paged_attn_noalloc.h"

namespace {

// The scratch itself. In host code this name is only a handle for the runtime's symbol table, not
// a device address: the address is obtained with cudaGetSymbolAddress below and that is what the
// kernel receives.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SKYGDR_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {nullptr};

int fail(int code, char* err, size_t err_len, const char* fmt, const char* a = "", long long b = 0, long long c = 0) {
    if (err && err_len) snprintf(err, err_len, fmt, a, b, c);
    return code;
}

// Device address of the scratch on the current device; looked up once per device. The first lookup on a device is what
// makes the runtime load this module there (lazy loading), which is when the array's memory is reserved; the kernels'
// per-device attributes are set in the same step so that nothing is left to load or set at the first launch.
int scratch_for_current_device(void** out, char* err, size_t err_len) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(SKYGDR_NOALLOC_E_CUDA, err, err_len, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%sdevice ordinal %lld out of range", "", dev);
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(SKYGDR_NOALLOC_E_CUDA, err, err_len, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        e = sky::prepare_paged_attn_decode();
        if (e != cudaSuccess)
            return fail(SKYGDR_NOALLOC_E_CUDA, err, err_len, "kernel set-up (cudaFuncSetAttribute): %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return SKYGDR_NOALLOC_OK;
}

sky::LaunchStatus* status_slot(void* base) {
    unsigned char* b = static_cast<unsigned char*>(base);
    return reinterpret_cast<sky::LaunchStatus*>(b + (size_t)SKYGDR_NOALLOC_MAX_ROWS * 130 * 4 + (size_t)SKYGDR_NOALLOC_MAX_PAIRS * 4);
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int skygdr_paged_attn_noalloc_init(char* err, size_t err_len) {
    void* base = nullptr;
    return scratch_for_current_device(&base, err, err_len);
}

extern "C" __attribute__((visibility("default"))) int skygdr_paged_attn_noalloc_status(unsigned int* code, unsigned int* detail, void* stream) {
    if (!code) return SKYGDR_NOALLOC_E_BAD_ARG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SKYGDR_NOALLOC_E_CUDA;
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> g(g_mu);
        base = g_scratch_addr[dev];
    }
    if (!base) return SKYGDR_NOALLOC_E_BAD_ARG;            // no call has been made on this device
    unsigned int words[2] = {0, 0};                        // LaunchStatus begins with status, detail
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(words, status_slot(base), sizeof words, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return SKYGDR_NOALLOC_E_CUDA;
    *code = words[0];
    if (detail) *detail = words[1];
    return SKYGDR_NOALLOC_OK;
}

extern "C" __attribute__((visibility("default"))) int skygdr_paged_attn_decode_noalloc(
    const void* q, const void* kv_layer, void* out, const int* block_table, const int* ctx_lens, long long block_stride,
    long long kv_stride, long long head_stride, int batch, int q_heads, int kv_heads, int max_blocks, int num_blocks, int max_ctx,
    int chunk_tokens, float scale, void* stream, char* err, size_t err_len) {
    if (!q || !kv_layer || !out || !block_table || !ctx_lens)
        return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%snull pointer argument");
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || max_blocks <= 0 || max_ctx <= 0)
        return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%sbatch, head counts, max_blocks and max_ctx must be positive, q_heads a multiple of kv_heads");
    const int group = q_heads / kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 8)
        return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%sq_heads / kv_heads must be 1, 2, 4 or 8 (got %lld)", "", group);
    if ((long long)max_ctx > (long long)max_blocks * 16)
        return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%smax_ctx = %lld but a block-table row covers only %lld tokens", "", max_ctx,
                    (long long)max_blocks * 16);
    if (num_blocks < 0) return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%snum_blocks must be >= 0 (0 = unknown)");
    if (chunk_tokens <= 0 || chunk_tokens % 64)
        return fail(SKYGDR_NOALLOC_E_BAD_ARG, err, err_len, "%schunk_tokens must be a positive multiple of 64 (got %lld)", "", chunk_tokens);
    const long long splits = ((long long)max_ctx + chunk_tokens - 1) / chunk_tokens;
    const long long rows = (long long)batch * q_heads * splits;
    const long long pairs = (long long)batch * kv_heads;
    if (rows > SKYGDR_NOALLOC_MAX_ROWS)
        return fail(SKYGDR_NOALLOC_E_TOO_LARGE, err, err_len,
                    "%sbatch*q_heads*ceil(max_ctx/chunk_tokens) = %lld exceeds the built-in scratch (%lld rows): use a larger chunk_tokens, a smaller batch, or the allocating entry point",
                    "", rows, (long long)SKYGDR_NOALLOC_MAX_ROWS);
    if (pairs > SKYGDR_NOALLOC_MAX_PAIRS)
        return fail(SKYGDR_NOALLOC_E_TOO_LARGE, err, err_len, "%sbatch*kv_heads = %lld exceeds the built-in scratch (%lld pairs)", "", pairs,
                    (long long)SKYGDR_NOALLOC_MAX_PAIRS);

    void* base = nullptr;
    int rc = scratch_for_current_device(&base, err, err_len);
    if (rc != SKYGDR_NOALLOC_OK) return rc;

    // carve the array: [part_o rows*128 f32][part_m rows f32][part_l rows f32][counters][status]
    unsigned char* b = static_cast<unsigned char*>(base);
    float* part_o = reinterpret_cast<float*>(b);
    float* part_m = reinterpret_cast<float*>(b + (size_t)SKYGDR_NOALLOC_MAX_ROWS * 128 * 4);
    float* part_l = part_m + SKYGDR_NOALLOC_MAX_ROWS;
    unsigned int* counters = reinterpret_cast<unsigned int*>(part_l + SKYGDR_NOALLOC_MAX_ROWS);
    sky::LaunchStatus* status = status_slot(base);
    static_assert(sizeof(sky::LaunchStatus) <= 256, "status block must fit its slot");

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // what must start at zero: the counters of the pairs in use (a previous call that was cut short
    // may have left them mid-count) and the status block
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)pairs * sizeof(unsigned int), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(status, 0, 256, s);
    if (e != cudaSuccess) return fail(SKYGDR_NOALLOC_E_CUDA, err, err_len, "cudaMemsetAsync(scratch): %s", cudaGetErrorString(e));

    sky::PagedAttnParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.kv = static_cast<const __nv_bfloat16*>(kv_layer);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.block_table = block_table;
    p.ctx_lens = ctx_lens;
    p.block_stride = block_stride; p.kv_stride = kv_stride; p.head_stride = head_stride;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = 128; p.block_tokens = 16; p.max_blocks = max_blocks;
    p.num_blocks = num_blocks;
    p.max_ctx = max_ctx; p.chunk_tokens = chunk_tokens; p.max_splits = (int)splits; p.scale = scale;
    p.part_o = part_o; p.part_m = part_m; p.part_l = part_l; p.counters = counters; p.status = status;
    e = sky::launch_paged_attn_decode(p, s);
    if (e != cudaSuccess) return fail(SKYGDR_NOALLOC_E_CUDA, err, err_len, "paged attention launch: %s", cudaGetErrorString(e));
    return SKYGDR_NOALLOC_OK;
}
