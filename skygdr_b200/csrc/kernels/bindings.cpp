// Python bindings of the CUDA side (module skygdr_b200._C).
//
// Tensors own all local GPU memory. Peer or host-mapped destinations are passed
// as integer addresses, because they are not tensors of this process.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>

#include "common_host.h"
#include "fused_ops.h"
#include "gemm_tcgen05.h"
#include "kv_transfer.h"
#include "memhog.h"
#include "multicast.h"
#include "paged_attn.h"
#include "pcie_task.h"
#include "peer_store_probe.h"
#include "prefill_attn.h"
#include "tp_fused.h"

namespace py = pybind11;
using namespace sky;

#define SKY_CUDA_CHECK(expr)                                                                              \
    do {                                                                                                  \
        cudaError_t _e = (expr);                                                                          \
        TORCH_CHECK(_e == cudaSuccess, #expr, " failed: ", cudaGetErrorString(_e));                       \
    } while (0)

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static const __nv_bfloat16* bf16_ptr(const torch::Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, "expected a CUDA bf16 tensor");
    return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr());
}
static __nv_bfloat16* bf16_mut(torch::Tensor& t) { return const_cast<__nv_bfloat16*>(bf16_ptr(t)); }
static const int* i32_ptr(const torch::Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), "expected a contiguous CUDA int32 tensor");
    return t.data_ptr<int>();
}
static LaunchStatus* status_ptr(torch::Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.numel() * t.element_size() >= (int64_t)sizeof(LaunchStatus), "status tensor too small");
    return reinterpret_cast<LaunchStatus*>(t.data_ptr());
}

// A fresh status block: OK, cursor and t_start at their "unset" value of all ones.
static torch::Tensor new_status(int64_t device) {
    LaunchStatus h;
    memset(&h, 0, sizeof h);
    h.cursor = ~0ull;
    h.t_start_ns = ~0ull;
    auto cpu = torch::empty({(int64_t)sizeof(LaunchStatus)}, torch::kUInt8);
    memcpy(cpu.data_ptr(), &h, sizeof h);
    return cpu.to(torch::Device(torch::kCUDA, device));
}
static void reset_status(torch::Tensor& t) {
    LaunchStatus h;
    memset(&h, 0, sizeof h);
    h.cursor = ~0ull;
    h.t_start_ns = ~0ull;
    SKY_CUDA_CHECK(cudaMemcpyAsync(t.data_ptr(), &h, sizeof h, cudaMemcpyHostToDevice, cur_stream()));
}
static py::dict read_status(const torch::Tensor& t) {
    auto cpu = t.cpu();
    LaunchStatus h;
    memcpy(&h, cpu.data_ptr(), sizeof h);
    py::dict d;
    d["status"] = h.status; d["detail"] = h.detail; d["cursor"] = h.cursor; d["chunks_done"] = h.chunks_done;
    d["bytes_done"] = h.bytes_done; d["stall_ns"] = h.stall_ns; d["t_start_ns"] = h.t_start_ns; d["t_end_ns"] = h.t_end_ns;
    d["ctas_done"] = h.ctas_done;
    return d;
}

// ---- mapped host memory (credit pages, offload targets) ----
static std::pair<uint64_t, uint64_t> host_alloc_mapped(uint64_t bytes) {
    void* h = nullptr;
    SKY_CUDA_CHECK(cudaHostAlloc(&h, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(h, 0, bytes);
    void* d = nullptr;
    SKY_CUDA_CHECK(cudaHostGetDevicePointer(&d, h, 0));
    return {(uint64_t)h, (uint64_t)d};
}
static void host_free_mapped(uint64_t host_ptr) { cudaFreeHost((void*)host_ptr); }
// Page-locks and maps an existing host range (a /dev/shm credit page mapped by the caller).
static uint64_t host_register(uint64_t host_ptr, uint64_t bytes) {
    SKY_CUDA_CHECK(cudaHostRegister((void*)host_ptr, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
    void* d = nullptr;
    SKY_CUDA_CHECK(cudaHostGetDevicePointer(&d, (void*)host_ptr, 0));
    return (uint64_t)d;
}
static void host_unregister(uint64_t host_ptr) { cudaHostUnregister((void*)host_ptr); }

// Grant half of a credit page that lives in this process (in-process pacing without a daemon).
static void credit_page_init(uint64_t host_ptr, uint32_t flow_id, bool unlimited) {
    auto* p = (SkyCreditPage*)host_ptr;
    memset(p, 0, sizeof *p);
    p->flow_id = flow_id;
    p->mode = SKY_MODE_HIGH;
    p->unlimited = unlimited ? 1 : 0;
    __atomic_store_n(&p->magic, SKYGDR_CREDIT_MAGIC, __ATOMIC_RELEASE);
}
static void credit_page_grant(uint64_t host_ptr, uint64_t granted, bool unlimited, bool stop) {
    auto* p = (SkyCreditPage*)host_ptr;
    p->unlimited = unlimited ? 1 : 0;
    p->stop = stop ? 1 : 0;
    __atomic_store_n(&p->granted_bytes, granted, __ATOMIC_RELEASE);
    __atomic_store_n(&p->epoch, p->epoch + 1, __ATOMIC_RELEASE);
}
static void credit_page_heartbeat(uint64_t host_ptr, uint64_t window_ns, uint32_t dead_after_windows, uint32_t dead_policy,
                                  uint64_t fallback_per_window) {
    auto* p = (SkyCreditPage*)host_ptr;
    p->window_ns = window_ns;
    p->dead_policy = dead_policy;
    p->fallback_per_window = fallback_per_window;
    __atomic_store_n(&p->dead_after_windows, dead_after_windows, __ATOMIC_RELEASE);
}
static py::dict credit_page_read(uint64_t host_ptr) {
    auto* p = (SkyCreditPage*)host_ptr;
    py::dict d;
    d["granted_bytes"] = p->granted_bytes; d["epoch"] = p->epoch; d["unlimited"] = p->unlimited; d["stop"] = p->stop;
    d["mode"] = p->mode; d["consumed_bytes"] = p->consumed_bytes; d["completed_bytes"] = p->completed_bytes;
    d["stall_ns"] = p->stall_ns; d["busy_ns"] = p->busy_ns; d["chunks"] = p->chunks; d["yields"] = p->yields;
    d["backlog_bytes"] = p->backlog_bytes; d["last_ts_ns"] = p->last_ts_ns;
    d["heartbeat_lost"] = p->heartbeat_lost; d["heartbeat_lost_ns"] = p->heartbeat_lost_ns; d["window_ns"] = p->window_ns;
    d["dead_after_windows"] = p->dead_after_windows; d["dead_policy"] = p->dead_policy;
    return d;
}

// ---- peer memory through CUDA IPC ----
static std::pair<uint64_t, py::bytes> ipc_alloc(uint64_t bytes) {
    void* d = nullptr;
    SKY_CUDA_CHECK(cudaMalloc(&d, bytes));
    SKY_CUDA_CHECK(cudaMemset(d, 0, bytes));
    cudaIpcMemHandle_t h;
    SKY_CUDA_CHECK(cudaIpcGetMemHandle(&h, d));
    return {(uint64_t)d, py::bytes(reinterpret_cast<const char*>(&h), sizeof h)};
}
static uint64_t ipc_open(const std::string& handle) {
    TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle.data(), sizeof h);
    void* d = nullptr;
    SKY_CUDA_CHECK(cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess));
    return (uint64_t)d;
}
static void ipc_close(uint64_t ptr) { cudaIpcCloseMemHandle((void*)ptr); }
static void ipc_free(uint64_t ptr) { cudaFree((void*)ptr); }
static torch::Tensor tensor_from_ptr(uint64_t ptr, std::vector<int64_t> shape, py::object dtype, int64_t device) {
    auto st = torch::python::detail::py_object_to_dtype(dtype);
    return torch::from_blob((void*)ptr, shape, torch::TensorOptions().dtype(st).device(torch::kCUDA, device));
}
// Single-process multi-GPU (tests): lets `device` reach `peer`'s memory.
// Store-only probe of the SM write path: launches on `device` (its current stream), writes to `dst_ptr` (a peer pointer or a
// multicast address), returns the device time of the launch in milliseconds (CUDA events around it).
static double peer_store_probe(int device, uint64_t dst_ptr, uint64_t total_bytes, int mode, int store_bytes, int inflight, int ctas, int iters) {
    c10::cuda::CUDAGuard g(c10::Device(c10::kCUDA, (c10::DeviceIndex)device));
    cudaStream_t s = cur_stream();
    cudaEvent_t e0, e1;
    SKY_CUDA_CHECK(cudaEventCreate(&e0));
    SKY_CUDA_CHECK(cudaEventCreate(&e1));
    SKY_CUDA_CHECK(cudaEventRecord(e0, s));
    cudaError_t err = launch_peer_store_probe((void*)dst_ptr, total_bytes, mode, (unsigned)store_bytes, inflight, ctas, iters, s);
    cudaEventRecord(e1, s);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    SKY_CUDA_CHECK(err);
    return (double)ms;
}

static bool enable_peer_access(int device, int peer) {
    int can = 0;
    SKY_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, device, peer));
    if (!can) return false;
    c10::cuda::CUDAGuard g(device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return true; }
    return e == cudaSuccess;
}

// ---- kv transfer ----
static void kv_transfer(torch::Tensor src_pool, std::vector<uint64_t> dst_ptrs, std::vector<uint64_t> dst_scale_ptrs,
                        std::vector<uint64_t> done_flag_ptrs, torch::Tensor src_blocks, torch::Tensor dst_blocks, int layers, int heads,
                        int block_tokens, int head_dim, std::vector<int64_t> src_strides, std::vector<int64_t> dst_strides,
                        int heads_per_dst, bool replicate, bool fp8, bool keep_layout, int pages_per_chunk, int ctas, uint64_t credit_dev_ptr,
                        uint64_t consumed_base, uint64_t max_wait_ns, uint64_t first_chunk, uint32_t done_value, torch::Tensor status,
                        bool use_tma, uint64_t multicast_ptr, int src_num_blocks, int dst_num_blocks) {
    TORCH_CHECK(!(multicast_ptr && (use_tma || fp8 || !replicate)), "a multicast destination takes replicated bf16 pages from the register path");
    TORCH_CHECK(dst_ptrs.size() >= 1 && dst_ptrs.size() <= (size_t)KV_MAX_DST, "1..8 destinations");
    TORCH_CHECK(src_strides.size() == 3 && dst_strides.size() == 3, "strides are (block, layer, kv)");
    TORCH_CHECK(src_blocks.numel() == dst_blocks.numel(), "block lists differ in length");
    c10::cuda::CUDAGuard g(src_pool.device());
    KvTransferParams p;
    memset(&p, 0, sizeof p);
    p.src_pool = bf16_ptr(src_pool);
    for (size_t i = 0; i < dst_ptrs.size(); ++i) {
        p.dst[i] = (void*)dst_ptrs[i];
        p.dst_scales[i] = i < dst_scale_ptrs.size() ? (void*)dst_scale_ptrs[i] : nullptr;
        p.done_flag[i] = i < done_flag_ptrs.size() ? (unsigned int*)done_flag_ptrs[i] : nullptr;
    }
    p.mc_dst = (void*)multicast_ptr;
    p.src_num_blocks = src_num_blocks; p.dst_num_blocks = dst_num_blocks;
    p.src_blocks = i32_ptr(src_blocks);
    p.dst_blocks = i32_ptr(dst_blocks);
    p.n_pairs = (int)src_blocks.numel();
    p.layers = layers; p.heads = heads; p.block_tokens = block_tokens; p.head_dim = head_dim;
    p.src_block_stride = src_strides[0]; p.src_layer_stride = src_strides[1]; p.src_kv_stride = src_strides[2];
    p.dst_block_stride = dst_strides[0]; p.dst_layer_stride = dst_strides[1]; p.dst_kv_stride = dst_strides[2];
    p.n_dst = (int)dst_ptrs.size();
    p.heads_per_dst = heads_per_dst; p.replicate = replicate; p.fp8 = fp8; p.keep_layout = keep_layout;
    p.pages_per_chunk = pages_per_chunk;
    p.done_value = done_value;
    p.page = (const SkyCreditPage*)credit_dev_ptr;
    p.usage = (SkyCreditPage*)credit_dev_ptr;
    p.consumed_base = consumed_base; p.max_wait_ns = max_wait_ns; p.first_chunk = first_chunk;
    p.status = status_ptr(status);
    if (p.n_pairs == 0) return;
    if (use_tma) SKY_CUDA_CHECK(launch_kv_transfer_tma(p, src_pool.numel(), ctas, cur_stream()));
    else SKY_CUDA_CHECK(launch_kv_transfer(p, ctas, cur_stream()));
}

// ---- causal prefill attention over the paged pool ----
static void prefill_attn(torch::Tensor q, torch::Tensor kv_layer, torch::Tensor out, torch::Tensor block_table, torch::Tensor seq_start,
                         int64_t block_stride, int64_t kv_stride, int64_t head_stride, int64_t tok_stride, int kv_heads, int max_len, double scale,
                         torch::Tensor status, int64_t pool_rows, c10::optional<torch::Tensor> pos0) {
    c10::cuda::CUDAGuard g(q.device());
    TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.is_contiguous() && out.is_contiguous() && out.sizes() == q.sizes(), "q/out: contiguous [tokens][heads][128]");
    TORCH_CHECK(block_table.dim() == 2 && seq_start.numel() == block_table.size(0) + 1, "seq_start holds n_seqs + 1 offsets");
    PrefillAttnParams p;
    memset(&p, 0, sizeof p);
    p.q = bf16_ptr(q); p.kv = bf16_ptr(kv_layer); p.out = bf16_mut(out);
    p.block_table = i32_ptr(block_table); p.seq_start = i32_ptr(seq_start);
    p.block_stride = block_stride; p.kv_stride = kv_stride; p.head_stride = head_stride; p.tok_stride = tok_stride;
    p.n_seqs = (int)block_table.size(0); p.q_heads = (int)q.size(1); p.kv_heads = kv_heads; p.max_blocks = (int)block_table.size(1);
    p.max_len = max_len; p.total_tokens = (int)q.size(0); p.scale = (float)scale;
    if (pos0.has_value()) {
        TORCH_CHECK(pos0->scalar_type() == torch::kInt32 && pos0->is_contiguous() && pos0->numel() == block_table.size(0), "pos0: int32, one entry per sequence");
        p.pos0 = i32_ptr(*pos0);
    }
    p.status = status_ptr(status);
    SKY_CUDA_CHECK(launch_prefill_attn_tc(p, pool_rows, cur_stream()));
}

// ---- memhog ----
static void memhog(torch::Tensor a, torch::Tensor b, int op, int iters, uint64_t duration_ns, uint64_t duty_on_ns, uint64_t duty_off_ns,
                   uint64_t chunk_bytes, int ctas, int threads, uint64_t credit_dev_ptr, uint64_t consumed_base, uint64_t max_wait_ns,
                   float alpha, torch::Tensor sink, torch::Tensor status) {
    TORCH_CHECK(a.is_cuda() && a.is_contiguous() && a.numel() * a.element_size() % 16 == 0, "a: contiguous CUDA tensor, multiple of 16 bytes");
    c10::cuda::CUDAGuard g(a.device());
    MemhogParams p;
    memset(&p, 0, sizeof p);
    p.a = (float4*)a.data_ptr();
    p.b = b.defined() && b.numel() ? (float4*)b.data_ptr() : nullptr;
    p.n_vec = (uint64_t)(a.numel() * a.element_size() / 16);
    TORCH_CHECK(op == MEMHOG_READ || (p.b && (uint64_t)(b.numel() * b.element_size() / 16) >= p.n_vec), "b too small for this op");
    p.op = op; p.iters = iters; p.duration_ns = duration_ns; p.duty_on_ns = duty_on_ns; p.duty_off_ns = duty_off_ns;
    p.chunk_vec = std::max<uint64_t>(1, chunk_bytes / 16);
    p.page = (const SkyCreditPage*)credit_dev_ptr; p.usage = (SkyCreditPage*)credit_dev_ptr;
    p.consumed_base = consumed_base; p.max_wait_ns = max_wait_ns; p.alpha = alpha;
    p.sink = sink.defined() && sink.numel() ? sink.data_ptr<double>() : nullptr;
    p.status = status_ptr(status);
    SKY_CUDA_CHECK(launch_memhog(p, ctas, threads, cur_stream()));
}

// ---- paged attention ----
static void paged_attn_decode(torch::Tensor q, torch::Tensor kv_layer, torch::Tensor out, torch::Tensor block_table, torch::Tensor ctx_lens,
                              int64_t block_stride, int64_t kv_stride, int64_t head_stride, int kv_heads, int max_ctx, int chunk_tokens,
                              double scale, torch::Tensor part_o, torch::Tensor part_m, torch::Tensor part_l, torch::Tensor counters,
                              torch::Tensor status, int64_t pool_rows, int64_t num_blocks) {
    c10::cuda::CUDAGuard g(q.device());
    TORCH_CHECK(block_table.dim() == 2 && (int64_t)max_ctx <= block_table.size(1) * 16, "max_ctx = ", max_ctx, " but a block-table row covers ",
                block_table.size(1) * 16, " tokens");
    TORCH_CHECK(num_blocks >= 0 && num_blocks <= 0x7fffffffLL, "num_blocks out of range");
    TORCH_CHECK(q.dim() == 3 && q.is_contiguous() && out.is_contiguous(), "q/out: contiguous [batch][heads][128]");
    PagedAttnParams p;
    memset(&p, 0, sizeof p);
    p.q = bf16_ptr(q); p.kv = bf16_ptr(kv_layer); p.out = bf16_mut(out);
    p.block_table = i32_ptr(block_table); p.ctx_lens = i32_ptr(ctx_lens);
    p.block_stride = block_stride; p.kv_stride = kv_stride; p.head_stride = head_stride;
    p.batch = (int)q.size(0); p.q_heads = (int)q.size(1); p.kv_heads = kv_heads; p.head_dim = (int)q.size(2);
    p.block_tokens = 16; p.max_blocks = (int)block_table.size(1); p.num_blocks = (int)num_blocks;
    p.max_ctx = max_ctx; p.chunk_tokens = chunk_tokens; p.scale = (float)scale;
    p.max_splits = (int)part_m.size(2);
    TORCH_CHECK(part_o.scalar_type() == torch::kFloat32 && part_o.numel() >= (int64_t)p.batch * p.q_heads * p.max_splits * 128, "part_o too small");
    TORCH_CHECK(counters.numel() >= (int64_t)p.batch * kv_heads, "counters too small");
    p.part_o = part_o.data_ptr<float>(); p.part_m = part_m.data_ptr<float>(); p.part_l = part_l.data_ptr<float>();
    p.counters = reinterpret_cast<unsigned int*>(counters.data_ptr());
    p.status = status_ptr(status);
    if (pool_rows > 0) SKY_CUDA_CHECK(launch_paged_attn_decode_tc(p, pool_rows, cur_stream()));
    else SKY_CUDA_CHECK(launch_paged_attn_decode(p, cur_stream()));
}

// ---- small ops ----
static void rmsnorm(torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor w, torch::Tensor y, double eps) {
    c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.is_contiguous() && y.is_contiguous(), "contiguous");
    const int hidden = (int)x.size(-1), rows = (int)(x.numel() / hidden);
    __nv_bfloat16* res = residual.has_value() ? bf16_mut(*residual) : nullptr;
    SKY_CUDA_CHECK(launch_rmsnorm(bf16_ptr(x), res, bf16_ptr(w), bf16_mut(y), rows, hidden, (float)eps, cur_stream()));
}
static void rope_append(torch::Tensor qkv, c10::optional<torch::Tensor> q_norm, c10::optional<torch::Tensor> k_norm, torch::Tensor q_out,
                        torch::Tensor kv_layer, torch::Tensor inv_freq, torch::Tensor block_table, torch::Tensor positions,
                        c10::optional<torch::Tensor> seq_ids, int64_t block_stride, int64_t kv_stride, int64_t head_stride, int64_t tok_stride, int q_heads,
                        int kv_heads, double eps) {
    c10::cuda::CUDAGuard g(qkv.device());
    RopeAppendParams p;
    memset(&p, 0, sizeof p);
    p.qkv = bf16_ptr(qkv);
    p.q_norm = q_norm.has_value() ? bf16_ptr(*q_norm) : nullptr;
    p.k_norm = k_norm.has_value() ? bf16_ptr(*k_norm) : nullptr;
    p.q_out = bf16_mut(q_out); p.kv = bf16_mut(kv_layer);
    TORCH_CHECK(inv_freq.scalar_type() == torch::kFloat32 && inv_freq.numel() == 64, "inv_freq: 64 floats");
    p.inv_freq = inv_freq.data_ptr<float>();
    p.block_table = i32_ptr(block_table); p.positions = i32_ptr(positions);
    p.seq_ids = seq_ids.has_value() ? i32_ptr(*seq_ids) : nullptr;
    p.block_stride = block_stride; p.kv_stride = kv_stride; p.head_stride = head_stride; p.tok_stride = tok_stride;
    p.tokens = (int)positions.numel(); p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.max_blocks = (int)block_table.size(1); p.block_tokens = 16; p.eps = (float)eps;
    TORCH_CHECK(qkv.numel() == (int64_t)p.tokens * (q_heads + 2 * kv_heads) * 128, "qkv shape");
    SKY_CUDA_CHECK(launch_rope_append(p, cur_stream()));
}
static void silu_mul(torch::Tensor gate_up, torch::Tensor out) {
    c10::cuda::CUDAGuard g(gate_up.device());
    const int ffn = (int)out.size(-1), rows = (int)(out.numel() / ffn);
    SKY_CUDA_CHECK(launch_silu_mul(bf16_ptr(gate_up), bf16_mut(out), rows, ffn, cur_stream()));
}
static void embedding(torch::Tensor ids, torch::Tensor table, torch::Tensor out) {
    c10::cuda::CUDAGuard g(table.device());
    SKY_CUDA_CHECK(launch_embedding(i32_ptr(ids), bf16_ptr(table), bf16_mut(out), (int)ids.numel(), (int)table.size(1), (int)table.size(0), cur_stream()));
}
static void argmax(torch::Tensor logits, torch::Tensor out) {
    c10::cuda::CUDAGuard g(logits.device());
    TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits: [rows][vocab]");
    SKY_CUDA_CHECK(launch_argmax(bf16_ptr(logits), out.data_ptr<int>(), (int)logits.size(0), (int)logits.size(1), logits.stride(0), cur_stream()));
}

static void sample(torch::Tensor logits, torch::Tensor out, double temperature, int64_t seed, c10::optional<torch::Tensor> positions) {
    c10::cuda::CUDAGuard g(logits.device());
    TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == torch::kBFloat16, "logits: bf16 [rows][vocab]");
    TORCH_CHECK(out.scalar_type() == torch::kInt32 && out.numel() >= logits.size(0), "out: int32, one entry per row");
    TORCH_CHECK(temperature > 0, "temperature must be positive (use argmax for greedy)");
    const int* pos = nullptr;
    if (positions.has_value()) {
        TORCH_CHECK(positions->scalar_type() == torch::kInt32 && positions->is_contiguous() && positions->numel() >= logits.size(0), "positions: int32, one per row");
        pos = positions->data_ptr<int>();
    }
    SKY_CUDA_CHECK(launch_sample(bf16_ptr(logits), out.data_ptr<int>(), (int)logits.size(0), (int)logits.size(1), logits.stride(0),
                                 (float)temperature, (unsigned int)seed, pos, cur_stream()));
}

// ---- GEMM ----
// ss_in / ss_out: fp32 vectors of at least M entries (see GemmNormFuse); residual: y is the residual stream, updated in place.
static void gemm(torch::Tensor x, torch::Tensor w, torch::Tensor y, int splits, bool gated, c10::optional<torch::Tensor> workspace,
                 c10::optional<torch::Tensor> counters, torch::Tensor status, int ntok, int persistent, bool cluster_split) {
    c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1, "row-major 2-D tensors");
    GemmParams p{};
    memset(&p, 0, sizeof p);
    p.x = bf16_ptr(x); p.w = bf16_ptr(w); p.y = bf16_mut(y);
    p.M = (int)x.size(0); p.K = (int)x.size(1);
    p.N = gated ? (int)w.size(0) / 2 : (int)w.size(0);
    TORCH_CHECK(w.size(1) == p.K && y.size(0) == p.M && y.size(1) == p.N, "shape mismatch");
    p.ldx = x.stride(0); p.ldw = w.stride(0); p.ldy = y.stride(0);
    p.splits = splits; p.gated = gated; p.ntok = ntok; p.cluster_split = cluster_split ? 1 : 0;
    if (splits > 1 && !cluster_split) {
        TORCH_CHECK(workspace.has_value() && counters.has_value(), "split-K needs workspace and counters");
        TORCH_CHECK((size_t)workspace->numel() >= gemm_workspace_floats(p.M, p.N, splits, gated, ntok), "workspace too small");
        TORCH_CHECK((size_t)counters->numel() >= gemm_counter_count(p.M, p.N, gated, ntok), "counters too small");
        p.workspace = workspace->data_ptr<float>();
        p.counters = reinterpret_cast<unsigned int*>(counters->data_ptr());
    }
    p.status = status_ptr(status);
    TORCH_CHECK(!persistent || splits == 1, "the persistent form is the plain projection without split-K");
    p.persistent = persistent;          // 0: one tile per CTA, 1: persistent with 128-row tiles, 2: persistent with 256 x 256 tiles
    SKY_CUDA_CHECK(launch_gemm(p, cur_stream()));
}

// ---- tensor-parallel fused paths ----
static TpSeq make_seq(uint64_t step_ptr, unsigned uses_per_step, unsigned use_index, unsigned arrivals) {
    TpSeq s;
    s.step = (const unsigned int*)step_ptr; s.uses_per_step = uses_per_step; s.use_index = use_index; s.arrivals_per_use = arrivals;
    return s;
}

// ag = (n_src, counters_ptr, step_ptr, uses_per_step, use_index, arrivals_per_use, timeout_ns) or empty
// rs = (world, src_rank, rows_per_rank, [dst ptrs], [counter ptrs]) or empty
static void gemm_tp(torch::Tensor x, torch::Tensor w, torch::Tensor y, int splits, bool gated, c10::optional<torch::Tensor> workspace,
                    c10::optional<torch::Tensor> counters, torch::Tensor status, py::tuple ag, py::tuple rs, int ntok, bool cluster_split) {
    c10::cuda::CUDAGuard g(x.device());
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "row-major 2-D tensors");
    GemmParams p{};
    memset(&p, 0, sizeof p);
    p.x = bf16_ptr(x); p.w = bf16_ptr(w);
    p.M = (int)x.size(0); p.K = (int)x.size(1);
    p.N = gated ? (int)w.size(0) / 2 : (int)w.size(0);
    TORCH_CHECK(w.size(1) == p.K, "shape mismatch");
    p.ldx = x.stride(0); p.ldw = w.stride(0);
    if (rs.size() == 0) {
        TORCH_CHECK(y.dim() == 2 && y.size(0) == p.M && y.size(1) == p.N && y.stride(1) == 1, "y shape");
        p.y = bf16_mut(y); p.ldy = y.stride(0);
    }
    p.splits = splits; p.gated = gated; p.ntok = ntok; p.cluster_split = cluster_split ? 1 : 0;
    if (splits > 1 && !cluster_split) {
        TORCH_CHECK(workspace.has_value() && counters.has_value(), "split-K needs workspace and counters");
        TORCH_CHECK((size_t)workspace->numel() >= gemm_workspace_floats(p.M, p.N, splits, gated, ntok), "workspace too small");
        TORCH_CHECK((size_t)counters->numel() >= gemm_counter_count(p.M, p.N, gated, ntok), "counters too small");
        p.workspace = workspace->data_ptr<float>();
        p.counters = reinterpret_cast<unsigned int*>(counters->data_ptr());
    }
    p.status = status_ptr(status);
    if (ag.size() > 0) {
        p.ag.n_src = ag[0].cast<int>();
        p.ag.counters = (const unsigned int*)ag[1].cast<uint64_t>();
        p.ag.seq = make_seq(ag[2].cast<uint64_t>(), ag[3].cast<unsigned>(), ag[4].cast<unsigned>(), ag[5].cast<unsigned>());
        p.ag.timeout_ns = ag[6].cast<uint64_t>();
    }
    if (rs.size() > 0) {
        p.rs.world = rs[0].cast<int>(); p.rs.src_rank = rs[1].cast<int>(); p.rs.rows_per_rank = rs[2].cast<int>();
        p.rs.all = rs.size() > 5 && rs[5].cast<bool>() ? 1 : 0;
        auto dst = rs[3].cast<std::vector<uint64_t>>();
        auto ctr = rs[4].cast<std::vector<uint64_t>>();
        TORCH_CHECK((int)dst.size() == p.rs.world && (int)ctr.size() == p.rs.world && p.rs.world <= TP_MAX_RANKS, "rs pointer lists");
        TORCH_CHECK(p.M <= (p.rs.all ? 1 : p.rs.world) * p.rs.rows_per_rank, "more token rows than the receive buffers hold");
        for (int i = 0; i < p.rs.world; ++i) { p.rs.dst[i] = (__nv_bfloat16*)dst[i]; p.rs.counters[i] = (unsigned int*)ctr[i]; }
    }
    SKY_CUDA_CHECK(launch_gemm(p, cur_stream()));
}

static void tp_norm(uint64_t rs_buf, uint64_t rs_counter, py::tuple rs_seq, torch::Tensor resid, torch::Tensor w,
                    std::vector<uint64_t> ag_dst, std::vector<uint64_t> ag_counter, int rank, double eps, uint64_t timeout_ns,
                    torch::Tensor status, int rs_world) {
    c10::cuda::CUDAGuard g(resid.device());
    TpNormParams p;
    memset(&p, 0, sizeof p);
    p.rs_buf = (const __nv_bfloat16*)rs_buf;
    p.rs_counter = (const unsigned int*)rs_counter;
    if (rs_buf) p.rs_seq = make_seq(rs_seq[0].cast<uint64_t>(), rs_seq[1].cast<unsigned>(), rs_seq[2].cast<unsigned>(), rs_seq[3].cast<unsigned>());
    p.resid = bf16_mut(resid); p.w = bf16_ptr(w);
    // rs_world = 0: reduce-scatter / all-gather form (as many partials as all-gather destinations, rows offset by the rank);
    // rs_world > 0: one-shot all-reduce form (rs_world full-size partials, the normed rows go to ag_dst as they are).
    p.ag_n = (int)ag_dst.size();
    p.world = rs_world > 0 ? rs_world : p.ag_n;
    p.rank = rank; p.rows = (int)resid.size(0); p.hidden = (int)resid.size(1);
    p.ag_row0 = rs_world > 0 ? 0 : rank * p.rows;
    TORCH_CHECK(p.world >= 1 && p.world <= TP_MAX_RANKS && p.ag_n >= 1 && p.ag_n <= TP_MAX_RANKS && ag_counter.size() == ag_dst.size(), "peer lists");
    for (int i = 0; i < p.ag_n; ++i) { p.ag_dst[i] = (__nv_bfloat16*)ag_dst[i]; p.ag_counter[i] = (unsigned int*)ag_counter[i]; }
    p.eps = (float)eps; p.timeout_ns = timeout_ns; p.status = status_ptr(status);
    SKY_CUDA_CHECK(launch_tp_norm(p, cur_stream()));
}

static void tp_argmax(torch::Tensor logits, int vocab_lo, int rank, std::vector<uint64_t> slots, std::vector<uint64_t> counters,
                      uint64_t my_slots, uint64_t my_counters, py::tuple seq, torch::Tensor next_ids, uint64_t timeout_ns,
                      torch::Tensor status) {
    c10::cuda::CUDAGuard g(logits.device());
    TpArgmaxParams p;
    memset(&p, 0, sizeof p);
    p.logits = bf16_ptr(logits); p.row_stride = logits.stride(0);
    p.rows = (int)logits.size(0); p.vocab_local = (int)logits.size(1); p.vocab_lo = vocab_lo;
    p.world = (int)slots.size(); p.rank = rank;
    TORCH_CHECK(p.world >= 1 && p.world <= TP_MAX_RANKS && counters.size() == slots.size(), "peer lists");
    for (int i = 0; i < p.world; ++i) { p.slots[i] = (unsigned long long*)slots[i]; p.counters[i] = (unsigned int*)counters[i]; }
    p.my_slots = (const unsigned long long*)my_slots; p.my_counters = (const unsigned int*)my_counters;
    p.seq = make_seq(seq[0].cast<uint64_t>(), seq[1].cast<unsigned>(), seq[2].cast<unsigned>(), seq[3].cast<unsigned>());
    p.next_ids = next_ids.data_ptr<int>(); p.timeout_ns = timeout_ns; p.status = status_ptr(status);
    SKY_CUDA_CHECK(launch_tp_argmax(p, cur_stream()));
}
static void step_increment(torch::Tensor step) {
    c10::cuda::CUDAGuard g(step.device());
    SKY_CUDA_CHECK(launch_step_increment(reinterpret_cast<unsigned int*>(step.data_ptr()), cur_stream()));
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "SkyGDR-B200 sm_100a kernels";
    m.def("new_status", &new_status);
    m.def("reset_status", &reset_status);
    m.def("read_status", &read_status);
    m.def("host_alloc_mapped", &host_alloc_mapped);
    m.def("host_free_mapped", &host_free_mapped);
    m.def("host_register", &host_register);
    m.def("host_unregister", &host_unregister);
    m.def("credit_page_init", &credit_page_init);
    m.def("paged_attn_tc_page_box", &sky::paged_attn_tc_page_box);
    m.def("credit_page_grant", &credit_page_grant);
    m.def("credit_page_read", &credit_page_read);
    m.def("credit_page_heartbeat", &credit_page_heartbeat);
    m.def("ipc_alloc", &ipc_alloc);
    m.def("ipc_open", &ipc_open);
    m.def("ipc_close", &ipc_close);
    m.def("ipc_free", &ipc_free);
    m.def("tensor_from_ptr", &tensor_from_ptr);
    m.def("enable_peer_access", &enable_peer_access);
    m.def("peer_store_probe", &peer_store_probe, py::arg("device"), py::arg("dst_ptr"), py::arg("total_bytes"), py::arg("mode"),
          py::arg("store_bytes") = 32768, py::arg("inflight") = 4, py::arg("ctas") = 148, py::arg("iters") = 1,
          py::call_guard<py::gil_scoped_release>());
    m.def("kv_transfer", &kv_transfer, py::call_guard<py::gil_scoped_release>(), py::arg("src_pool"), py::arg("dst_ptrs"),
          py::arg("dst_scale_ptrs"), py::arg("done_flag_ptrs"), py::arg("src_blocks"), py::arg("dst_blocks"), py::arg("layers"),
          py::arg("heads"), py::arg("block_tokens"), py::arg("head_dim"), py::arg("src_strides"), py::arg("dst_strides"),
          py::arg("heads_per_dst"), py::arg("replicate"), py::arg("fp8"), py::arg("keep_layout"), py::arg("pages_per_chunk"),
          py::arg("ctas"), py::arg("credit_dev_ptr"), py::arg("consumed_base"), py::arg("max_wait_ns"), py::arg("first_chunk"),
          py::arg("done_value"), py::arg("status"), py::arg("use_tma"), py::arg("multicast_ptr") = 0,
          py::arg("src_num_blocks") = 0, py::arg("dst_num_blocks") = 0);
    m.def("multicast_supported", [](int device) {
        std::string why;
        bool ok = multicast_supported(device, &why);
        return std::make_pair(ok, why);
    });
    py::class_<MulticastRegion>(m, "MulticastRegion")
        .def_readonly("devices", &MulticastRegion::devices)
        .def_readonly("bytes", &MulticastRegion::bytes)
        .def_readonly("granularity", &MulticastRegion::granularity)
        .def_readonly("unicast", &MulticastRegion::unicast)
        .def_readonly("multicast", &MulticastRegion::multicast);
    m.def("multicast_create", [](std::vector<int> devices, uint64_t bytes) {
        try {
            return multicast_create(devices, (size_t)bytes);
        } catch (const std::exception& e) { TORCH_CHECK(false, e.what()); }
    }, py::return_value_policy::reference);
    m.def("multicast_destroy", [](MulticastRegion* r) { multicast_destroy(r); });
    m.def("memhog", &memhog, py::call_guard<py::gil_scoped_release>());
    m.def("paged_attn_decode", &paged_attn_decode, py::arg("q"), py::arg("kv_layer"), py::arg("out"), py::arg("block_table"), py::arg("ctx_lens"),
          py::arg("block_stride"), py::arg("kv_stride"), py::arg("head_stride"), py::arg("kv_heads"), py::arg("max_ctx"), py::arg("chunk_tokens"),
          py::arg("scale"), py::arg("part_o"), py::arg("part_m"), py::arg("part_l"), py::arg("counters"), py::arg("status"), py::arg("pool_rows"),
          py::arg("num_blocks") = 0);
    m.def("prefill_attn", &prefill_attn, py::arg("q"), py::arg("kv_layer"), py::arg("out"), py::arg("block_table"), py::arg("seq_start"),
          py::arg("block_stride"), py::arg("kv_stride"), py::arg("head_stride"), py::arg("tok_stride"), py::arg("kv_heads"), py::arg("max_len"),
          py::arg("scale"), py::arg("status"), py::arg("pool_rows"), py::arg("pos0") = py::none());
    m.def("rmsnorm", &rmsnorm);
    m.def("rope_append", &rope_append);
    m.def("silu_mul", &silu_mul);
    m.def("embedding", &embedding);
    m.def("argmax", &argmax);
    m.def("sample", &sample, py::arg("logits"), py::arg("out"), py::arg("temperature"), py::arg("seed"), py::arg("positions") = py::none());
    m.def("gemm", &gemm, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("splits"), py::arg("gated"), py::arg("workspace"), py::arg("counters"),
          py::arg("status"), py::arg("ntok"), py::arg("persistent") = 0, py::arg("cluster_split") = false);
    m.def("gemm_tp", &gemm_tp, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("splits"), py::arg("gated"), py::arg("workspace"), py::arg("counters"),
          py::arg("status"), py::arg("ag"), py::arg("rs"), py::arg("ntok"), py::arg("cluster_split") = false);
    m.def("tp_norm", &tp_norm, py::arg("rs_buf"), py::arg("rs_counter"), py::arg("rs_seq"), py::arg("resid"), py::arg("w"), py::arg("ag_dst"),
          py::arg("ag_counter"), py::arg("rank"), py::arg("eps"), py::arg("timeout_ns"), py::arg("status"), py::arg("rs_world") = 0);
    m.def("tp_argmax", &tp_argmax);
    m.def("step_increment", &step_increment);
    m.def("gemm_workspace_floats", &gemm_workspace_floats, py::arg("M"), py::arg("N"), py::arg("splits"), py::arg("gated"), py::arg("ntok") = 0);
    m.def("gemm_counter_count", &gemm_counter_count, py::arg("M"), py::arg("N"), py::arg("gated"), py::arg("ntok") = 0);
    m.def("gemm_pick_ntok", &gemm_pick_ntok);
    m.attr("STATUS_BYTES") = py::int_(sizeof(LaunchStatus));

    py::class_<PcieTaskConfig>(m, "PcieTaskConfig")
        .def(py::init<>())
        .def_readwrite("device", &PcieTaskConfig::device)
        .def_readwrite("h2d", &PcieTaskConfig::h2d)
        .def_readwrite("chunk_bytes", &PcieTaskConfig::chunk_bytes)
        .def_readwrite("streams", &PcieTaskConfig::streams)
        .def_readwrite("batch", &PcieTaskConfig::batch)
        .def_readwrite("inflight", &PcieTaskConfig::inflight)
        .def_readwrite("pinned", &PcieTaskConfig::pinned)
        .def_readwrite("low_priority", &PcieTaskConfig::low_priority)
        .def_readwrite("seconds", &PcieTaskConfig::seconds)
        .def_readwrite("total_bytes", &PcieTaskConfig::total_bytes)
        .def_readwrite("max_outstanding_bytes", &PcieTaskConfig::max_outstanding_bytes)
        .def_readwrite("progress_ms", &PcieTaskConfig::progress_ms)
        .def_readwrite("smooth_windows", &PcieTaskConfig::smooth_windows)
        .def_readwrite("duty_on_ms", &PcieTaskConfig::duty_on_ms)
        .def_readwrite("duty_off_ms", &PcieTaskConfig::duty_off_ms)
        .def_readwrite("consumed_base", &PcieTaskConfig::consumed_base)
        .def_readwrite("min_issue_bytes", &PcieTaskConfig::min_issue_bytes)
        .def_readwrite("external_bytes", &PcieTaskConfig::external_bytes)
        .def("set_credit_page", [](PcieTaskConfig& c, uint64_t host_ptr) { c.credit_page = (SkyCreditPage*)host_ptr; })
        .def("set_external", [](PcieTaskConfig& c, uint64_t host_ptr, uint64_t dev_ptr, uint64_t bytes) {
            c.external_host = (void*)host_ptr; c.external_dev = (void*)dev_ptr; c.external_bytes = bytes;
        });
    py::class_<PcieProgress>(m, "PcieProgress")
        .def_readonly("ts_unix_ms", &PcieProgress::ts_unix_ms)
        .def_readonly("elapsed_ms", &PcieProgress::elapsed_ms)
        .def_readonly("issued_bytes", &PcieProgress::issued_bytes)
        .def_readonly("completed_bytes", &PcieProgress::completed_bytes)
        .def_readonly("remaining_bytes", &PcieProgress::remaining_bytes)
        .def_readonly("window_bytes", &PcieProgress::window_bytes)
        .def_readonly("inst_bw_gib_s", &PcieProgress::inst_bw_gib_s)
        .def_readonly("smooth_bw_gib_s", &PcieProgress::smooth_bw_gib_s)
        .def_readonly("avg_bw_gib_s", &PcieProgress::avg_bw_gib_s)
        .def_readonly("done", &PcieProgress::done)
        .def("csv", [](const PcieProgress& p) { return PcieTask::csv_row(p); });
    py::class_<PcieTask>(m, "PcieTask")
        .def(py::init<const PcieTaskConfig&>())
        .def("setup", &PcieTask::setup, py::call_guard<py::gil_scoped_release>())
        .def("start", &PcieTask::start, py::call_guard<py::gil_scoped_release>())
        .def("stop", &PcieTask::stop)
        .def("join", &PcieTask::join, py::call_guard<py::gil_scoped_release>())
        .def_property_readonly("running", &PcieTask::running)
        .def("progress", &PcieTask::progress)
        .def("rows", &PcieTask::rows)
        .def("error", &PcieTask::error)
        .def("stdout_line", &PcieTask::stdout_line)
        .def_static("csv_header", [] { return std::string(PcieTask::csv_header()); });

}
