// Host<->device copy task: chunked asynchronous copies on low-priority streams
// with a cap on outstanding bytes, an optional duty cycle, an optional credit
// gate, and progress reporting in the reference's formats.
//
// It is both the best-effort PCIe task and the async-copy variant of
// kv_offload. Reference: src/gpu_be_pcie_memcpy_task.cu (flags :53-72, default
// outstanding cap :191-196, issue loop :398-497, progress rows :336-396). The
// design differs: a worker thread owned by an object (so a Python driver can
// run it beside kernels), per-stream FIFOs of (event, bytes) instead of fixed
// event rings, copies that walk through the buffers instead of re-copying
// offset 0, and a byte budget read from a credit page instead of only a static
// outstanding cap.
#include "pcie_task.h"

#include <algorithm>
#include <chrono>
#include <cinttypes>
#include <cstring>
#include <thread>

namespace sky {

static uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
static uint64_t unix_ms_now() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

PcieTask::PcieTask(const PcieTaskConfig& cfg) : cfg_(cfg) {
    if (cfg_.streams < 1) cfg_.streams = 1;
    if (cfg_.batch < 1) cfg_.batch = 1;
    if (cfg_.inflight < 1) cfg_.inflight = 1;
    if (cfg_.max_outstanding_bytes == 0)
        cfg_.max_outstanding_bytes = std::max<uint64_t>(2ull * cfg_.chunk_bytes * cfg_.streams, 512ull << 20);
}

PcieTask::~PcieTask() { stop(); join(); release(); }

bool PcieTask::setup() {
    if (ready_) return true;
    if (cudaSetDevice(cfg_.device) != cudaSuccess) return fail("cudaSetDevice");
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);  // lo = lowest priority (largest number)
    lanes_.resize(cfg_.streams);
    for (auto& ln : lanes_) {
        if (cudaStreamCreateWithPriority(&ln.stream, cudaStreamNonBlocking, cfg_.low_priority ? lo : hi) != cudaSuccess)
            return fail("cudaStreamCreateWithPriority");
        if (cfg_.external_host) ln.host = nullptr;
        else if (cfg_.pinned) { if (cudaHostAlloc(&ln.host, cfg_.chunk_bytes, cudaHostAllocDefault) != cudaSuccess) return fail("cudaHostAlloc"); }
        else { ln.host = malloc(cfg_.chunk_bytes); if (!ln.host) return fail("malloc"); memset(ln.host, 0, cfg_.chunk_bytes); }
        if (!cfg_.external_dev && cudaMalloc(&ln.dev, cfg_.chunk_bytes) != cudaSuccess) return fail("cudaMalloc");
    }
    ready_ = true;
    return true;
}

void PcieTask::release() {
    for (auto& ln : lanes_) {
        for (auto& pe : ln.pending) cudaEventDestroy(pe.ev);
        ln.pending.clear();
        for (auto ev : ln.free_events) cudaEventDestroy(ev);
        ln.free_events.clear();
        if (ln.stream) cudaStreamDestroy(ln.stream);
        if (ln.host && !cfg_.external_host) { if (cfg_.pinned) cudaFreeHost(ln.host); else free(ln.host); }
        if (ln.dev && !cfg_.external_dev) cudaFree(ln.dev);
        ln = Lane();
    }
    lanes_.clear();
    ready_ = false;
}

bool PcieTask::fail(const char* what) {
    std::lock_guard<std::mutex> g(mu_);
    error_ = std::string(what) + ": " + cudaGetErrorString(cudaGetLastError());
    return false;
}

bool PcieTask::start() {
    if (running_.load()) return false;
    if (!setup()) return false;
    stop_.store(false);
    {
        std::lock_guard<std::mutex> g(mu_);
        prog_ = PcieProgress();
        rows_.clear();
    }
    running_.store(true);
    worker_ = std::thread([this] { run(); running_.store(false); });
    return true;
}

void PcieTask::stop() { stop_.store(true); }
void PcieTask::join() { if (worker_.joinable()) worker_.join(); }

void PcieTask::settle(Lane& ln, bool block_one) {
    while (!ln.pending.empty()) {
        auto& pe = ln.pending.front();
        cudaError_t q = block_one ? cudaEventSynchronize(pe.ev) : cudaEventQuery(pe.ev);
        block_one = false;
        if (q == cudaErrorNotReady) break;
        completed_ += pe.bytes;
        ln.free_events.push_back(pe.ev);
        ln.pending.pop_front();
    }
}

void PcieTask::run() {
    cudaSetDevice(cfg_.device);
    const uint64_t t0 = now_ns();
    uint64_t last_report = t0, last_bytes = 0;
    issued_ = completed_ = 0;
    std::deque<std::pair<double, double>> windows;  // (bytes, seconds)
    const bool duty = cfg_.duty_on_ms > 0 && cfg_.duty_off_ms > 0;
    SkyCreditPage* page = cfg_.credit_page;
    const uint64_t base = cfg_.consumed_base;
    size_t ext_off = 0;

    auto report = [&](bool final_row) {
        uint64_t now = now_ns();
        double dt = (now - last_report) * 1e-9;
        if (!final_row && dt * 1e3 < cfg_.progress_ms) return;
        double wbytes = double(completed_ - last_bytes);
        windows.emplace_back(wbytes, dt);
        while ((int)windows.size() > cfg_.smooth_windows) windows.pop_front();
        double sb = 0, ss = 0;
        for (auto& w : windows) { sb += w.first; ss += w.second; }
        PcieProgress pr;
        pr.ts_unix_ms = unix_ms_now();
        pr.elapsed_ms = (now - t0) * 1e-6;
        pr.issued_bytes = issued_;
        pr.completed_bytes = completed_;
        pr.remaining_bytes = cfg_.total_bytes > completed_ ? cfg_.total_bytes - completed_ : 0;
        pr.window_bytes = (uint64_t)wbytes;
        pr.inst_bw_gib_s = dt > 0 ? wbytes / dt / 1073741824.0 : 0;
        pr.smooth_bw_gib_s = ss > 0 ? sb / ss / 1073741824.0 : 0;
        pr.avg_bw_gib_s = pr.elapsed_ms > 0 ? double(completed_) / (pr.elapsed_ms * 1e-3) / 1073741824.0 : 0;
        pr.done = final_row ? 1 : 0;
        {
            std::lock_guard<std::mutex> g(mu_);
            prog_ = pr;
            rows_.push_back(pr);
            if (rows_.size() > 100000) rows_.pop_front();
        }
        if (page) {
            __atomic_store_n(&page->consumed_bytes, base + issued_, __ATOMIC_RELAXED);
            __atomic_store_n(&page->completed_bytes, base + completed_, __ATOMIC_RELEASE);
            __atomic_store_n(&page->backlog_bytes, pr.remaining_bytes, __ATOMIC_RELAXED);
        }
        last_report = now;
        last_bytes = completed_;
    };

    SkyHeartbeatWatch heartbeat = {0, 0, 0};
    while (!stop_.load()) {
        for (auto& ln : lanes_) settle(ln, false);
        uint64_t now = now_ns();
        double elapsed_s = (now - t0) * 1e-9;
        if (cfg_.seconds > 0 && elapsed_s >= cfg_.seconds) break;
        if (cfg_.total_bytes > 0 && completed_ >= cfg_.total_bytes) break;
        if (page && __atomic_load_n(&page->stop, __ATOMIC_RELAXED)) break;
        bool on = true;
        if (duty) {
            uint64_t period = (uint64_t)(cfg_.duty_on_ms + cfg_.duty_off_ms) * 1000000ull;
            uint64_t ph = (now - t0) % period;
            if (ph >= (uint64_t)cfg_.duty_on_ms * 1000000ull) {
                on = false;
                uint64_t left = period - ph;
                std::this_thread::sleep_for(std::chrono::nanoseconds(std::min<uint64_t>(left, 2000000ull)));
            }
        }
        bool issued_any = false;
        if (on) {
            for (auto& ln : lanes_) {
                if ((int)ln.pending.size() >= cfg_.inflight) continue;
                uint64_t batch_bytes = 0;
                for (int b = 0; b < cfg_.batch; ++b) {
                    uint64_t n = cfg_.chunk_bytes;
                    if (cfg_.total_bytes > 0) {
                        if (issued_ >= cfg_.total_bytes) break;
                        n = std::min<uint64_t>(n, cfg_.total_bytes - issued_);
                    }
                    uint64_t outstanding = issued_ - completed_;
                    if (outstanding >= cfg_.max_outstanding_bytes) break;
                    n = std::min<uint64_t>(n, cfg_.max_outstanding_bytes - outstanding);
                    if (page && !__atomic_load_n(&page->unlimited, __ATOMIC_RELAXED)) {
                        uint64_t granted = sky_host_allowance(page, &heartbeat, now);      // the grant, or the page's dead-control rule
                        if (granted == ~0ull) granted = base + issued_ + n;
                        uint64_t used = base + issued_;
                        if (granted <= used) break;
                        // Do not shred the flow into tiny copies when credit trickles in: wait for a worthwhile piece.
                        const uint64_t piece = std::min<uint64_t>(n, cfg_.min_issue_bytes);
                        if (granted - used < piece) break;
                        // A copy cut to the credit at hand keeps a size that is a multiple of 1 MiB, of 4 KiB under a smaller
                        // min_issue_bytes; the rest of the credit stays for the next copy.
                        if (granted - used < n) {                                   // (never the final tail: that one is not cut)
                            const uint64_t unit = piece >= (1ull << 20) ? (1ull << 20) : (piece >= 4096 ? 4096 : 1);
                            n = (granted - used) / unit * unit;
                        }
                    }
                    if (n == 0) break;
                    void* h = ln.host;
                    void* d = ln.dev;
                    if (cfg_.external_host) { h = (char*)cfg_.external_host + ext_off; }
                    if (cfg_.external_dev) { d = (char*)cfg_.external_dev + ext_off; }
                    if (cfg_.external_host || cfg_.external_dev) {
                        ext_off += n;
                        if (ext_off + cfg_.chunk_bytes > cfg_.external_bytes) ext_off = 0;
                    }
                    cudaError_t e = cfg_.h2d ? cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, ln.stream)
                                             : cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, ln.stream);
                    if (e != cudaSuccess) { fail("cudaMemcpyAsync"); stop_.store(true); break; }
                    batch_bytes += n;
                    issued_ += n;
                    if (page) __atomic_store_n(&page->consumed_bytes, base + issued_, __ATOMIC_RELAXED);   // the pacer's view of use
                }
                if (batch_bytes) {
                    cudaEvent_t ev;
                    if (!ln.free_events.empty()) { ev = ln.free_events.back(); ln.free_events.pop_back(); }
                    else cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
                    cudaEventRecord(ev, ln.stream);
                    ln.pending.push_back({ev, batch_bytes});
                    issued_any = true;
                }
            }
            if (!issued_any) {
                // Nothing could be issued: wait for the oldest copy, or nap if the gate is what holds us.
                bool waited = false;
                for (auto& ln : lanes_) if (!ln.pending.empty()) { settle(ln, true); waited = true; break; }
                if (!waited) std::this_thread::sleep_for(std::chrono::microseconds(200));
            }
        }
        report(false);
    }
    for (auto& ln : lanes_) { cudaStreamSynchronize(ln.stream); settle(ln, false); }
    report(true);
}

PcieProgress PcieTask::progress() const { std::lock_guard<std::mutex> g(mu_); return prog_; }
std::vector<PcieProgress> PcieTask::rows() const { std::lock_guard<std::mutex> g(mu_); return {rows_.begin(), rows_.end()}; }
std::string PcieTask::error() const { std::lock_guard<std::mutex> g(mu_); return error_; }

const char* PcieTask::csv_header() {
    return "ts_unix_ms,elapsed_ms,issued_bytes,completed_bytes,remaining_bytes,window_bytes,inst_bw_gib_s,smooth_bw_gib_s,avg_bw_gib_s,done";
}
std::string PcieTask::csv_row(const PcieProgress& p) {
    char b[320];
    snprintf(b, sizeof b, "%" PRIu64 ",%.3f,%" PRIu64 ",%" PRIu64 ",%" PRIu64 ",%" PRIu64 ",%.6f,%.6f,%.6f,%d", p.ts_unix_ms, p.elapsed_ms,
             p.issued_bytes, p.completed_bytes, p.remaining_bytes, p.window_bytes, p.inst_bw_gib_s, p.smooth_bw_gib_s, p.avg_bw_gib_s, p.done);
    return b;
}
std::string PcieTask::stdout_line(const PcieProgress& p) const {
    char b[512];
    snprintf(b, sizeof b,
             "[pcie] t=%.2fs dir=%s bw_gib_s=%.3f bytes=%" PRIu64 " streams=%d batch=%d inflight=%d chunk_bytes=%" PRIu64
             " pinned=%d issued_total=%" PRIu64 " completed_total=%" PRIu64 " remaining_bytes=%" PRIu64,
             p.elapsed_ms * 1e-3, cfg_.h2d ? "h2d" : "d2h", p.inst_bw_gib_s, p.window_bytes, cfg_.streams, cfg_.batch, cfg_.inflight,
             cfg_.chunk_bytes, cfg_.pinned ? 1 : 0, p.issued_bytes, p.completed_bytes, p.remaining_bytes);
    return b;
}

}  // namespace sky
