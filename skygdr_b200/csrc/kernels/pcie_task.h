// Host<->device copy task (see pcie_task.cpp).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "credit_page.h"

namespace sky {

struct PcieTaskConfig {
    int device = 0;
    bool h2d = false;                    // default direction is device -> host
    uint64_t chunk_bytes = 128ull << 20;
    int streams = 8, batch = 8, inflight = 8;
    bool pinned = true;
    bool low_priority = true;
    double seconds = 0;                  // 0: no time limit
    uint64_t total_bytes = 0;            // 0: unbounded
    uint64_t max_outstanding_bytes = 0;  // 0: max(2*chunk*streams, 512 MiB)
    int progress_ms = 1000, smooth_windows = 5;
    int duty_on_ms = 0, duty_off_ms = 0;
    SkyCreditPage* credit_page = nullptr;  // host address of the flow's page; nullptr = ungated
    uint64_t consumed_base = 0;
    uint64_t min_issue_bytes = 8ull << 20; // under a credit gate, smallest copy worth issuing (except a final tail)
    // Optional caller-owned buffers walked through in chunk steps (kv_offload of a real pool).
    void* external_host = nullptr;
    void* external_dev = nullptr;
    uint64_t external_bytes = 0;
};

struct PcieProgress {
    uint64_t ts_unix_ms = 0;
    double elapsed_ms = 0;
    uint64_t issued_bytes = 0, completed_bytes = 0, remaining_bytes = 0, window_bytes = 0;
    double inst_bw_gib_s = 0, smooth_bw_gib_s = 0, avg_bw_gib_s = 0;
    int done = 0;
};

class PcieTask {
public:
    explicit PcieTask(const PcieTaskConfig& cfg);
    ~PcieTask();
    bool setup();          // allocates streams and buffers (done by start() if needed)
    bool start();          // spawns the worker thread
    void stop();           // asks the worker to drain and finish
    void join();
    bool running() const { return running_.load(); }
    PcieProgress progress() const;
    std::vector<PcieProgress> rows() const;
    std::string error() const;
    std::string stdout_line(const PcieProgress& p) const;
    static const char* csv_header();
    static std::string csv_row(const PcieProgress& p);
    const PcieTaskConfig& config() const { return cfg_; }

private:
    struct Pending { cudaEvent_t ev; uint64_t bytes; };
    struct Lane {
        cudaStream_t stream = nullptr;
        void* host = nullptr;
        void* dev = nullptr;
        std::deque<Pending> pending;
        std::vector<cudaEvent_t> free_events;
    };
    void run();
    void settle(Lane& ln, bool block_one);
    void release();
    bool fail(const char* what);

    PcieTaskConfig cfg_;
    std::vector<Lane> lanes_;
    std::thread worker_;
    std::atomic<bool> stop_{false}, running_{false};
    bool ready_ = false;
    uint64_t issued_ = 0, completed_ = 0;
    mutable std::mutex mu_;
    PcieProgress prog_;
    std::deque<PcieProgress> rows_;
    std::string error_;
};

}  // namespace sky
