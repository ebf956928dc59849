// Line protocol of a flow end-point and of the daemon.
//
// The legacy subset is the reference's control port: one text command per
// connection, `HIGH | LOW | LOW1..LOW4 | SLEEP <us> | STOP | STATUS`, answered
// by one state line (src/cpu_client.cc:158-236). The reply format and the
// counting rule (`commands` counts mode changes and STOP, not STATUS) are kept
// so that the reference's tools (src/tools/cpu_client_control.py,
// src/tools/pcie_case_study_controller.py:82-99) can talk to an end-point of
// this runtime unchanged.
//
// The extension adds flow registration with goals, which the reference only
// describes (README.md:34-54):
//   REGISTER <name> <priority:high|normal|low|besteffort|int> <target_gbps> [kind]
//   RENEW <flow_id> | UNREGISTER <flow_id> | BUDGET <flow_id> | FLOWS
//   FLOW <flow_id> <legacy command>      (address one flow of a daemon)
//   POLICY <name> | WINDOW <us>
#pragma once
#include <atomic>
#include <cstdio>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "credit_page.h"
#include "util.hpp"

namespace skygdr {

inline const char* mode_name(int mode) {
    static const char* names[] = {"DISABLED", "HIGH", "LOW1", "LOW2", "LOW3", "LOW4", "CUSTOM"};
    return (mode >= 0 && mode <= 6) ? names[mode] : "DISABLED";
}

inline int mode_from_name(const std::string& s) {
    if (s == "HIGH") return SKY_MODE_HIGH;
    if (s == "LOW" || s == "LOW1") return SKY_MODE_LOW1;
    if (s == "LOW2") return SKY_MODE_LOW2;
    if (s == "LOW3") return SKY_MODE_LOW3;
    if (s == "LOW4") return SKY_MODE_LOW4;
    if (s == "CUSTOM") return SKY_MODE_CUSTOM;
    if (s == "DISABLED") return SKY_MODE_DISABLED;
    return -1;
}

// Pacing state of one flow end-point. Readers are data loops on other
// threads; independent scalars, so relaxed atomics suffice.
class ControlState {
public:
    // Sleep presets in microseconds, index = SkyMode (HIGH..LOW4 used).
    // LOW2/3/4 default to 1.25x/1.5x/1.75x LOW1 when not given
    // (src/cpu_client.cc:536-542).
    void configure(uint32_t high_us, uint32_t low1_us, int64_t low2_us = -1, int64_t low3_us = -1,
                   int64_t low4_us = -1) {
        preset_[SKY_MODE_HIGH] = high_us;
        preset_[SKY_MODE_LOW1] = low1_us;
        preset_[SKY_MODE_LOW2] = low2_us >= 0 ? (uint32_t)low2_us : (uint32_t)(low1_us * 1.25);
        preset_[SKY_MODE_LOW3] = low3_us >= 0 ? (uint32_t)low3_us : (uint32_t)(low1_us * 1.5);
        preset_[SKY_MODE_LOW4] = low4_us >= 0 ? (uint32_t)low4_us : (uint32_t)(low1_us * 1.75);
    }
    // A control-enabled end-point starts in HIGH (src/cpu_client.cc:544-545).
    void enable() { mode_.store(SKY_MODE_HIGH); sleep_us_.store(preset_[SKY_MODE_HIGH]); }

    int mode() const { return mode_.load(std::memory_order_relaxed); }
    uint32_t sleep_us() const { return sleep_us_.load(std::memory_order_relaxed); }
    uint32_t preset(int m) const { return preset_[m]; }
    uint64_t commands() const { return commands_.load(std::memory_order_relaxed); }
    bool stop_requested() const { return stop_.load(std::memory_order_relaxed) != 0; }
    void clear_stop() { stop_.store(0); }

    void apply(int mode, uint32_t sleep_us) {
        mode_.store(mode, std::memory_order_relaxed);
        sleep_us_.store(sleep_us, std::memory_order_relaxed);
        commands_.fetch_add(1, std::memory_order_relaxed);
        if (on_change) on_change(mode, sleep_us);
    }

    std::string status_line(const char* prefix) const {
        char buf[320];
        snprintf(buf, sizeof buf,
                 "%s mode=%s sleep_us=%u high_sleep_us=%u low1_sleep_us=%u low2_sleep_us=%u "
                 "low3_sleep_us=%u low4_sleep_us=%u commands=%lu stop=%d\n",
                 prefix, mode_name(mode()), sleep_us(), preset_[SKY_MODE_HIGH], preset_[SKY_MODE_LOW1],
                 preset_[SKY_MODE_LOW2], preset_[SKY_MODE_LOW3], preset_[SKY_MODE_LOW4],
                 (unsigned long)commands(), stop_requested() ? 1 : 0);
        return buf;
    }

    // Executes one legacy command and returns the reply line.
    std::string handle(const std::string& raw) {
        std::string cmd = trim(raw);
        if (cmd.empty()) return status_line("ERR empty");
        if (cmd == "STATUS") return status_line("OK");
        if (cmd == "STOP") {
            stop_.store(1, std::memory_order_relaxed);
            commands_.fetch_add(1, std::memory_order_relaxed);
            if (on_stop) on_stop();
            return status_line("OK");
        }
        if (cmd.compare(0, 6, "SLEEP ") == 0) {
            unsigned long us = strtoul(cmd.c_str() + 6, nullptr, 10);
            apply(SKY_MODE_CUSTOM, (uint32_t)us);
            return status_line("OK");
        }
        int m = mode_from_name(cmd);
        if (m >= SKY_MODE_HIGH && m <= SKY_MODE_LOW4) {
            apply(m, preset_[m]);
            return status_line("OK");
        }
        return status_line("ERR unknown_cmd");
    }

    std::function<void(int, uint32_t)> on_change;  // hook: mirror into a credit page
    std::function<void()> on_stop;

private:
    std::atomic<int> mode_{SKY_MODE_DISABLED};
    std::atomic<uint32_t> sleep_us_{0};
    std::atomic<uint64_t> commands_{0};
    std::atomic<int> stop_{0};
    uint32_t preset_[7] = {0, 0, 0, 0, 0, 0, 0};
};

// ---------------------------------------------------------------------------
// Flow registry with leases.

enum FlowKind { FLOW_KV_TRANSFER = 0, FLOW_KV_OFFLOAD = 1, FLOW_BEST_EFFORT = 2, FLOW_TP_COLLECTIVE = 3, FLOW_OTHER = 4 };

inline const char* kind_name(int k) {
    static const char* n[] = {"kv_transfer", "kv_offload", "best_effort", "tp_collective", "other"};
    return (k >= 0 && k <= 4) ? n[k] : "other";
}
inline int kind_from_name(const std::string& s) {
    for (int k = 0; k <= 4; ++k) if (s == kind_name(k)) return k;
    return FLOW_OTHER;
}

// Priority: larger = more important. Names map to fixed levels.
inline bool parse_priority(const std::string& s, int* out) {
    if (s == "high") { *out = 100; return true; }
    if (s == "normal") { *out = 50; return true; }
    if (s == "low") { *out = 10; return true; }
    if (s == "besteffort" || s == "best-effort" || s == "best_effort") { *out = 0; return true; }
    char* end = nullptr;
    long v = strtol(s.c_str(), &end, 10);
    if (end == s.c_str() || *end) return false;
    *out = (int)v;
    return true;
}

struct FlowInfo {
    uint32_t id = 0;
    std::string name;
    int priority = 0;
    double target_gbps = 0.0;   // decimal GB/s; 0 = best effort
    int kind = FLOW_OTHER;
    uint64_t lease_deadline_ns = 0;
    uint64_t registered_ns = 0;
    // Control state of the flow (mode ladder), and the budget the policy last gave it.
    int mode = SKY_MODE_HIGH;
    double budget_gbps = -1.0;  // <0 = unlimited
    bool stop = false;
    SkyCreditPage* page = nullptr;  // where grants are written (may be null in simulations)
    std::string page_path;          // shm name when the page is a /dev/shm file
};

class FlowRegistry {
public:
    explicit FlowRegistry(uint64_t lease_ns = 5'000'000'000ull) : lease_ns_(lease_ns) {}

    uint32_t add(const std::string& name, int prio, double target_gbps, int kind, uint64_t now_ns) {
        std::lock_guard<std::mutex> g(mu_);
        FlowInfo f;
        f.id = next_id_++;
        f.name = name;
        f.priority = prio;
        f.target_gbps = target_gbps;
        f.kind = kind;
        f.registered_ns = now_ns;
        f.lease_deadline_ns = now_ns + lease_ns_;
        flows_[f.id] = f;
        return f.id;
    }
    bool renew(uint32_t id, uint64_t now_ns) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = flows_.find(id);
        if (it == flows_.end()) return false;
        it->second.lease_deadline_ns = now_ns + lease_ns_;
        return true;
    }
    bool remove(uint32_t id) {
        std::lock_guard<std::mutex> g(mu_);
        return flows_.erase(id) > 0;
    }
    // Drops flows whose lease ran out; returns their ids.
    std::vector<uint32_t> expire(uint64_t now_ns) {
        std::lock_guard<std::mutex> g(mu_);
        std::vector<uint32_t> gone;
        for (auto it = flows_.begin(); it != flows_.end();) {
            if (it->second.lease_deadline_ns <= now_ns) { gone.push_back(it->first); it = flows_.erase(it); }
            else ++it;
        }
        return gone;
    }
    bool get(uint32_t id, FlowInfo* out) const {
        std::lock_guard<std::mutex> g(mu_);
        auto it = flows_.find(id);
        if (it == flows_.end()) return false;
        *out = it->second;
        return true;
    }
    bool update(uint32_t id, const std::function<void(FlowInfo&)>& fn) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = flows_.find(id);
        if (it == flows_.end()) return false;
        fn(it->second);
        return true;
    }
    std::vector<FlowInfo> snapshot() const {
        std::lock_guard<std::mutex> g(mu_);
        std::vector<FlowInfo> v;
        for (auto& kv : flows_) v.push_back(kv.second);
        return v;
    }
    size_t size() const { std::lock_guard<std::mutex> g(mu_); return flows_.size(); }
    uint64_t lease_ns() const { return lease_ns_; }
    // Restores a flow under its old id (daemon --restore).
    void restore(const FlowInfo& f) {
        std::lock_guard<std::mutex> g(mu_);
        flows_[f.id] = f;
        if (f.id >= next_id_) next_id_ = f.id + 1;
    }

private:
    mutable std::mutex mu_;
    std::map<uint32_t, FlowInfo> flows_;
    uint32_t next_id_ = 1;
    uint64_t lease_ns_;
};

}  // namespace skygdr
