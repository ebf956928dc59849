// Core of the control daemon, free of sockets and threads so that tests can
// drive it with a fake clock: flow registry + per-window signal -> policy ->
// action step + credit-page writers + snapshot/restore.
//
// Reference counterpart: the loop of
// src/tools/pcie_case_study_controller.py:273-352, which polls CSV files every
// 100 ms and sends mode names to one end-point over TCP. Here a window is
// 1-10 ms, the signals are the usage halves of the flows' credit pages (and
// optional NVML link counters), and the action is a store of a byte grant into
// each page, which a kernel or copy worker reads directly.
#pragma once
#include <chrono>
#include <thread>
#include <atomic>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cinttypes>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>

#include "credit_page.h"
#include "policy.hpp"
#include "protocol.hpp"
#include "util.hpp"

namespace skygdr {

// Creates or opens a credit page backed by a file under /dev/shm, so that a GPU
// process can map it and page-lock it for device access.
inline SkyCreditPage* map_credit_page(const std::string& path, bool create) {
    int fd = open(path.c_str(), create ? (O_RDWR | O_CREAT) : O_RDWR, 0600);
    if (fd < 0) return nullptr;
    if (create && ftruncate(fd, 4096) != 0) { close(fd); return nullptr; }
    void* p = mmap(nullptr, 4096, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return nullptr;
    return reinterpret_cast<SkyCreditPage*>(p);
}
inline void unmap_credit_page(SkyCreditPage* p) { if (p) munmap(p, 4096); }

// A control side for ONE page without a daemon: a native thread that adds `rate` worth of bytes to the page's grant every
// window (with a burst allowance of a few windows for a flow that fell behind) and bumps the epoch, so that an in-process
// flow is paced without a Python thread (and its interpreter lock) in the loop.
class PagePacer {
public:
    PagePacer(SkyCreditPage* page, double rate_gbps, uint64_t window_ns, double burst_windows)
        : page_(page), rate_(rate_gbps), window_ns_(window_ns ? window_ns : 1000000), burst_(burst_windows) {}
    ~PagePacer() { stop(); }
    void start(uint64_t base) {
        stop();
        stop_.store(false);
        page_->unlimited = 0;
        page_->window_ns = window_ns_;
        page_->budget_per_window = (uint64_t)(rate_ * 1e9 * double(window_ns_) * 1e-9);
        __atomic_store_n(&page_->granted_bytes, base, __ATOMIC_RELEASE);
        __atomic_store_n(&page_->epoch, page_->epoch + 1, __ATOMIC_RELEASE);
        thread_ = std::thread([this, base] {
            double granted = double(base);
            uint64_t t_prev = mono_ns();
            while (!stop_.load(std::memory_order_relaxed)) {
                std::this_thread::sleep_for(std::chrono::nanoseconds(window_ns_));
                const uint64_t now = mono_ns();
                const double add = rate_ * double(now - t_prev);           // GB/s x ns = bytes
                t_prev = now;
                const double used = double(__atomic_load_n(&page_->consumed_bytes, __ATOMIC_RELAXED));
                granted = used < granted ? std::min(granted + add, std::max(granted, used + add * burst_)) : granted + add;
                __atomic_store_n(&page_->granted_bytes, (uint64_t)granted, __ATOMIC_RELEASE);
                __atomic_store_n(&page_->epoch, page_->epoch + 1, __ATOMIC_RELEASE);
                windows_.fetch_add(1, std::memory_order_relaxed);
            }
        });
    }
    void stop() {
        stop_.store(true);
        if (thread_.joinable()) thread_.join();
    }
    uint64_t windows() const { return windows_.load(); }

private:
    SkyCreditPage* page_;
    double rate_;
    uint64_t window_ns_;
    double burst_;
    std::atomic<bool> stop_{true};
    std::atomic<uint64_t> windows_{0};
    std::thread thread_;
};

struct DaemonConfig {
    double capacity_gbps = 64.0;          // capacity of the shared domain
    uint64_t window_ns = 5'000'000;       // control window
    uint64_t lease_ns = 5'000'000'000ull; // flow lease
    std::string policy = "target_track";
    PolicyConfig pcfg;
    std::string page_dir = "/dev/shm";    // "" = pages on the heap (tests, in-process use)
    std::string tag = "skygdr";
    int smooth_windows = 5;
    double burst_windows = 2.0;
    bool external_util = false;           // link utilisation is supplied (NVML) instead of summed from flows
    // Heartbeat contract written into every page: a data path that sees `epoch` unchanged for this many windows while it
    // waits for credit takes the daemon for dead and follows dead_policy (SkyDeadPolicy). 0 = no heartbeat check.
    uint32_t dead_after_windows = 0;
    uint32_t dead_policy = SKY_DEAD_STALL;
    double dead_fallback_gbps = 1.0;      // SKY_DEAD_STATIC: the rate a flow grants itself
};

class DaemonCore {
public:
    explicit DaemonCore(const DaemonConfig& cfg) : cfg_(cfg), reg_(cfg.lease_ns) {
        if (!make_policy(cfg_.policy, cfg_.pcfg)) cfg_.policy = "none";
        links_.push_back(Link{"default", cfg_.capacity_gbps, make_policy(cfg_.policy, cfg_.pcfg)});
    }
    ~DaemonCore() {
        for (auto& kv : state_) release_page(kv.second, /*at_exit=*/true);
    }

    struct WindowLog {
        uint64_t window_id; uint64_t ts_unix_ms; uint32_t flow_id; std::string flow; int mode; std::string decision;
        double budget_bytes; double inst_gbps, smooth_gbps; uint64_t backlog_bytes; double link_util_pct; uint64_t granted;
    };

    // ---- protocol ----
    std::string handle_line(const std::string& raw, uint64_t now_ns) {
        std::string line = trim(raw);
        if (line.empty()) return "ERR empty\n";
        auto tok = split_ws(line);
        const std::string& cmd = tok[0];
        char buf[512];
        if (cmd == "REGISTER") {
            if (tok.size() < 4) return "ERR usage REGISTER <name> <priority> <target_gbps> [kind] [link=<name>]\n";
            int prio;
            if (!parse_priority(tok[2], &prio)) return "ERR bad_priority\n";
            char* end = nullptr;
            double target = strtod(tok[3].c_str(), &end);
            if (end == tok[3].c_str() || *end || !(target >= 0) || !std::isfinite(target)) return "ERR bad_target\n";
            // optional tail, in either order: the flow's kind and the link whose capacity it shares (default: the first link)
            int kind = kind_from_name(tok[1]), link = 0;
            for (size_t i = 4; i < tok.size(); ++i) {
                if (tok[i].compare(0, 5, "link=") == 0) {
                    link = find_link(tok[i].substr(5));
                    if (link < 0) return "ERR unknown_link\n";
                } else kind = kind_from_name(tok[i]);
            }
            uint32_t id = reg_.add(tok[1], prio, target, kind, now_ns);
            FlowState& st = state_[id];
            st.link = link;
            st.smooth = WindowSmoother(cfg_.smooth_windows);
            st.bucket.burst_windows = cfg_.burst_windows;
            if (!attach_page(id, st)) { reg_.remove(id); state_.erase(id); return "ERR page_alloc\n"; }
            init_page(id, st, prio, target);
            snprintf(buf, sizeof buf, "OK flow_id=%u page=%s lease_ms=%" PRIu64 " window_us=%" PRIu64 " link=%s\n", id,
                     st.path.empty() ? "-" : st.path.c_str(), cfg_.lease_ns / 1000000, cfg_.window_ns / 1000, links_[link].name.c_str());
            return buf;
        }
        if (cmd == "RENEW" || cmd == "UNREGISTER" || cmd == "BUDGET") {
            if (tok.size() < 2) return "ERR usage\n";
            uint32_t id = (uint32_t)strtoul(tok[1].c_str(), nullptr, 10);
            if (cmd == "RENEW") return reg_.renew(id, now_ns) ? "OK\n" : "ERR unknown_flow\n";
            if (cmd == "UNREGISTER") {
                if (!reg_.remove(id)) return "ERR unknown_flow\n";
                drop_state(id);
                return "OK\n";
            }
            FlowInfo f;
            if (!reg_.get(id, &f)) return "ERR unknown_flow\n";
            FlowState& st = state_[id];
            snprintf(buf, sizeof buf, "OK flow_id=%u mode=%s budget_gbps=%.6f granted=%" PRIu64 " consumed=%" PRIu64
                     " completed=%" PRIu64 " epoch=%" PRIu64 "\n", id, mode_name(f.mode), f.budget_gbps,
                     st.page->granted_bytes, st.page->consumed_bytes, st.page->completed_bytes, st.page->epoch);
            return buf;
        }
        if (cmd == "FLOWS") {
            std::ostringstream os;
            auto flows = reg_.snapshot();
            os << "OK n=" << flows.size();
            for (auto& f : flows) {
                os << " " << f.id << ":" << f.name << ":" << f.priority << ":" << f.target_gbps << ":" << kind_name(f.kind)
                   << ":" << mode_name(f.mode);
                auto it = state_.find(f.id);
                if (it != state_.end() && it->second.link != 0) os << ":" << links_[it->second.link].name;   // only when not the default
            }
            os << "\n";
            return os.str();
        }
        if (cmd == "POLICY") {
            if (tok.size() < 2) { return std::string("OK policy=") + links_[0].policy->name() + "\n"; }
            if (!make_policy(tok[1], cfg_.pcfg)) return "ERR unknown_policy\n";
            cfg_.policy = tok[1];
            for (auto& l : links_) l.policy = make_policy(cfg_.policy, cfg_.pcfg);     // every link runs its own instance
            return std::string("OK policy=") + links_[0].policy->name() + "\n";
        }
        if (cmd == "WINDOW") {
            if (tok.size() < 2) { snprintf(buf, sizeof buf, "OK window_us=%" PRIu64 "\n", cfg_.window_ns / 1000); return buf; }
            uint64_t us = strtoull(tok[1].c_str(), nullptr, 10);
            if (us < 100 || us > 10'000'000) return "ERR bad_window\n";
            cfg_.window_ns = us * 1000;
            snprintf(buf, sizeof buf, "OK window_us=%" PRIu64 "\n", us);
            return buf;
        }
        if (cmd == "CAPACITY") {
            if (tok.size() >= 2) { double c = atof(tok[1].c_str()); if (c > 0) { cfg_.capacity_gbps = c; links_[0].capacity_gbps = c; } }
            snprintf(buf, sizeof buf, "OK capacity_gbps=%.3f\n", cfg_.capacity_gbps);
            return buf;
        }
        if (cmd == "LINK") {
            // LINK <name> [capacity_gbps]: defines a link (or changes its capacity); without a capacity, reports it.
            if (tok.size() < 2) return "ERR usage LINK <name> [capacity_gbps]\n";
            int li = find_link(tok[1]);
            if (tok.size() >= 3) {
                char* end = nullptr;
                const double c = strtod(tok[2].c_str(), &end);
                if (end == tok[2].c_str() || *end || !(c > 0) || !std::isfinite(c)) return "ERR bad_capacity\n";
                if (li < 0) {
                    if (!valid_link_name(tok[1])) return "ERR bad_link_name\n";
                    if (links_.size() >= 64) return "ERR too_many_links\n";
                    links_.push_back(Link{tok[1], c, make_policy(cfg_.policy, cfg_.pcfg)});
                    li = (int)links_.size() - 1;
                } else {
                    links_[li].capacity_gbps = c;
                    if (li == 0) cfg_.capacity_gbps = c;
                }
            }
            if (li < 0) return "ERR unknown_link\n";
            size_t n = 0;
            for (auto& kv : state_) n += kv.second.link == li;
            snprintf(buf, sizeof buf, "OK link=%s capacity_gbps=%.3f flows=%zu\n", links_[li].name.c_str(), links_[li].capacity_gbps, n);
            return buf;
        }
        if (cmd == "LINKS") {
            std::ostringstream os;
            os << "OK n=" << links_.size();
            for (auto& l : links_) os << " " << l.name << ":" << l.capacity_gbps;
            os << "\n";
            return os.str();
        }
        if (cmd == "FLOW") {
            // FLOW <id> <legacy command>: manual override of one flow, same reply line as an end-point.
            if (tok.size() < 3) return "ERR usage FLOW <id> <HIGH|LOWn|SLEEP us|STOP|STATUS>\n";
            uint32_t id = (uint32_t)strtoul(tok[1].c_str(), nullptr, 10);
            auto it = state_.find(id);
            if (it == state_.end()) return "ERR unknown_flow\n";
            std::string rest = line.substr(line.find(tok[2], cmd.size() + 1 + tok[1].size()));
            std::string reply = it->second.ctl.handle(rest);
            FlowState& st = it->second;
            if (reply.compare(0, 2, "OK") == 0) {
                st.manual = rest != "STATUS";
                reg_.update(id, [&](FlowInfo& f) { f.mode = st.ctl.mode(); f.stop = st.ctl.stop_requested(); });
                st.page->mode = (uint32_t)st.ctl.mode();
                st.page->pace_sleep_us = st.ctl.sleep_us();
                if (st.ctl.stop_requested()) st.page->stop = 1;
                if (rest == "HIGH") st.manual = false;  // HIGH hands the flow back to the policy
            }
            return reply;
        }
        if (cmd == "STATS") {
            // the daemon about itself: how many windows it has run, what a policy + grant pass costs, how busy every link was
            std::ostringstream os;
            os << "OK windows=" << window_id_ << " flows=" << reg_.size() << " expired=" << expired_ << " policy=" << links_[0].policy->name()
               << " window_us=" << cfg_.window_ns / 1000 << " step_us_last=" << double(step_cost_last_ns_) * 1e-3
               << " step_us_max=" << double(step_cost_max_ns_) * 1e-3 << " links=" << links_.size();
            for (auto& l : links_) os << " util_pct:" << l.name << "=" << l.last_util_pct;
            os << "\n";
            return os.str();
        }
        if (cmd == "PING") return "OK pong\n";
        return "ERR unknown_cmd\n";
    }

    // ---- one control window ----
    // external_util_pct is used when cfg.external_util is set (e.g. NVML PCIe utilisation).
    // link_gbps (optional): measured traffic per link name in GB/s (NVML counters of the GPU the link belongs to); a link found
    // there takes its utilisation from it instead of from the sum over its registered flows, which misses traffic that did
    // not register.
    std::vector<WindowLog> step_window(uint64_t now_ns, double external_util_pct = 0.0,
                                       const std::map<std::string, double>* link_gbps = nullptr) {
        const auto t_step0 = std::chrono::steady_clock::now();
        for (uint32_t id : reg_.expire(now_ns)) { drop_state(id); ++expired_; }
        auto flows = reg_.snapshot();
        std::vector<FlowSignal> sig;
        double dt = last_step_ns_ ? double(now_ns - last_step_ns_) * 1e-9 : double(cfg_.window_ns) * 1e-9;
        if (dt <= 0) dt = double(cfg_.window_ns) * 1e-9;
        std::vector<double> sum_gbps(links_.size(), 0.0);
        std::vector<std::vector<size_t>> members(links_.size());       // flows of every link, in registry order
        for (auto& f : flows) {
            FlowState& st = state_[f.id];
            uint64_t done = st.page->completed_bytes;
            uint64_t delta = done >= st.last_completed ? done - st.last_completed : 0;
            st.last_completed = done;
            st.smooth.push(double(delta), dt);
            FlowSignal s;
            s.id = f.id; s.priority = f.priority; s.target_gbps = f.target_gbps;
            s.inst_gbps = double(delta) / dt / 1e9;
            s.smooth_gbps = st.smooth.rate() / 1e9;
            s.backlog_bytes = st.page->backlog_bytes;
            s.active = s.backlog_bytes > 0 || delta > 0;
            if (!s.active) st.smooth.clear();
            const size_t li = (size_t)st.link < links_.size() ? (size_t)st.link : 0;
            sum_gbps[li] += s.inst_gbps;
            members[li].push_back(sig.size());
            sig.push_back(s);
        }
        std::vector<WindowLog> logs;
        uint64_t ts = unix_ms();
        // One policy pass per link: flows only compete with the flows that share their link's capacity.
        for (size_t li = 0; li < links_.size(); ++li) {
            if (members[li].empty()) continue;
            std::vector<FlowSignal> lsig;
            for (size_t i : members[li]) lsig.push_back(sig[i]);
            LinkSignal link;
            link.capacity_gbps = links_[li].capacity_gbps;
            // a supplied utilisation (NVML) describes the first link; the others are summed from their flows
            link.util_pct = (cfg_.external_util && li == 0) ? external_util_pct : 100.0 * sum_gbps[li] / std::max(1e-9, link.capacity_gbps);
            if (link_gbps) {
                auto m = link_gbps->find(links_[li].name);
                if (m != link_gbps->end() && std::isfinite(m->second) && m->second >= 0)
                    link.util_pct = 100.0 * m->second / std::max(1e-9, link.capacity_gbps);
            }
            links_[li].last_util_pct = link.util_pct;
            auto dec = links_[li].policy->step(lsig, link);
            for (size_t k = 0; k < dec.size() && k < members[li].size(); ++k) {
                const size_t i = members[li][k];
                const FlowDecision& d = dec[k];
                FlowState& st = state_[d.id];
                int mode = d.mode;
                double budget = d.budget_gbps;
                std::string label = d.decision;
                if (st.manual) {  // an operator pinned this flow with FLOW <id> LOWn / SLEEP
                    mode = st.ctl.mode();
                    budget = mode == SKY_MODE_HIGH ? -1.0
                           : mode == SKY_MODE_CUSTOM ? sleep_to_budget(st.ctl.sleep_us(), link.capacity_gbps)
                           : link.capacity_gbps * ladder_fraction(mode, cfg_.pcfg.low1_fraction);
                    label = "MANUAL";
                }
                SkyCreditPage* pg = st.page;
                if (budget < 0) {
                    pg->unlimited = 1;
                    pg->budget_per_window = 0;
                } else {
                    // Leaving the unlimited state: bytes taken while ungated were never counted against a grant.
                    if (pg->unlimited && pg->consumed_bytes > st.bucket.granted) st.bucket.granted = pg->consumed_bytes;
                    uint64_t g = st.bucket.refill(budget, (uint64_t)(dt * 1e9), pg->consumed_bytes);
                    pg->budget_per_window = (uint64_t)(budget * 1e9 * double(cfg_.window_ns) * 1e-9);
                    __atomic_store_n(&pg->granted_bytes, g, __ATOMIC_RELEASE);
                    pg->unlimited = 0;
                }
                pg->mode = (uint32_t)mode;
                pg->window_ns = cfg_.window_ns;
                __atomic_store_n(&pg->epoch, pg->epoch + 1, __ATOMIC_RELEASE);
                reg_.update(d.id, [&](FlowInfo& f) { f.mode = mode; f.budget_gbps = budget; });
                logs.push_back({window_id_, ts, d.id, flows[i].name, mode, label,
                                budget < 0 ? -1.0 : budget * 1e9 * double(cfg_.window_ns) * 1e-9, sig[i].inst_gbps,
                                sig[i].smooth_gbps, sig[i].backlog_bytes, link.util_pct, pg->granted_bytes});
            }
        }
        last_step_ns_ = now_ns;
        ++window_id_;
        step_cost_last_ns_ = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t_step0).count();
        step_cost_max_ns_ = std::max(step_cost_max_ns_, step_cost_last_ns_);
        return logs;
    }

    // `SLEEP <us>` as a budget: a chunk of the window's worth of bytes every (service + sleep).
    double sleep_to_budget(uint32_t sleep_us, double capacity_gbps) const {
        double win_s = double(cfg_.window_ns) * 1e-9;
        double chunk = capacity_gbps * 1e9 * win_s;  // bytes the link moves in one window
        double service = win_s;
        return chunk / (service + sleep_us * 1e-6) / 1e9;
    }

    static const char* window_csv_header() {
        return "ts_unix_ms,window_id,flow_id,flow,mode,decision,budget_bytes,inst_gbps,smooth_gbps,backlog_bytes,link_util_pct,granted_bytes";
    }
    static std::string window_csv_row(const WindowLog& w) {
        char b[512];
        snprintf(b, sizeof b, "%" PRIu64 ",%" PRIu64 ",%u,%s,%s,%s,%.0f,%.6f,%.6f,%" PRIu64 ",%.3f,%" PRIu64, w.ts_unix_ms,
                 w.window_id, w.flow_id, w.flow.c_str(), mode_name(w.mode), w.decision.c_str(), w.budget_bytes,
                 w.inst_gbps, w.smooth_gbps, w.backlog_bytes, w.link_util_pct, w.granted);
        return b;
    }

    // ---- snapshot / restore (JSON, one flow per array element) ----
    std::string snapshot_json() const {
        std::ostringstream os;
        os << "{\"policy\":\"" << links_[0].policy->name() << "\",\"window_ns\":" << cfg_.window_ns << ",\"capacity_gbps\":"
           << cfg_.capacity_gbps << ",\"window_id\":" << window_id_ << ",\"links\":[";
        for (size_t i = 0; i < links_.size(); ++i)
            os << (i ? "," : "") << "{\"link_name\":\"" << links_[i].name << "\",\"link_capacity_gbps\":" << links_[i].capacity_gbps << "}";
        os << "],\"flows\":[";
        bool first = true;
        for (auto& f : reg_.snapshot()) {
            auto it = state_.find(f.id);
            if (!first) os << ",";
            first = false;
            os << "{\"id\":" << f.id << ",\"name\":\"" << f.name << "\",\"priority\":" << f.priority << ",\"target_gbps\":"
               << f.target_gbps << ",\"kind\":\"" << kind_name(f.kind) << "\",\"mode\":\"" << mode_name(f.mode)
               << "\",\"budget_gbps\":" << f.budget_gbps << ",\"page\":\"" << (it != state_.end() ? it->second.path : "")
               << "\",\"granted\":" << (it != state_.end() ? it->second.page->granted_bytes : 0) << ",\"link\":\""
               << links_[it != state_.end() ? it->second.link : 0].name << "\"}";
        }
        os << "]}";
        return os.str();
    }

    // Restores flows from snapshot_json() output. A tiny purpose-built scanner: the
    // snapshot is machine-written, flat, and has no escapes.
    bool restore_json(const std::string& js, uint64_t now_ns) {
        size_t arr = js.find("\"flows\":[");
        if (arr == std::string::npos) return false;
        auto field = [](const std::string& obj, const std::string& key) -> std::string {
            size_t p = obj.find("\"" + key + "\":");
            if (p == std::string::npos) return "";
            p += key.size() + 3;
            if (obj[p] == '"') { size_t e = obj.find('"', p + 1); return obj.substr(p + 1, e - p - 1); }
            size_t e = obj.find_first_of(",}", p);
            return obj.substr(p, e - p);
        };
        std::string pol = field(js, "policy");
        if (!pol.empty() && make_policy(pol, cfg_.pcfg)) {
            cfg_.policy = pol;
            for (auto& l : links_) l.policy = make_policy(pol, cfg_.pcfg);
        }
        // links first (the array sits before the flows in the snapshot), so that the flows find theirs
        size_t lk = js.find("\"links\":[");
        if (lk != std::string::npos && lk < arr) {
            size_t q = lk + 9;
            while (true) {
                size_t b = js.find('{', q), close = js.find(']', q);
                if (b == std::string::npos || close < b) break;
                size_t e = js.find('}', b);
                if (e == std::string::npos) return false;
                std::string obj = js.substr(b, e - b + 1);
                const std::string name = field(obj, "link_name");
                const double cap = atof(field(obj, "link_capacity_gbps").c_str());
                if (valid_link_name(name) && cap > 0) {
                    int li = find_link(name);
                    if (li < 0 && links_.size() < 64) links_.push_back(Link{name, cap, make_policy(cfg_.policy, cfg_.pcfg)});
                    else if (li >= 0) { links_[li].capacity_gbps = cap; if (li == 0) cfg_.capacity_gbps = cap; }
                }
                q = e + 1;
            }
        }
        size_t p = arr + 9;
        while (true) {
            size_t b = js.find('{', p);
            if (b == std::string::npos) break;
            size_t e = js.find('}', b);
            if (e == std::string::npos) return false;
            std::string obj = js.substr(b, e - b + 1);
            FlowInfo f;
            f.id = (uint32_t)strtoul(field(obj, "id").c_str(), nullptr, 10);
            f.name = field(obj, "name");
            f.priority = atoi(field(obj, "priority").c_str());
            f.target_gbps = atof(field(obj, "target_gbps").c_str());
            f.kind = kind_from_name(field(obj, "kind"));
            int m = mode_from_name(field(obj, "mode"));
            f.mode = m < 0 ? SKY_MODE_HIGH : m;
            f.budget_gbps = atof(field(obj, "budget_gbps").c_str());
            f.registered_ns = now_ns;
            f.lease_deadline_ns = now_ns + reg_.lease_ns();
            if (f.id == 0) return false;
            reg_.restore(f);
            FlowState& st = state_[f.id];
            st.smooth = WindowSmoother(cfg_.smooth_windows);
            st.bucket.burst_windows = cfg_.burst_windows;
            st.link = std::max(0, find_link(field(obj, "link")));       // snapshots from before links existed: the first link
            if (!attach_page(f.id, st)) return false;
            if (st.page->magic != SKYGDR_CREDIT_MAGIC) init_page(f.id, st, f.priority, f.target_gbps);
            st.bucket.granted = st.page->granted_bytes;
            st.last_completed = st.page->completed_bytes;
            p = e + 1;
            if (js.find(']', p) < js.find('{', p)) break;
        }
        return true;
    }

    SkyCreditPage* page(uint32_t id) { auto it = state_.find(id); return it == state_.end() ? nullptr : it->second.page; }
    FlowRegistry& registry() { return reg_; }
    const DaemonConfig& config() const { return cfg_; }
    uint64_t windows() const { return window_id_; }
    uint64_t expired() const { return expired_; }
    const char* policy_name() const { return links_[0].policy->name(); }
    size_t link_count() const { return links_.size(); }

private:
    struct FlowState {
        SkyCreditPage* page = nullptr;
        bool heap = false;
        std::string path;
        uint64_t last_completed = 0;
        WindowSmoother smooth;
        TokenBucket bucket;
        ControlState ctl;
        bool manual = false;
        int link = 0;              // index into links_: the capacity this flow shares
    };
    // A link is one shared capacity (a GPU's NVLink egress, its PCIe link, ...) with its own policy state. Link 0, "default",
    // always exists and carries the configured capacity; more are defined with `LINK <name> <capacity_gbps>`.
    struct Link {
        std::string name;
        double capacity_gbps;
        std::unique_ptr<Policy> policy;
        double last_util_pct = 0;      // utilisation seen in the last window that had flows on this link
    };
    int find_link(const std::string& name) const {
        for (size_t i = 0; i < links_.size(); ++i)
            if (links_[i].name == name) return (int)i;
        return -1;
    }
    static bool valid_link_name(const std::string& n) {
        if (n.empty() || n.size() > 32) return false;
        for (char c : n)
            if (!(isalnum((unsigned char)c) || c == '_' || c == '-' || c == '.' || c == ':' || c == '>')) return false;
        return true;
    }

    bool attach_page(uint32_t id, FlowState& st) {
        if (cfg_.page_dir.empty()) {
            void* p = nullptr;
            if (posix_memalign(&p, 4096, 4096) != 0) return false;
            memset(p, 0, 4096);
            st.page = reinterpret_cast<SkyCreditPage*>(p);
            st.heap = true;
            return true;
        }
        st.path = cfg_.page_dir + "/" + cfg_.tag + "_flow" + std::to_string(id);
        st.page = map_credit_page(st.path, true);
        return st.page != nullptr;
    }
    void init_page(uint32_t id, FlowState& st, int prio, double target) {
        memset(st.page, 0, sizeof(SkyCreditPage));
        st.page->flow_id = id;
        st.page->priority = (uint32_t)std::max(0, prio);
        st.page->target_gbps = target;
        st.page->mode = SKY_MODE_HIGH;
        st.page->unlimited = 1;
        st.page->window_ns = cfg_.window_ns;
        st.page->dead_policy = cfg_.dead_policy;
        st.page->fallback_per_window = (uint64_t)(cfg_.dead_fallback_gbps * 1e9 * double(cfg_.window_ns) * 1e-9);
        st.page->dead_after_windows = cfg_.dead_after_windows;
        st.ctl.configure(0, 100);
        st.ctl.enable();
        __atomic_store_n(&st.page->magic, SKYGDR_CREDIT_MAGIC, __ATOMIC_RELEASE);
    }
    // A flow that is dropped (unregistered, lease expired) loses its page file; at daemon exit the files
    // stay when a snapshot is kept, so that a restarted daemon finds them.
    void release_page(FlowState& st, bool at_exit = false) {
        if (!st.page) return;
        if (st.heap) free(st.page);
        else { unmap_credit_page(st.page); if (!st.path.empty() && !(at_exit && keep_pages_)) unlink(st.path.c_str()); }
        st.page = nullptr;
    }
    void drop_state(uint32_t id) {
        auto it = state_.find(id);
        if (it == state_.end()) return;
        if (it->second.page) it->second.page->stop = 1;  // tell a still-running data path to drain
        release_page(it->second);
        state_.erase(it);
    }

public:
    void keep_pages_on_exit(bool v) { keep_pages_ = v; }

private:
    DaemonConfig cfg_;
    FlowRegistry reg_;
    std::vector<Link> links_;
    std::map<uint32_t, FlowState> state_;
    uint64_t window_id_ = 0, last_step_ns_ = 0, expired_ = 0, step_cost_last_ns_ = 0, step_cost_max_ns_ = 0;
    bool keep_pages_ = false;
};

}  // namespace skygdr
