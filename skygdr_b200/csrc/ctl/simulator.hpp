// CPU fabric simulator: one or more shared links, registered flows, and the
// signal -> policy -> action loop running on simulated time.
//
// The reference has no simulator; its loop needs two hosts and a RoCE NIC
// (src/README.md:58-64). This gives the same loop a fabric that runs
// anywhere: each control window the policy sees per-flow achieved rate,
// backlog and link utilisation (the signals of
// src/tools/pcie_case_study_controller.py:275-300) and answers with per-flow
// byte budgets; between control points the link is shared max-min fair among
// the transfers that are active, whatever their priority, which is how an
// unscheduled fabric behaves (README.md:27-30).
#pragma once
#include <algorithm>
#include <cmath>
#include <deque>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "policy.hpp"
#include "util.hpp"
#include "workload.hpp"

namespace skygdr {

struct SimFlowSpec {
    std::string name;
    int priority = 0;
    double target_gbps = 0;
    int kind = FLOW_OTHER;
    bool backlogged = false;          // always has bytes to send
    double offered_gbps = -1;         // cap on what the source can offer (<0: none)
    // Useful fraction of the flow's link share while at least one other flow is moving bytes in the same tick (1 = the
    // flow does not suffer from company). Models measured asymmetries such as the reference's: a copy-engine transfer keeps
    // its rate next to an HBM-bound decoder, the decoder loses about 10 %
    // (llm_problem_analysis/bench_results_20260515_092702/summary.txt:13-25). The link time is used up either way.
    double contended_efficiency = 1.0;
    int link = 0;                     // which of the simulated links the flow uses (0 = SimConfig::capacity_gbps)
    std::vector<Arrival> arrivals;    // finite requests, FIFO, one transfer at a time
};

struct SimConfig {
    double capacity_gbps = 64.0;
    std::vector<double> more_links_gbps;   // capacities of links 1, 2, ...: each is shared only by the flows that name it
    double window_ms = 5.0;
    double tick_ms = 0.25;
    double duration_s = 10.0;
    double drain_s = 5.0;             // extra time to let queued requests finish
    int policy_every_windows = 1;     // 20 = a 100 ms policy on 5 ms windows
    int smooth_windows = 5;
    std::string policy = "target_track";
    PolicyConfig pcfg;
};

struct SimWindowRow {
    uint64_t window_id;
    double t_ms;
    uint32_t flow_id;
    std::string flow;
    int mode;
    std::string decision;
    double budget_bytes;     // <0 unlimited
    double inst_gbps, smooth_gbps;
    uint64_t backlog_bytes;
    double link_util_pct;
};

struct SimRequestRecord { uint32_t flow_id; double arrival_ms, start_ms, finish_ms; uint64_t bytes; };

struct SimResult {
    std::vector<SimWindowRow> rows;
    std::vector<SimRequestRecord> requests;
    std::vector<double> bytes_moved;      // per flow
    std::vector<double> bytes_offered;    // per flow (sum of arrivals; backlogged: moved)
    double link_bytes = 0;
    double sim_time_s = 0;
    uint64_t windows = 0;
    std::vector<double> flow_times_ms(uint32_t flow_id) const {
        std::vector<double> v;
        for (auto& r : requests) if (r.flow_id == flow_id && r.finish_ms >= 0) v.push_back(r.finish_ms - r.arrival_ms);
        return v;
    }
};

// Max-min fair split of `capacity` among `demand[i]`; returns the allocation.
inline std::vector<double> maxmin_fair(const std::vector<double>& demand, double capacity) {
    std::vector<double> alloc(demand.size(), 0.0);
    std::vector<size_t> open;
    for (size_t i = 0; i < demand.size(); ++i) if (demand[i] > 0) open.push_back(i);
    double left = capacity;
    while (!open.empty() && left > 1e-9) {
        double share = left / double(open.size());
        bool any_sat = false;
        std::vector<size_t> still;
        for (size_t i : open) {
            double want = demand[i] - alloc[i];
            if (want <= share + 1e-12) { alloc[i] += want; left -= want; any_sat = true; }
            else still.push_back(i);
        }
        if (!any_sat) {
            for (size_t i : still) alloc[i] += share;
            left = 0;
            break;
        }
        open.swap(still);
    }
    return alloc;
}

// `custom` (optional): makes the policy instance of a link instead of make_policy(cfg.policy); one call per link.
inline SimResult run_simulation(const SimConfig& cfg, const std::vector<SimFlowSpec>& specs,
                                const std::function<std::unique_ptr<Policy>()>& custom = nullptr) {
    SimResult res;
    const size_t n = specs.size();
    // links: capacity, member flows, one policy instance each (as in the daemon)
    std::vector<double> link_cap{cfg.capacity_gbps};
    for (double c : cfg.more_links_gbps) link_cap.push_back(c > 0 ? c : cfg.capacity_gbps);
    const size_t n_links = link_cap.size();
    std::vector<std::vector<size_t>> members(n_links);
    for (size_t i = 0; i < n; ++i) members[(specs[i].link >= 0 && (size_t)specs[i].link < n_links) ? (size_t)specs[i].link : 0].push_back(i);
    std::vector<std::unique_ptr<Policy>> policies;
    for (size_t l = 0; l < n_links; ++l) {
        auto pol = custom ? custom() : make_policy(cfg.policy, cfg.pcfg);
        if (!pol) pol = make_policy("none", cfg.pcfg);
        policies.push_back(std::move(pol));
    }
    auto link_of = [&](size_t i) { return (specs[i].link >= 0 && (size_t)specs[i].link < n_links) ? (size_t)specs[i].link : (size_t)0; };

    struct Live {
        std::deque<SimRequestRecord> queue;  // arrived, unfinished (front = in flight)
        double front_left = 0;
        size_t next_arrival = 0;
        double budget_gbps = -1;             // decided by the policy
        double window_budget_left = -1;      // bytes; <0 unlimited
        double carry = 0;                    // unused credit carried into the next window (<= 1 window)
        double window_bytes = 0;
        WindowSmoother smooth;
        int mode = SKY_MODE_HIGH;
        std::string decision = "HOLD";
    };
    std::vector<Live> live(n);
    for (auto& l : live) l.smooth = WindowSmoother(cfg.smooth_windows);
    res.bytes_moved.assign(n, 0.0);
    res.bytes_offered.assign(n, 0.0);
    for (size_t i = 0; i < n; ++i) for (auto& a : specs[i].arrivals) res.bytes_offered[i] += double(a.bytes);

    const double tick_s = cfg.tick_ms * 1e-3, win_s = cfg.window_ms * 1e-3;
    const int ticks_per_window = std::max(1, (int)std::llround(cfg.window_ms / cfg.tick_ms));
    double t = 0;
    uint64_t window_id = 0;
    std::vector<double> window_link_bytes(n_links, 0.0);
    std::vector<std::vector<FlowDecision>> last_dec(n_links);

    auto all_done = [&]() {
        for (size_t i = 0; i < n; ++i) {
            if (specs[i].backlogged) continue;
            if (live[i].next_arrival < specs[i].arrivals.size() || !live[i].queue.empty()) return false;
        }
        return true;
    };

    while (t < cfg.duration_s + cfg.drain_s) {
        if (t >= cfg.duration_s && all_done()) break;
        // ---- start of a control window: set this window's byte budgets ----
        for (size_t i = 0; i < n; ++i) {
            Live& l = live[i];
            if (l.budget_gbps < 0) { l.window_budget_left = -1; l.carry = 0; }
            else {
                double add = l.budget_gbps * 1e9 * win_s;
                l.window_budget_left = add + std::min(l.carry, add);
            }
            l.window_bytes = 0;
        }
        std::fill(window_link_bytes.begin(), window_link_bytes.end(), 0.0);
        // ---- ticks ----
        for (int k = 0; k < ticks_per_window; ++k) {
            // arrivals up to the end of this tick become visible at its start + their offset
            for (size_t i = 0; i < n; ++i) {
                Live& l = live[i];
                while (l.next_arrival < specs[i].arrivals.size() && specs[i].arrivals[l.next_arrival].t_s <= t) {
                    const Arrival& a = specs[i].arrivals[l.next_arrival++];
                    SimRequestRecord r{(uint32_t)(i + 1), a.t_s * 1e3, -1, -1, a.bytes};
                    if (l.queue.empty()) { l.front_left = double(a.bytes); r.start_ms = t * 1e3; }
                    l.queue.push_back(r);
                }
            }
            std::vector<double> demand(n, 0.0);
            for (size_t i = 0; i < n; ++i) {
                Live& l = live[i];
                double want;
                bool past_end = t >= cfg.duration_s;
                const double link_tick = link_cap[link_of(i)] * 1e9 * tick_s;
                if (specs[i].backlogged) want = past_end ? 0.0 : link_tick;
                else want = l.queue.empty() ? 0.0 : l.front_left;
                if (specs[i].offered_gbps >= 0) want = std::min(want, specs[i].offered_gbps * 1e9 * tick_s);
                if (l.window_budget_left >= 0) want = std::min(want, l.window_budget_left);
                demand[i] = std::min(want, link_tick);
            }
            // every link is split max-min fair among its own flows
            std::vector<double> alloc(n, 0.0);
            std::vector<int> movers(n_links, 0);
            for (size_t lk = 0; lk < n_links; ++lk) {
                std::vector<double> dl;
                for (size_t i : members[lk]) dl.push_back(demand[i]);
                const std::vector<double> al = maxmin_fair(dl, link_cap[lk] * 1e9 * tick_s);
                for (size_t k = 0; k < members[lk].size(); ++k) { alloc[members[lk][k]] = al[k]; movers[lk] += al[k] > 0; }
            }
            for (size_t i = 0; i < n; ++i) {
                Live& l = live[i];
                double b = alloc[i];
                if (b <= 0) continue;
                window_link_bytes[link_of(i)] += b;                  // the share of the link is spent in full
                if (movers[link_of(i)] > 1) b *= std::min(1.0, std::max(0.0, specs[i].contended_efficiency));
                l.window_bytes += b;
                res.bytes_moved[i] += b;
                if (l.window_budget_left >= 0) l.window_budget_left -= b;
                if (!specs[i].backlogged) {
                    l.front_left -= b;
                    if (l.front_left <= 0.5) {
                        // finished somewhere inside this tick: interpolate the finish time
                        SimRequestRecord r = l.queue.front();
                        l.queue.pop_front();
                        r.finish_ms = (t + tick_s) * 1e3;
                        res.requests.push_back(r);
                        if (!l.queue.empty()) { l.front_left = double(l.queue.front().bytes); l.queue.front().start_ms = (t + tick_s) * 1e3; }
                        else l.front_left = 0;
                    }
                }
            }
            t += tick_s;
        }
        // ---- end of window: signals ----
        std::vector<LinkSignal> links(n_links);
        for (size_t lk = 0; lk < n_links; ++lk) {
            res.link_bytes += window_link_bytes[lk];
            links[lk] = LinkSignal{link_cap[lk], 100.0 * window_link_bytes[lk] / (link_cap[lk] * 1e9 * win_s)};
        }
        std::vector<FlowSignal> sig(n);
        for (size_t i = 0; i < n; ++i) {
            Live& l = live[i];
            l.smooth.push(l.window_bytes, win_s);
            if (l.window_budget_left > 0) l.carry = l.window_budget_left; else l.carry = 0;
            FlowSignal& s = sig[i];
            s.id = (uint32_t)(i + 1);
            s.priority = specs[i].priority;
            s.target_gbps = specs[i].target_gbps;
            s.inst_gbps = l.window_bytes / win_s / 1e9;
            s.smooth_gbps = l.smooth.rate() / 1e9;
            double backlog = l.front_left;
            for (size_t q = 1; q < l.queue.size(); ++q) backlog += double(l.queue[q].bytes);
            s.backlog_bytes = specs[i].backlogged ? UINT64_MAX / 2 : (uint64_t)backlog;
            s.oldest_age_ms = l.queue.empty() ? 0.0 : t * 1e3 - l.queue.front().arrival_ms;
            s.active = s.backlog_bytes > 0 || l.window_bytes > 0;
            if (!s.active) l.smooth.clear();
        }
        // ---- policy ----
        for (size_t lk = 0; lk < n_links; ++lk) {
            if (members[lk].empty()) continue;
            if (window_id % (uint64_t)std::max(1, cfg.policy_every_windows) == 0 || last_dec[lk].empty()) {
                std::vector<FlowSignal> lsig;
                for (size_t i : members[lk]) lsig.push_back(sig[i]);
                last_dec[lk] = policies[lk]->step(lsig, links[lk]);
            } else {
                for (auto& d : last_dec[lk]) d.decision = "HOLD";
            }
            for (auto& d : last_dec[lk]) {
                if (d.id == 0 || d.id > n) continue;
                Live& l = live[d.id - 1];
                l.budget_gbps = d.budget_gbps;
                l.mode = d.mode;
                l.decision = d.decision;
            }
        }
        for (size_t i = 0; i < n; ++i) {
            Live& l = live[i];
            res.rows.push_back({window_id, t * 1e3, (uint32_t)(i + 1), specs[i].name, l.mode, l.decision,
                                l.budget_gbps < 0 ? -1.0 : l.budget_gbps * 1e9 * win_s, sig[i].inst_gbps,
                                sig[i].smooth_gbps, specs[i].backlogged ? 0 : sig[i].backlog_bytes, links[link_of(i)].util_pct});
        }
        ++window_id;
    }
    // requests that never finished
    for (size_t i = 0; i < n; ++i)
        for (auto& r : live[i].queue) res.requests.push_back(r);
    res.sim_time_s = t;
    res.windows = window_id;
    return res;
}

}  // namespace skygdr
