// Policies: map per-window signals and per-flow goals to per-flow budgets.
//
// `ladder` reproduces the decision rule of the reference's controller
// (src/tools/pcie_case_study_controller.py:273-352): while the protected flow
// is unfinished, if its smoothed rate is below enter_ratio x baseline AND the
// shared link is busy (util >= threshold) for `enter_windows` consecutive
// windows, push every best-effort flow one notch down HIGH->LOW1->...->LOW4
// (:125-131); when the protected flow has nothing left, go back to HIGH. It
// never de-escalates while the protected flow is active: exit_ratio and
// exit_windows are parsed there but unused (:165,168).
//
// `target_track` is this runtime's default: a feed-forward reservation
// (capacity - sum of active protected targets) trimmed by AIMD feedback that
// does use the exit thresholds.
#pragma once
#include <cmath>
#include <memory>
#include <string>
#include <vector>

#include <functional>

#include "credit_page.h"
#include "protocol.hpp"

namespace skygdr {

struct FlowSignal {
    uint32_t id = 0;
    int priority = 0;
    double target_gbps = 0;     // 0 = best effort
    double inst_gbps = 0;       // achieved in the last window
    double smooth_gbps = 0;     // achieved over the last few windows
    uint64_t backlog_bytes = 0; // bytes queued and not yet delivered
    double oldest_age_ms = 0;   // age of the oldest unfinished request
    bool active = false;        // has backlog or moved bytes in the window
};

struct LinkSignal {
    double capacity_gbps = 0;
    double util_pct = 0;        // 0..100, share of capacity used in the last window
};

struct FlowDecision {
    uint32_t id = 0;
    int mode = SKY_MODE_HIGH;
    double budget_gbps = -1;    // <0: unlimited
    std::string decision = "HOLD";
};

struct PolicyConfig {
    double enter_ratio = 0.65;      // reference default (pcie_case_study_controller.py:164)
    double exit_ratio = 0.80;       // :165
    double util_threshold_pct = 85; // :166 (rx_threshold_pct)
    int enter_windows = 1;          // :167
    int exit_windows = 2;           // :168
    double low1_fraction = 0.5;     // share of link capacity a best-effort flow keeps in LOW1
    int static_mode = SKY_MODE_LOW1;// for the `static` policy
    double min_be_fraction = 0.02;  // floor for best-effort budgets (never starve entirely)
    double md_factor = 0.5;         // multiplicative decrease
    double ai_fraction = 0.05;      // additive increase per healthy streak, share of capacity
    int protect_priority = 50;      // flows with priority >= this and a target are protected
};

// Rate a flow keeps in ladder mode m, as a share of capacity. The reference's
// ladder is a sleep ladder, LOWn sleep = {1, 1.25, 1.5, 1.75} x LOW1 sleep
// (src/cpu_client.cc:536-542); with rate = batch / (service + sleep) and LOW1
// defined as share f1, the service time is s*f1/(1-f1) and LOWn keeps
// 1 / (1 + k_n * (1/f1 - 1)).
inline double ladder_fraction(int mode, double f1) {
    static const double k[] = {0, 0, 1.0, 1.25, 1.5, 1.75};
    if (mode <= SKY_MODE_HIGH || mode > SKY_MODE_LOW4) return 1.0;
    double r = 1.0 / f1 - 1.0;
    return 1.0 / (1.0 + k[mode] * r);
}

inline int next_protect_mode(int mode) {
    if (mode < SKY_MODE_HIGH || mode > SKY_MODE_LOW4) return SKY_MODE_HIGH;
    return mode == SKY_MODE_LOW4 ? SKY_MODE_LOW4 : mode + 1;
}

class Policy {
public:
    explicit Policy(const PolicyConfig& c) : cfg(c) {}
    virtual ~Policy() = default;
    virtual const char* name() const = 0;
    // One call per control window.
    virtual std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) = 0;
    virtual void reset() {}
    PolicyConfig cfg;

protected:
    bool is_protected(const FlowSignal& f) const { return f.target_gbps > 0 && f.priority >= cfg.protect_priority; }
};

// always-HIGH arm: no scheduling.
class NonePolicy : public Policy {
public:
    using Policy::Policy;
    const char* name() const override { return "none"; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal&) override {
        std::vector<FlowDecision> out;
        for (auto& f : flows) out.push_back({f.id, SKY_MODE_HIGH, -1.0, "HOLD"});
        return out;
    }
};

// always-LOW arm: best-effort flows are throttled all the time.
class StaticPolicy : public Policy {
public:
    using Policy::Policy;
    const char* name() const override { return "static"; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) override {
        std::vector<FlowDecision> out;
        for (auto& f : flows) {
            if (is_protected(f)) out.push_back({f.id, SKY_MODE_HIGH, -1.0, "HOLD"});
            else out.push_back({f.id, cfg.static_mode,
                                link.capacity_gbps * ladder_fraction(cfg.static_mode, cfg.low1_fraction), "HOLD"});
        }
        return out;
    }
};

class LadderPolicy : public Policy {
public:
    using Policy::Policy;
    const char* name() const override { return "ladder"; }
    void reset() override { mode_ = SKY_MODE_HIGH; streak_ = 0; was_active_ = false; }
    int mode() const { return mode_; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) override {
        // The protected flow is "unfinished" while it has backlog.
        bool any_active = false, bad = false;
        for (auto& f : flows) {
            if (!is_protected(f)) continue;
            if (f.backlog_bytes > 0) {
                any_active = true;
                double guard = f.smooth_gbps > 0 ? f.smooth_gbps : f.inst_gbps;
                if (!std::isnan(guard) && guard < cfg.enter_ratio * f.target_gbps &&
                    !std::isnan(link.util_pct) && link.util_pct >= cfg.util_threshold_pct)
                    bad = true;
            }
        }
        std::string label = "HOLD";
        if (any_active) {
            streak_ = bad ? streak_ + 1 : 0;
            if (streak_ >= cfg.enter_windows) {
                int nxt = next_protect_mode(mode_);
                if (nxt != mode_) {
                    label = std::string(mode_ == SKY_MODE_HIGH ? "SWITCH_" : "ESCALATE_") + mode_name(nxt);
                    mode_ = nxt;
                }
                streak_ = 0;
            }
            was_active_ = true;
        } else {
            if (was_active_ && mode_ != SKY_MODE_HIGH) label = "RESTORE_DONE_HIGH";
            mode_ = SKY_MODE_HIGH;
            streak_ = 0;
            was_active_ = false;
        }
        std::vector<FlowDecision> out;
        for (auto& f : flows) {
            if (is_protected(f)) out.push_back({f.id, SKY_MODE_HIGH, -1.0, "HOLD"});
            else {
                double b = mode_ == SKY_MODE_HIGH ? -1.0 : link.capacity_gbps * ladder_fraction(mode_, cfg.low1_fraction);
                out.push_back({f.id, mode_, b, label});
            }
        }
        return out;
    }

private:
    int mode_ = SKY_MODE_HIGH;
    int streak_ = 0;
    bool was_active_ = false;
};

class TargetTrackPolicy : public Policy {
public:
    using Policy::Policy;
    const char* name() const override { return "target_track"; }
    void reset() override { trim_ = 1.0; bad_streak_ = good_streak_ = 0; }
    double trim() const { return trim_; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) override {
        double reserve = 0;
        bool any_active = false, bad = false, healthy = true;
        int n_be = 0;
        for (auto& f : flows) {
            if (!is_protected(f)) { ++n_be; continue; }
            if (f.backlog_bytes == 0) continue;
            any_active = true;
            reserve += f.target_gbps;
            double guard = f.smooth_gbps > 0 ? f.smooth_gbps : f.inst_gbps;
            if (std::isnan(guard)) continue;  // stale or missing signal: hold
            if (guard < cfg.enter_ratio * f.target_gbps && link.util_pct >= cfg.util_threshold_pct) bad = true;
            if (guard < cfg.exit_ratio * f.target_gbps) healthy = false;
        }
        std::string label = "HOLD";
        if (!any_active) {
            // Nothing to protect: release in one step, remember nothing.
            if (trim_ < 1.0 || released_ == false) label = "RELEASE";
            trim_ = 1.0;
            bad_streak_ = good_streak_ = 0;
            released_ = true;
        } else {
            released_ = false;
            if (bad) { ++bad_streak_; good_streak_ = 0; }
            else if (healthy) { ++good_streak_; bad_streak_ = 0; }
            else { bad_streak_ = 0; good_streak_ = 0; }
            if (bad_streak_ >= cfg.enter_windows) {
                trim_ = std::max(cfg.min_be_fraction, trim_ * cfg.md_factor);
                bad_streak_ = 0;
                label = "DECREASE";
            } else if (good_streak_ >= cfg.exit_windows && trim_ < 1.0) {
                trim_ = std::min(1.0, trim_ + cfg.ai_fraction);
                good_streak_ = 0;
                label = "INCREASE";
            } else if (label == "HOLD") {
                label = "RESERVE";
            }
        }
        std::vector<FlowDecision> out;
        double be_total = -1.0;
        if (any_active) {
            double left = std::max(0.0, link.capacity_gbps - reserve);
            be_total = std::max(cfg.min_be_fraction * link.capacity_gbps, left * trim_);
        }
        for (auto& f : flows) {
            if (is_protected(f)) { out.push_back({f.id, SKY_MODE_HIGH, -1.0, "HOLD"}); continue; }
            if (be_total < 0) out.push_back({f.id, SKY_MODE_HIGH, -1.0, label});
            else out.push_back({f.id, SKY_MODE_CUSTOM, be_total / std::max(1, n_be), label});
        }
        return out;
    }

private:
    double trim_ = 1.0;
    int bad_streak_ = 0, good_streak_ = 0;
    bool released_ = true;
};

// target_track with the unprotected share split by priority instead of evenly: while a protected flow is being served, an
// unprotected flow i that is active gets (priority_i + 1) / sum over the active unprotected flows of what the link has left,
// and an idle one is offered what it would get if it woke up. Priorities below the protection line thus act as weights among
// the best-effort traffic (the reference knows two classes only: the protected restore and everything else).
class WeightedTrackPolicy : public TargetTrackPolicy {
public:
    using TargetTrackPolicy::TargetTrackPolicy;
    const char* name() const override { return "weighted_track"; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) override {
        std::vector<FlowDecision> out = TargetTrackPolicy::step(flows, link);
        double total = 0, weights_active = 0;
        int n_be = 0;
        for (size_t i = 0; i < flows.size() && i < out.size(); ++i) {
            if (is_protected(flows[i]) || out[i].budget_gbps < 0) continue;
            total += out[i].budget_gbps;                       // the even split adds up to the unprotected share
            ++n_be;
            if (flows[i].active) weights_active += weight(flows[i]);
        }
        if (n_be < 2) return out;
        for (size_t i = 0; i < flows.size() && i < out.size(); ++i) {
            if (is_protected(flows[i]) || out[i].budget_gbps < 0) continue;
            const double w = weight(flows[i]);
            const double denom = flows[i].active ? weights_active : weights_active + w;
            out[i].budget_gbps = std::max(cfg.min_be_fraction * link.capacity_gbps / n_be, total * w / std::max(1e-9, denom));
        }
        return out;
    }

private:
    static double weight(const FlowSignal& f) { return double(std::max(0, f.priority)) + 1.0; }
};

// A policy supplied by the embedding program (the Python binding wraps a callable in it): every window it gets the flows'
// signals and the link's and returns, per flow, a budget in GB/s (negative = unlimited). For trying a rule out against the
// simulator before writing it in C++.
class CallbackPolicy : public Policy {
public:
    using Fn = std::function<std::vector<double>(const std::vector<FlowSignal>&, const LinkSignal&)>;
    CallbackPolicy(const PolicyConfig& c, Fn fn) : Policy(c), fn_(std::move(fn)) {}
    const char* name() const override { return "callback"; }
    std::vector<FlowDecision> step(const std::vector<FlowSignal>& flows, const LinkSignal& link) override {
        const std::vector<double> budgets = fn_(flows, link);
        std::vector<FlowDecision> out;
        for (size_t i = 0; i < flows.size(); ++i) {
            const double b = i < budgets.size() && std::isfinite(budgets[i]) ? budgets[i] : -1.0;    // missing or NaN: leave the flow alone
            out.push_back({flows[i].id, b < 0 ? SKY_MODE_HIGH : SKY_MODE_CUSTOM, b < 0 ? -1.0 : b, b < 0 ? "HOLD" : "CALLBACK"});
        }
        return out;
    }

private:
    Fn fn_;
};

inline std::unique_ptr<Policy> make_policy(const std::string& name, const PolicyConfig& cfg) {
    if (name == "weighted_track") return std::make_unique<WeightedTrackPolicy>(cfg);
    if (name == "none" || name == "always_high") return std::make_unique<NonePolicy>(cfg);
    if (name == "static" || name == "always_low") return std::make_unique<StaticPolicy>(cfg);
    if (name == "ladder") return std::make_unique<LadderPolicy>(cfg);
    if (name == "target_track") return std::make_unique<TargetTrackPolicy>(cfg);
    return nullptr;
}

// Token bucket arithmetic used by every grant writer: cumulative grant after a
// window of `window_ns` at `budget_gbps` (decimal GB/s), with at most
// `burst_windows` windows of unused credit carried over.
struct TokenBucket {
    uint64_t granted = 0;
    double burst_windows = 2.0;
    // consumed = cumulative bytes the data path has taken so far.
    uint64_t refill(double budget_gbps, uint64_t window_ns, uint64_t consumed) {
        if (budget_gbps < 0) return granted;  // unlimited: the page's `unlimited` flag carries it
        double add = budget_gbps * 1e9 * (double(window_ns) * 1e-9);
        double cap = add * burst_windows;
        if (consumed >= granted) {
            // Tickets beyond the grant are waiting, not spent: extend by one window.
            granted += (uint64_t)add;
            return granted;
        }
        double unused = double(granted - consumed);
        uint64_t g = consumed + (uint64_t)std::min(cap, unused + add);
        if (g > granted) granted = g;  // monotonic even when the budget just shrank
        return granted;
    }
};

}  // namespace skygdr
