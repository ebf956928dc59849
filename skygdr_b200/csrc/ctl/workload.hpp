// Workload generators: trace-shaped token counts, KV sizes, arrival processes.
//
// The trace shape is the reference's: tokens per LLM call follow a piecewise
// log-uniform law pinned to p50/p90/p99/max of a Codex / SWE-bench-Pro trace,
// with 50 % of the mass in [p50/8, p50], 40 % in [p50, p90], 9 % in [p90, p99]
// and 1 % in [p99, max] (llm_problem_analysis/kv_nvlink_transfer_trace.cu:80-111,
// :214-244). Here it is one inverse-CDF evaluation of a log-linear quantile
// spline, driven by a counter-based generator, so a (seed, index) pair always
// gives the same sample on every platform.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

namespace skygdr {

// splitmix64: stateless mixing of a 64-bit counter.
inline uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

class Rng {
public:
    explicit Rng(uint64_t seed = 0) : s_(mix64(seed ^ 0x5ca1ab1e0ddba11ull)) {}
    uint64_t next_u64() { s_ += 0x9e3779b97f4a7c15ull; return mix64(s_); }
    // Uniform in [0,1) with 53 random bits.
    double uniform() { return double(next_u64() >> 11) * (1.0 / 9007199254740992.0); }
    double uniform(double lo, double hi) { return lo + (hi - lo) * uniform(); }
    double exponential(double rate) { return -std::log(1.0 - uniform()) / rate; }
    double normal() {  // Box-Muller, one value per call
        double u1 = 1.0 - uniform(), u2 = uniform();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
    // Log-normal given its median and sigma of the underlying normal, clipped.
    double lognormal(double median, double sigma, double lo, double hi) {
        double v = median * std::exp(sigma * normal());
        return std::min(hi, std::max(lo, v));
    }
private:
    uint64_t s_;
};

struct QuantileKnot { double prob; double value; };

// Quantile spline, linear in log(value) between knots.
class QuantileSpline {
public:
    QuantileSpline() = default;
    explicit QuantileSpline(std::vector<QuantileKnot> k) : knots_(std::move(k)) {}
    double inverse_cdf(double u) const {
        if (knots_.empty()) return 0;
        if (u <= knots_.front().prob) return knots_.front().value;
        for (size_t i = 1; i < knots_.size(); ++i) {
            if (u < knots_[i].prob || i + 1 == knots_.size()) {
                const auto &a = knots_[i - 1], &b = knots_[i];
                double t = (std::min(u, b.prob) - a.prob) / (b.prob - a.prob);
                double la = std::log(std::max(1.0, a.value)), lb = std::log(std::max(1.0, b.value));
                return std::exp(la + (lb - la) * t);
            }
        }
        return knots_.back().value;
    }
    const std::vector<QuantileKnot>& knots() const { return knots_; }
private:
    std::vector<QuantileKnot> knots_;
};

// name in {input, cached, computed}; max_override > 0 replaces the cap.
inline bool trace_dist(const std::string& name, uint64_t max_override, QuantileSpline* out) {
    double p50, p90, p99, cap;
    if (name == "input") { p50 = 63917; p90 = 114888; p99 = 166322; cap = 200000; }
    else if (name == "cached") { p50 = 60928; p90 = 112512; p99 = 162048; cap = 200000; }
    else if (name == "computed") { p50 = 758; p90 = 8736; p99 = 53323; cap = 70000; }
    else return false;
    if (max_override > 0) cap = double(max_override);
    cap = std::max(cap, p99);
    double lo = std::max(1.0, std::floor(p50 / 8.0));
    *out = QuantileSpline({{0.0, lo}, {0.5, p50}, {0.9, p90}, {0.99, p99}, {1.0, cap}});
    return true;
}

inline uint64_t sample_tokens(const QuantileSpline& d, Rng& rng) {
    return (uint64_t)std::max(1.0, std::floor(d.inverse_cdf(rng.uniform())));
}

// tokens x layers x kv_heads x head_dim x 2 (K and V) x elem_bytes, rounded up
// to 256 B (llm_problem_analysis/kv_nvlink_transfer_trace.cu:190-203).
inline uint64_t kv_bytes_for_tokens(uint64_t tokens, uint64_t layers, uint64_t kv_heads, uint64_t head_dim,
                                    uint64_t elem_bytes, uint64_t align = 256) {
    unsigned __int128 b = (unsigned __int128)tokens * layers * kv_heads * head_dim * 2 * elem_bytes;
    uint64_t v = b > (unsigned __int128)UINT64_MAX ? UINT64_MAX : (uint64_t)b;
    if (align > 1 && v <= UINT64_MAX - align) v = (v + align - 1) / align * align;
    return v;
}

struct Arrival { double t_s; uint64_t bytes; };

// Poisson arrivals at `rate` per second over `duration_s`, sizes uniform in
// [lo_bytes, hi_bytes].
inline std::vector<Arrival> poisson_uniform(uint64_t seed, double rate, double duration_s, double lo_bytes,
                                            double hi_bytes) {
    Rng rng(seed);
    std::vector<Arrival> out;
    double t = 0;
    for (;;) {
        t += rng.exponential(rate);
        if (t >= duration_s) break;
        out.push_back({t, (uint64_t)rng.uniform(lo_bytes, hi_bytes)});
    }
    return out;
}

}  // namespace skygdr
