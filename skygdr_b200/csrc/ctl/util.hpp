// Small host utilities shared by the control plane: size parsing, clocks,
// percentiles and a line-oriented CSV writer.
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

namespace skygdr {

constexpr double kGiB = 1073741824.0;
constexpr double kGB = 1e9;

// "64", "128K", "4M", "2G": binary suffixes, like the reference's parse_size
// (src/cpu_client.cc:66-82, src/tools/pcie_case_study_controller.py:17-31).
// Returns false on malformed input or overflow.
inline bool parse_size(const std::string& text, uint64_t* out) {
    if (text.empty()) return false;
    size_t i = 0;
    unsigned __int128 v = 0;
    bool any = false;
    for (; i < text.size() && text[i] >= '0' && text[i] <= '9'; ++i) {
        v = v * 10 + unsigned(text[i] - '0');
        any = true;
        if (v > (unsigned __int128)UINT64_MAX) return false;
    }
    if (!any) return false;
    unsigned shift = 0;
    if (i < text.size()) {
        char c = text[i];
        if (c == 'k' || c == 'K') shift = 10;
        else if (c == 'm' || c == 'M') shift = 20;
        else if (c == 'g' || c == 'G') shift = 30;
        else if (c == 't' || c == 'T') shift = 40;
        else return false;
        ++i;
        if (i < text.size() && (text[i] == 'i')) ++i;
        if (i < text.size() && (text[i] == 'B' || text[i] == 'b')) ++i;
        if (i != text.size()) return false;
    }
    v <<= shift;
    if (v > (unsigned __int128)UINT64_MAX) return false;
    *out = (uint64_t)v;
    return true;
}

inline uint64_t mono_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch()).count();
}

inline uint64_t unix_ms() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(
               std::chrono::system_clock::now().time_since_epoch()).count();
}

// Percentile by linear interpolation between order statistics of a sorted
// sample (rank = q*(n-1)), the rule of the reference's window flush
// (src/cpu_client.cc:904-913).
inline double percentile_sorted(const std::vector<double>& sorted, double q) {
    if (sorted.empty()) return 0.0;
    if (sorted.size() == 1) return sorted[0];
    q = std::min(1.0, std::max(0.0, q));
    double pos = q * double(sorted.size() - 1);
    size_t lo = (size_t)std::floor(pos);
    size_t hi = std::min(sorted.size() - 1, lo + 1);
    double frac = pos - double(lo);
    return sorted[lo] + (sorted[hi] - sorted[lo]) * frac;
}

inline double percentile(std::vector<double> v, double q) {
    std::sort(v.begin(), v.end());
    return percentile_sorted(v, q);
}

inline std::string trim(std::string s) {
    while (!s.empty() && (s.back() == '\n' || s.back() == '\r' || s.back() == ' ' || s.back() == '\t')) s.pop_back();
    size_t p = 0;
    while (p < s.size() && (s[p] == ' ' || s[p] == '\t')) ++p;
    return s.substr(p);
}

inline std::vector<std::string> split_ws(const std::string& s) {
    std::vector<std::string> out;
    size_t i = 0;
    while (i < s.size()) {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\t')) ++i;
        size_t j = i;
        while (j < s.size() && s[j] != ' ' && s[j] != '\t') ++j;
        if (j > i) out.push_back(s.substr(i, j - i));
        i = j;
    }
    return out;
}

// Exponentially-free moving mean over the last N windows, as the memcpy worker's
// "smooth" bandwidth (src/gpu_be_pcie_memcpy_task.cu:336-396).
class WindowSmoother {
public:
    explicit WindowSmoother(size_t n = 5) : n_(n ? n : 1) {}
    void push(double bytes, double seconds) {
        bytes_.push_back(bytes);
        secs_.push_back(seconds);
        if (bytes_.size() > n_) { bytes_.erase(bytes_.begin()); secs_.erase(secs_.begin()); }
    }
    double rate() const {
        double b = 0, s = 0;
        for (size_t i = 0; i < bytes_.size(); ++i) { b += bytes_[i]; s += secs_[i]; }
        return s > 0 ? b / s : 0.0;
    }
    void clear() { bytes_.clear(); secs_.clear(); }
private:
    size_t n_;
    std::vector<double> bytes_, secs_;
};

}  // namespace skygdr
