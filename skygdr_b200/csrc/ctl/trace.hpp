// Timeline ranges for the control plane (nsys -t nvtx shows them next to the kernels they pace).
//
// NVTX v3 is header-only: nothing is linked, and without a profiler attached a range is one branch on a
// cached flag. Ranges are emitted only when SKYGDR_NVTX=1 is in the environment, the same switch as the
// Python side (skygdr_b200/utils/nvtx.py). Built without the CUDA toolkit's headers, TraceRange is empty.
//
// The reference documents `nsys profile -t cuda,nvtx` (llm_problem_analysis/README.md:1003-1021) and emits
// no ranges anywhere.
#pragma once
#include <cstdlib>
#include <cstring>

#if defined(SKYGDR_WITH_NVTX) && defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define SKYGDR_NVTX_AVAILABLE 1
#endif
#endif

namespace skygdr {

inline bool trace_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("SKYGDR_NVTX");
        return v != nullptr && std::strcmp(v, "1") == 0;
    }();
    return on;
}

#ifdef SKYGDR_NVTX_AVAILABLE
class TraceRange {
public:
    explicit TraceRange(const char* name) : on_(trace_enabled()) { if (on_) nvtxRangePushA(name); }
    ~TraceRange() { if (on_) nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
private:
    bool on_;
};
inline void trace_mark(const char* name) { if (trace_enabled()) nvtxMarkA(name); }
inline constexpr bool trace_compiled_in() { return true; }
#else
class TraceRange {
public:
    explicit TraceRange(const char*) {}
};
inline void trace_mark(const char*) {}
inline constexpr bool trace_compiled_in() { return false; }
#endif

}  // namespace skygdr
