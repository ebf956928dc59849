// Shared layout of a per-flow credit page.
//
// One page per registered flow. The control side (fabricd, or an in-process
// pacer thread) owns the "grant" half; the data path (a CUDA kernel or a host
// copy worker) owns the "usage" half. The page lives in host memory that is
// mapped into the GPU's address space (pinned + mapped, or a /dev/shm file
// that the GPU process page-locks), so the control side never calls the CUDA
// API: it only stores to plain memory.
//
// This replaces the reference's pacing knob, a sleep after each post batch
// (src/cpu_client.cc:875-879, modes at :93-102), with a byte budget that the
// data path checks per chunk.
//
// The struct is plain C so that it compiles for host C++17, for device code
// and can be mirrored from Python with ctypes/struct.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKYGDR_CREDIT_MAGIC 0x534b59474452ull /* "SKYGDR" */
#define SKYGDR_CREDIT_PAGE_BYTES 256

// Control modes keep the reference's names and numbering
// (src/cpu_client.cc:93-102).
enum SkyMode {
    SKY_MODE_DISABLED = 0,
    SKY_MODE_HIGH = 1,
    SKY_MODE_LOW1 = 2,
    SKY_MODE_LOW2 = 3,
    SKY_MODE_LOW3 = 4,
    SKY_MODE_LOW4 = 5,
    SKY_MODE_CUSTOM = 6,
};

// Status codes a data-path kernel leaves in its status word.
enum SkyStatus {
    SKY_STATUS_OK = 0,
    SKY_STATUS_YIELD_CREDIT = 1,   // ran out of credit before the deadline; cursor says where to resume
    SKY_STATUS_STOPPED = 2,        // stop flag was set; cursor says where it stopped
    SKY_STATUS_TIMEOUT_FLAG = 3,   // a bounded wait on a peer flag gave up
    SKY_STATUS_BAD_INDEX = 4,      // a bounds check rejected an index (debug builds)
    SKY_STATUS_TIMEOUT_MBAR = 5,   // a bounded wait on an mbarrier gave up
    SKY_STATUS_CONTROL_LOST = 6,   // the control side's heartbeat went stale and the page says to stall then
};

// What a data path does once the control side's epoch has not moved for `dead_after_windows` windows
// (a daemon that died or hung): the reference has no heartbeat at all.
enum SkyDeadPolicy {
    SKY_DEAD_STALL = 0,            // keep the last grant; give up with SKY_STATUS_CONTROL_LOST when it runs out
    SKY_DEAD_UNPACED = 1,          // carry on without a gate
    SKY_DEAD_STATIC = 2,           // grant itself `fallback_per_window` bytes per window from the moment of detection
};

typedef struct SkyCreditPage {
    // ---- grant half: written by the control side only ----
    uint64_t magic;            // SKYGDR_CREDIT_MAGIC once initialised
    uint64_t granted_bytes;    // cumulative bytes the flow may consume (monotonic)
    uint64_t epoch;            // control-window counter; a heartbeat
    uint64_t window_ns;        // length of one control window
    uint64_t budget_per_window;// bytes added to granted_bytes each window (0 = none)
    uint32_t mode;             // SkyMode
    uint32_t unlimited;        // 1: no gate at all (HIGH with no cap)
    uint32_t stop;             // 1: data path should drain and return
    uint32_t pace_sleep_us;    // legacy sleep knob for host-issued flows
    uint32_t flow_id;
    uint32_t priority;
    double   target_gbps;      // goal of the flow (0 = best effort)
    uint32_t dead_after_windows;   // heartbeat: epoch unchanged for this many windows = control side gone (0 = never)
    uint32_t dead_policy;          // SkyDeadPolicy
    uint64_t fallback_per_window;  // SKY_DEAD_STATIC: bytes per window
    uint64_t _pad_grant[5];
    // ---- usage half: written by the data path only (offset 128) ----
    uint64_t consumed_bytes;   // tickets taken so far (cumulative)
    uint64_t completed_bytes;  // bytes known to be delivered (cumulative)
    uint64_t stall_ns;         // time spent waiting for credit
    uint64_t busy_ns;          // time spent moving bytes
    uint64_t last_ts_ns;       // globaltimer / CLOCK_MONOTONIC stamp of last update
    uint64_t chunks;           // chunks moved
    uint64_t yields;           // times the data path gave up and returned early
    uint64_t backlog_bytes;    // bytes requested of the flow and not yet delivered
    uint64_t heartbeat_lost;   // 0, or 1 + the epoch at which the data path last found the heartbeat stale
    uint64_t heartbeat_lost_ns;// data-path clock at that moment
    uint64_t _pad_usage[6];
} SkyCreditPage;

// Host-side data paths (copy workers, the compat client) follow the same heartbeat rule as the kernels: the bytes
// a flow may have consumed by `now_ns`, given the page and a watch that the caller keeps between calls.
typedef struct SkyHeartbeatWatch {
    uint64_t epoch;        // last epoch seen
    uint64_t t_change_ns;  // when it last changed (caller's clock); 0 = not started
    uint64_t t_dead_ns;    // when the control side was taken for dead; 0 = alive
} SkyHeartbeatWatch;

#if !defined(__CUDA_ARCH__)
static inline uint64_t sky_host_allowance(SkyCreditPage* p, SkyHeartbeatWatch* w, uint64_t now_ns) {
    if (__atomic_load_n(&p->unlimited, __ATOMIC_RELAXED)) return ~0ull;
    const uint64_t granted = __atomic_load_n(&p->granted_bytes, __ATOMIC_ACQUIRE);
    const uint32_t n = __atomic_load_n(&p->dead_after_windows, __ATOMIC_RELAXED);
    if (n == 0) return granted;
    const uint64_t e = __atomic_load_n(&p->epoch, __ATOMIC_ACQUIRE);
    if (w->t_change_ns == 0 || e != w->epoch) {
        w->epoch = e;
        w->t_change_ns = now_ns;
        w->t_dead_ns = 0;
        return granted;
    }
    if (w->t_dead_ns == 0) {
        if (now_ns - w->t_change_ns <= (uint64_t)n * p->window_ns) return granted;
        w->t_dead_ns = now_ns;
        p->heartbeat_lost_ns = now_ns;
        __atomic_store_n(&p->heartbeat_lost, e + 1, __ATOMIC_RELEASE);
    }
    if (p->dead_policy == SKY_DEAD_UNPACED) return ~0ull;
    if (p->dead_policy == SKY_DEAD_STATIC) {
        const uint64_t win = p->window_ns ? p->window_ns : 1;
        return granted + (now_ns - w->t_dead_ns) / win * p->fallback_per_window;
    }
    return granted;        // SKY_DEAD_STALL: what was granted is all there is
}
#endif

#ifdef __cplusplus
}
static_assert(sizeof(SkyCreditPage) == SKYGDR_CREDIT_PAGE_BYTES, "credit page must be 256 bytes");
#endif
