// Signal collectors: NVML-based link and memory counters with the CSV schemas
// of the reference's samplers, behind a function table so tests can install a
// fake NVML.
//
//  * PCIe TX/RX throughput and utilisation against the MAX link generation and
//    width: src/tools/gpu_metrics_logger.py:38-67,298-303,319-321,363-368.
//  * Memory-controller utilisation times a per-GPU peak:
//    src/tools/bandwidth_usage.py:11-25,66-76 (whose table has no H200/B200
//    row; this one does).
//  * NVLink TX/RX byte counters (not sampled by the reference at all).
//
// NVML is opened with dlopen at run time, read-only calls only; nothing here
// changes a GPU setting.
#pragma once
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <string>

#include "util.hpp"

namespace skygdr {

struct NvmlUtilization { unsigned gpu = 0, memory = 0; };

// The subset of NVML that the collectors use. Every member may be empty;
// callers check. Return value 0 = success, as in NVML.
struct NvmlApi {
    std::function<int()> init;
    std::function<int()> shutdown;
    std::function<int(unsigned, void**)> device_by_index;
    std::function<int(void*, std::string*)> device_name;
    std::function<int(void*, unsigned /*0=tx,1=rx*/, unsigned* /*KB/s*/)> pcie_throughput;
    std::function<int(void*, NvmlUtilization*)> utilization;
    std::function<int(void*, unsigned*)> max_pcie_gen, max_pcie_width, cur_pcie_gen, cur_pcie_width;
    std::function<int(void*, unsigned /*0=graphics,1=sm,2=mem*/, unsigned*)> clock_mhz;
    std::function<int(void*, unsigned*)> power_mw;
    // Cumulative NVLink data bytes summed over links: (tx_kib, rx_kib).
    std::function<int(void*, uint64_t*, uint64_t*)> nvlink_kib;
    bool ok() const { return bool(init) && bool(device_by_index); }

    // Binds to libnvidia-ml.so.1 if it is present. Returns an empty table otherwise.
    static NvmlApi load() {
        NvmlApi api;
        void* h = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
        if (!h) return api;
        auto sym = [h](const char* n) { return dlsym(h, n); };
        using fn0 = int (*)();
        using fn_idx = int (*)(unsigned, void**);
        using fn_name = int (*)(void*, char*, unsigned);
        using fn_pcie = int (*)(void*, int, unsigned*);
        using fn_util = int (*)(void*, NvmlUtilization*);
        using fn_u = int (*)(void*, unsigned*);
        using fn_clk = int (*)(void*, int, unsigned*);
        struct FieldValue { unsigned fieldId, scopeId; long long timestamp, latencyUsec; int valueType; int nvmlReturn; unsigned long long value; };
        using fn_fields = int (*)(void*, int, FieldValue*);
        if (auto f = (fn0)sym("nvmlInit_v2")) api.init = [f] { return f(); };
        if (auto f = (fn0)sym("nvmlShutdown")) api.shutdown = [f] { return f(); };
        if (auto f = (fn_idx)sym("nvmlDeviceGetHandleByIndex_v2")) api.device_by_index = [f](unsigned i, void** d) { return f(i, d); };
        if (auto f = (fn_name)sym("nvmlDeviceGetName"))
            api.device_name = [f](void* d, std::string* s) { char b[128] = {0}; int r = f(d, b, sizeof b); *s = b; return r; };
        if (auto f = (fn_pcie)sym("nvmlDeviceGetPcieThroughput")) api.pcie_throughput = [f](void* d, unsigned c, unsigned* v) { return f(d, (int)c, v); };
        if (auto f = (fn_util)sym("nvmlDeviceGetUtilizationRates")) api.utilization = [f](void* d, NvmlUtilization* u) { return f(d, u); };
        if (auto f = (fn_u)sym("nvmlDeviceGetMaxPcieLinkGeneration")) api.max_pcie_gen = [f](void* d, unsigned* v) { return f(d, v); };
        if (auto f = (fn_u)sym("nvmlDeviceGetMaxPcieLinkWidth")) api.max_pcie_width = [f](void* d, unsigned* v) { return f(d, v); };
        if (auto f = (fn_u)sym("nvmlDeviceGetCurrPcieLinkGeneration")) api.cur_pcie_gen = [f](void* d, unsigned* v) { return f(d, v); };
        if (auto f = (fn_u)sym("nvmlDeviceGetCurrPcieLinkWidth")) api.cur_pcie_width = [f](void* d, unsigned* v) { return f(d, v); };
        if (auto f = (fn_clk)sym("nvmlDeviceGetClockInfo")) api.clock_mhz = [f](void* d, unsigned t, unsigned* v) { return f(d, (int)t, v); };
        if (auto f = (fn_u)sym("nvmlDeviceGetPowerUsage")) api.power_mw = [f](void* d, unsigned* v) { return f(d, v); };
        if (auto f = (fn_fields)sym("nvmlDeviceGetFieldValues")) {
            api.nvlink_kib = [f](void* d, uint64_t* tx, uint64_t* rx) {
                // NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX = 138, _RX = 139; scope UINT_MAX = all links.
                FieldValue v[2];
                memset(v, 0, sizeof v);
                v[0].fieldId = 138; v[0].scopeId = 0xffffffffu;
                v[1].fieldId = 139; v[1].scopeId = 0xffffffffu;
                int r = f(d, 2, v);
                if (r != 0) return r;
                if (v[0].nvmlReturn != 0) return v[0].nvmlReturn;
                *tx = v[0].value; *rx = v[1].value;
                return 0;
            };
        }
        return api;
    }
};

// Usable GB/s (decimal) of one PCIe lane per generation, after encoding overhead.
inline double pcie_lane_gbs(unsigned gen) {
    static const double t[] = {0, 0.25, 0.5, 0.985, 1.969, 3.938, 7.563};
    return gen < 7 ? t[gen] : t[6];
}

// Nominal HBM/GDDR peak in GB/s by product name; 0 when unknown.
inline double hbm_peak_gbs(const std::string& name) {
    struct Row { const char* key; double gbs; };
    static const Row rows[] = {
        {"B200", 7700}, {"GB200", 8000}, {"B100", 7700}, {"H200", 4800}, {"H100 PCIe", 2000}, {"H100", 3350},
        {"A100-SXM4-80GB", 2039}, {"A100 80GB", 1935}, {"A100", 1555}, {"V100", 900}, {"L40", 864},
        {"RTX 4090", 1008}, {"RTX 3090", 936},
    };
    for (auto& r : rows) if (name.find(r.key) != std::string::npos) return r.gbs;
    return 0;
}

// Nominal NVLink bandwidth per direction per GPU in GB/s by product name (all links together); 0 when unknown or absent.
inline double nvlink_peak_gbs(const std::string& name) {
    struct Row { const char* key; double gbs; };
    static const Row rows[] = {
        {"GB200", 900}, {"B200", 900}, {"B100", 900}, {"H200", 450}, {"H100 PCIe", 0}, {"H100", 450}, {"A100-SXM", 300}, {"A100", 300}, {"V100", 150},
    };
    for (auto& r : rows) if (name.find(r.key) != std::string::npos) return r.gbs;
    return 0;
}

struct PcieSample {
    uint64_t ts_unix_ms = 0;
    double t_ms = 0;
    double tx_gib_s = 0, rx_gib_s = 0, tx_util_pct = 0, rx_util_pct = 0, tx_peak_util_pct = 0, rx_peak_util_pct = 0;
    bool valid = false;
};

struct HbmSample {
    uint64_t ts_unix_ms = 0;
    double elapsed_ms = 0, memory_util_pct = 0, estimated_gb_s = 0, peak_gb_s = 0;
    unsigned gpu_index = 0;
    std::string gpu_name;
    bool valid = false;
};

struct NvlinkSample {
    uint64_t ts_unix_ms = 0;
    double elapsed_ms = 0, tx_gb_s = 0, rx_gb_s = 0;
    bool valid = false;
};

class GpuSignals {
public:
    GpuSignals(NvmlApi api, unsigned gpu_index, double hbm_peak_override_gbs = 0)
        : api_(std::move(api)), index_(gpu_index) {
        if (!api_.ok()) return;
        if (api_.init() != 0) return;
        inited_ = true;
        if (api_.device_by_index(gpu_index, &dev_) != 0) { dev_ = nullptr; return; }
        if (api_.device_name) api_.device_name(dev_, &name_);
        unsigned gen = 0, width = 0;
        if (api_.max_pcie_gen && api_.max_pcie_gen(dev_, &gen) == 0 && api_.max_pcie_width &&
            api_.max_pcie_width(dev_, &width) == 0)
            pcie_peak_gib_s_ = pcie_lane_gbs(gen) * width * kGB / kGiB;
        hbm_peak_gbs_ = hbm_peak_override_gbs > 0 ? hbm_peak_override_gbs : hbm_peak_gbs(name_);
        t0_ns_ = mono_ns();
    }
    ~GpuSignals() { if (inited_ && api_.shutdown) api_.shutdown(); }
    GpuSignals(const GpuSignals&) = delete;
    GpuSignals& operator=(const GpuSignals&) = delete;

    bool available() const { return dev_ != nullptr; }
    const std::string& name() const { return name_; }
    double pcie_peak_gib_s() const { return pcie_peak_gib_s_; }

    PcieSample sample_pcie() {
        PcieSample s;
        s.ts_unix_ms = unix_ms();
        s.t_ms = (mono_ns() - t0_ns_) * 1e-6;
        if (!dev_ || !api_.pcie_throughput) return s;
        unsigned tx = 0, rx = 0;
        if (api_.pcie_throughput(dev_, 0, &tx) != 0 || api_.pcie_throughput(dev_, 1, &rx) != 0) return s;
        // NVML reports KB/s; the reference reads it as KiB/s (gpu_metrics_logger.py:57-63). Kept.
        s.tx_gib_s = double(tx) * 1024.0 / kGiB;
        s.rx_gib_s = double(rx) * 1024.0 / kGiB;
        if (pcie_peak_gib_s_ > 0) {
            s.tx_util_pct = 100.0 * s.tx_gib_s / pcie_peak_gib_s_;
            s.rx_util_pct = 100.0 * s.rx_gib_s / pcie_peak_gib_s_;
        }
        tx_peak_ = std::max(tx_peak_, s.tx_util_pct);
        rx_peak_ = std::max(rx_peak_, s.rx_util_pct);
        s.tx_peak_util_pct = tx_peak_;
        s.rx_peak_util_pct = rx_peak_;
        s.valid = true;
        return s;
    }

    HbmSample sample_hbm() {
        HbmSample s;
        s.ts_unix_ms = unix_ms();
        s.elapsed_ms = (mono_ns() - t0_ns_) * 1e-6;
        s.gpu_index = index_;
        s.gpu_name = name_;
        s.peak_gb_s = hbm_peak_gbs_;
        if (!dev_ || !api_.utilization) return s;
        NvmlUtilization u;
        if (api_.utilization(dev_, &u) != 0) return s;
        s.memory_util_pct = u.memory;
        s.estimated_gb_s = hbm_peak_gbs_ * u.memory / 100.0;
        s.valid = true;
        return s;
    }

    NvlinkSample sample_nvlink() {
        NvlinkSample s;
        s.ts_unix_ms = unix_ms();
        uint64_t now = mono_ns();
        s.elapsed_ms = (now - t0_ns_) * 1e-6;
        if (!dev_ || !api_.nvlink_kib) return s;
        uint64_t tx = 0, rx = 0;
        if (api_.nvlink_kib(dev_, &tx, &rx) != 0) return s;
        if (have_nvl_) {
            double dt = (now - nvl_ns_) * 1e-9;
            if (dt > 0) {
                s.tx_gb_s = double(tx - nvl_tx_) * 1024.0 / dt / 1e9;
                s.rx_gb_s = double(rx - nvl_rx_) * 1024.0 / dt / 1e9;
                s.valid = true;
            }
        }
        have_nvl_ = true; nvl_tx_ = tx; nvl_rx_ = rx; nvl_ns_ = now;
        return s;
    }

    static const char* pcie_csv_header() {
        return "ts_unix_ms,t_ms,pcie_tx_GiB_s,pcie_rx_GiB_s,pcie_tx_util_pct,pcie_rx_util_pct,pcie_tx_peak_util_pct,pcie_rx_peak_util_pct";
    }
    static std::string pcie_csv_row(const PcieSample& s) {
        char b[256];
        snprintf(b, sizeof b, "%llu,%.3f,%.6f,%.6f,%.3f,%.3f,%.3f,%.3f", (unsigned long long)s.ts_unix_ms, s.t_ms,
                 s.tx_gib_s, s.rx_gib_s, s.tx_util_pct, s.rx_util_pct, s.tx_peak_util_pct, s.rx_peak_util_pct);
        return b;
    }
    static const char* hbm_csv_header() {
        return "ts_unix_ms,elapsed_ms,memory_util_pct,estimated_mem_bw_GB_s,peak_mem_bw_GB_s,gpu_index,gpu_name";
    }
    static std::string hbm_csv_row(const HbmSample& s) {
        char b[320];
        snprintf(b, sizeof b, "%llu,%.3f,%.1f,%.3f,%.3f,%u,%s", (unsigned long long)s.ts_unix_ms, s.elapsed_ms,
                 s.memory_util_pct, s.estimated_gb_s, s.peak_gb_s, s.gpu_index, s.gpu_name.c_str());
        return b;
    }

private:
    NvmlApi api_;
    unsigned index_;
    void* dev_ = nullptr;
    bool inited_ = false;
    std::string name_;
    double pcie_peak_gib_s_ = 0, hbm_peak_gbs_ = 0;
    double tx_peak_ = 0, rx_peak_ = 0;
    uint64_t t0_ns_ = 0;
    bool have_nvl_ = false;
    uint64_t nvl_tx_ = 0, nvl_rx_ = 0, nvl_ns_ = 0;
};

}  // namespace skygdr
