// Python bindings of the control plane (module skygdr_b200._ctl). CPU only.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "daemon_core.hpp"
#include "policy.hpp"
#include "protocol.hpp"
#include "signals.hpp"
#include "simulator.hpp"
#include "util.hpp"
#include "workload.hpp"

namespace py = pybind11;
using namespace skygdr;

PYBIND11_MODULE(_ctl, m) {
    m.doc() = "SkyGDR-B200 control plane: protocol, registry, policies, simulator, samplers";

    m.def("parse_size", [](const std::string& s) -> py::object {
        uint64_t v;
        if (!parse_size(s, &v)) return py::none();
        return py::int_(v);
    });
    m.def("percentile", &percentile, py::arg("values"), py::arg("q"));
    m.def("mode_name", &mode_name);
    m.def("mode_from_name", &mode_from_name);
    m.def("ladder_fraction", &ladder_fraction);
    m.def("next_protect_mode", &next_protect_mode);
    m.def("maxmin_fair", &maxmin_fair);
    m.def("kv_bytes_for_tokens", &kv_bytes_for_tokens, py::arg("tokens"), py::arg("layers"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("elem_bytes"), py::arg("align") = 256);
    m.def("pcie_lane_gbs", &pcie_lane_gbs);
    m.def("hbm_peak_gbs", &hbm_peak_gbs);
    m.def("nvlink_peak_gbs", &nvlink_peak_gbs);
    m.attr("CREDIT_MAGIC") = py::int_((uint64_t)SKYGDR_CREDIT_MAGIC);
    m.attr("CREDIT_PAGE_BYTES") = py::int_(SKYGDR_CREDIT_PAGE_BYTES);

    py::class_<ControlState>(m, "ControlState")
        .def(py::init<>())
        .def("configure", &ControlState::configure, py::arg("high_us"), py::arg("low1_us"), py::arg("low2_us") = -1,
             py::arg("low3_us") = -1, py::arg("low4_us") = -1)
        .def("enable", &ControlState::enable)
        .def("handle", &ControlState::handle)
        .def_property_readonly("mode", &ControlState::mode)
        .def_property_readonly("sleep_us", &ControlState::sleep_us)
        .def_property_readonly("commands", &ControlState::commands)
        .def_property_readonly("stop_requested", &ControlState::stop_requested);

    py::class_<PolicyConfig>(m, "PolicyConfig")
        .def(py::init<>())
        .def_readwrite("enter_ratio", &PolicyConfig::enter_ratio)
        .def_readwrite("exit_ratio", &PolicyConfig::exit_ratio)
        .def_readwrite("util_threshold_pct", &PolicyConfig::util_threshold_pct)
        .def_readwrite("enter_windows", &PolicyConfig::enter_windows)
        .def_readwrite("exit_windows", &PolicyConfig::exit_windows)
        .def_readwrite("low1_fraction", &PolicyConfig::low1_fraction)
        .def_readwrite("static_mode", &PolicyConfig::static_mode)
        .def_readwrite("min_be_fraction", &PolicyConfig::min_be_fraction)
        .def_readwrite("md_factor", &PolicyConfig::md_factor)
        .def_readwrite("ai_fraction", &PolicyConfig::ai_fraction)
        .def_readwrite("protect_priority", &PolicyConfig::protect_priority);

    py::class_<FlowSignal>(m, "FlowSignal")
        .def(py::init<>())
        .def_readwrite("id", &FlowSignal::id)
        .def_readwrite("priority", &FlowSignal::priority)
        .def_readwrite("target_gbps", &FlowSignal::target_gbps)
        .def_readwrite("inst_gbps", &FlowSignal::inst_gbps)
        .def_readwrite("smooth_gbps", &FlowSignal::smooth_gbps)
        .def_readwrite("backlog_bytes", &FlowSignal::backlog_bytes)
        .def_readwrite("oldest_age_ms", &FlowSignal::oldest_age_ms)
        .def_readwrite("active", &FlowSignal::active);
    py::class_<LinkSignal>(m, "LinkSignal")
        .def(py::init<>())
        .def_readwrite("capacity_gbps", &LinkSignal::capacity_gbps)
        .def_readwrite("util_pct", &LinkSignal::util_pct);
    py::class_<FlowDecision>(m, "FlowDecision")
        .def_readonly("id", &FlowDecision::id)
        .def_readonly("mode", &FlowDecision::mode)
        .def_readonly("budget_gbps", &FlowDecision::budget_gbps)
        .def_readonly("decision", &FlowDecision::decision);

    py::class_<Policy>(m, "Policy")
        .def("step", &Policy::step)
        .def("reset", &Policy::reset)
        .def_property_readonly("name", [](const Policy& p) { return std::string(p.name()); });
    m.def("make_policy", [](const std::string& name, const PolicyConfig& c) { return make_policy(name, c); },
          py::arg("name"), py::arg("cfg") = PolicyConfig());

    py::class_<TokenBucket>(m, "TokenBucket")
        .def(py::init<>())
        .def_readwrite("granted", &TokenBucket::granted)
        .def_readwrite("burst_windows", &TokenBucket::burst_windows)
        .def("refill", &TokenBucket::refill);

    // ---- workload ----
    py::class_<Rng>(m, "Rng")
        .def(py::init<uint64_t>(), py::arg("seed") = 0)
        .def("next_u64", &Rng::next_u64)
        .def("uniform", py::overload_cast<>(&Rng::uniform))
        .def("uniform_range", py::overload_cast<double, double>(&Rng::uniform))
        .def("exponential", &Rng::exponential)
        .def("normal", &Rng::normal)
        .def("lognormal", &Rng::lognormal);
    py::class_<QuantileSpline>(m, "QuantileSpline").def("inverse_cdf", &QuantileSpline::inverse_cdf);
    m.def("trace_dist", [](const std::string& name, uint64_t max_override) {
        QuantileSpline q;
        if (!trace_dist(name, max_override, &q)) throw py::value_error("dist must be input|cached|computed");
        return q;
    }, py::arg("name"), py::arg("max_override") = 0);
    m.def("sample_trace_tokens", [](const std::string& name, uint64_t seed, size_t n, uint64_t max_override) {
        QuantileSpline q;
        if (!trace_dist(name, max_override, &q)) throw py::value_error("dist must be input|cached|computed");
        Rng rng(seed);
        std::vector<uint64_t> out(n);
        for (auto& v : out) v = sample_tokens(q, rng);
        return out;
    }, py::arg("name"), py::arg("seed"), py::arg("n"), py::arg("max_override") = 0);
    m.def("poisson_uniform", [](uint64_t seed, double rate, double dur, double lo, double hi) {
        std::vector<std::pair<double, uint64_t>> out;
        for (auto& a : poisson_uniform(seed, rate, dur, lo, hi)) out.emplace_back(a.t_s, a.bytes);
        return out;
    });

    // ---- simulator ----
    py::class_<SimFlowSpec>(m, "SimFlowSpec")
        .def(py::init<>())
        .def_readwrite("name", &SimFlowSpec::name)
        .def_readwrite("priority", &SimFlowSpec::priority)
        .def_readwrite("target_gbps", &SimFlowSpec::target_gbps)
        .def_readwrite("kind", &SimFlowSpec::kind)
        .def_readwrite("backlogged", &SimFlowSpec::backlogged)
        .def_readwrite("offered_gbps", &SimFlowSpec::offered_gbps)
        .def_readwrite("contended_efficiency", &SimFlowSpec::contended_efficiency)
        .def_readwrite("link", &SimFlowSpec::link)
        .def("set_arrivals", [](SimFlowSpec& s, const std::vector<std::pair<double, uint64_t>>& a) {
            s.arrivals.clear();
            for (auto& p : a) s.arrivals.push_back({p.first, p.second});
        })
        .def_property_readonly("n_arrivals", [](const SimFlowSpec& s) { return s.arrivals.size(); });
    py::class_<SimConfig>(m, "SimConfig")
        .def(py::init<>())
        .def_readwrite("capacity_gbps", &SimConfig::capacity_gbps)
        .def_readwrite("more_links_gbps", &SimConfig::more_links_gbps)
        .def_readwrite("window_ms", &SimConfig::window_ms)
        .def_readwrite("tick_ms", &SimConfig::tick_ms)
        .def_readwrite("duration_s", &SimConfig::duration_s)
        .def_readwrite("drain_s", &SimConfig::drain_s)
        .def_readwrite("policy_every_windows", &SimConfig::policy_every_windows)
        .def_readwrite("smooth_windows", &SimConfig::smooth_windows)
        .def_readwrite("policy", &SimConfig::policy)
        .def_readwrite("pcfg", &SimConfig::pcfg);
    py::class_<SimWindowRow>(m, "SimWindowRow")
        .def_readonly("window_id", &SimWindowRow::window_id)
        .def_readonly("t_ms", &SimWindowRow::t_ms)
        .def_readonly("flow_id", &SimWindowRow::flow_id)
        .def_readonly("flow", &SimWindowRow::flow)
        .def_readonly("mode", &SimWindowRow::mode)
        .def_readonly("decision", &SimWindowRow::decision)
        .def_readonly("budget_bytes", &SimWindowRow::budget_bytes)
        .def_readonly("inst_gbps", &SimWindowRow::inst_gbps)
        .def_readonly("smooth_gbps", &SimWindowRow::smooth_gbps)
        .def_readonly("backlog_bytes", &SimWindowRow::backlog_bytes)
        .def_readonly("link_util_pct", &SimWindowRow::link_util_pct);
    py::class_<SimRequestRecord>(m, "SimRequestRecord")
        .def_readonly("flow_id", &SimRequestRecord::flow_id)
        .def_readonly("arrival_ms", &SimRequestRecord::arrival_ms)
        .def_readonly("start_ms", &SimRequestRecord::start_ms)
        .def_readonly("finish_ms", &SimRequestRecord::finish_ms)
        .def_readonly("bytes", &SimRequestRecord::bytes);
    py::class_<SimResult>(m, "SimResult")
        .def_readonly("rows", &SimResult::rows)
        .def_readonly("requests", &SimResult::requests)
        .def_readonly("bytes_moved", &SimResult::bytes_moved)
        .def_readonly("bytes_offered", &SimResult::bytes_offered)
        .def_readonly("link_bytes", &SimResult::link_bytes)
        .def_readonly("sim_time_s", &SimResult::sim_time_s)
        .def_readonly("windows", &SimResult::windows)
        .def("flow_times_ms", &SimResult::flow_times_ms);
    // policy: None = cfg.policy by name; or a callable(flows: list[FlowSignal], link: LinkSignal) -> list of budgets in GB/s
    // (negative = unlimited), called once per control window and link.
    m.def("run_simulation", [](const SimConfig& cfg, const std::vector<SimFlowSpec>& specs, py::object policy) {
        if (policy.is_none()) {
            py::gil_scoped_release rel;
            return run_simulation(cfg, specs);
        }
        py::function fn = policy.cast<py::function>();      // owns the callable for the whole call
        // The policy objects live and die inside run_simulation, where the GIL is not held: they keep a non-owning handle and
        // take the GIL around every call.
        const py::handle h = fn;
        auto make = [&cfg, h]() -> std::unique_ptr<Policy> {
            return std::make_unique<CallbackPolicy>(cfg.pcfg, [h](const std::vector<FlowSignal>& flows, const LinkSignal& link) {
                py::gil_scoped_acquire gil;
                return py::reinterpret_borrow<py::function>(h)(flows, link).cast<std::vector<double>>();
            });
        };
        py::gil_scoped_release rel;
        return run_simulation(cfg, specs, make);
    }, py::arg("cfg"), py::arg("specs"), py::arg("policy") = py::none());

    // ---- daemon core ----
    py::class_<DaemonConfig>(m, "DaemonConfig")
        .def(py::init<>())
        .def_readwrite("capacity_gbps", &DaemonConfig::capacity_gbps)
        .def_readwrite("window_ns", &DaemonConfig::window_ns)
        .def_readwrite("lease_ns", &DaemonConfig::lease_ns)
        .def_readwrite("policy", &DaemonConfig::policy)
        .def_readwrite("pcfg", &DaemonConfig::pcfg)
        .def_readwrite("page_dir", &DaemonConfig::page_dir)
        .def_readwrite("tag", &DaemonConfig::tag)
        .def_readwrite("smooth_windows", &DaemonConfig::smooth_windows)
        .def_readwrite("burst_windows", &DaemonConfig::burst_windows)
        .def_readwrite("external_util", &DaemonConfig::external_util)
        .def_readwrite("dead_after_windows", &DaemonConfig::dead_after_windows)
        .def_readwrite("dead_policy", &DaemonConfig::dead_policy)
        .def_readwrite("dead_fallback_gbps", &DaemonConfig::dead_fallback_gbps);
    py::class_<DaemonCore::WindowLog>(m, "WindowLog")
        .def_readonly("window_id", &DaemonCore::WindowLog::window_id)
        .def_readonly("flow_id", &DaemonCore::WindowLog::flow_id)
        .def_readonly("flow", &DaemonCore::WindowLog::flow)
        .def_readonly("mode", &DaemonCore::WindowLog::mode)
        .def_readonly("decision", &DaemonCore::WindowLog::decision)
        .def_readonly("budget_bytes", &DaemonCore::WindowLog::budget_bytes)
        .def_readonly("inst_gbps", &DaemonCore::WindowLog::inst_gbps)
        .def_readonly("smooth_gbps", &DaemonCore::WindowLog::smooth_gbps)
        .def_readonly("backlog_bytes", &DaemonCore::WindowLog::backlog_bytes)
        .def_readonly("link_util_pct", &DaemonCore::WindowLog::link_util_pct)
        .def_readonly("granted", &DaemonCore::WindowLog::granted)
        .def("csv", [](const DaemonCore::WindowLog& w) { return DaemonCore::window_csv_row(w); });
    py::class_<DaemonCore>(m, "DaemonCore")
        .def(py::init<const DaemonConfig&>())
        .def("handle_line", &DaemonCore::handle_line)
        .def("step_window", [](DaemonCore& d, uint64_t now_ns, double external_util_pct, py::object link_gbps) {
            if (link_gbps.is_none()) return d.step_window(now_ns, external_util_pct);
            const auto m = link_gbps.cast<std::map<std::string, double>>();
            return d.step_window(now_ns, external_util_pct, &m);
        }, py::arg("now_ns"), py::arg("external_util_pct") = 0.0, py::arg("link_gbps") = py::none())
        .def("snapshot_json", &DaemonCore::snapshot_json)
        .def("restore_json", &DaemonCore::restore_json)
        .def("keep_pages_on_exit", &DaemonCore::keep_pages_on_exit)
        .def_property_readonly("windows", &DaemonCore::windows)
        .def_property_readonly("expired", &DaemonCore::expired)
        .def_property_readonly("policy_name", [](const DaemonCore& d) { return std::string(d.policy_name()); })
        .def_property_readonly("link_count", &DaemonCore::link_count)
        .def_property_readonly("n_flows", [](DaemonCore& d) { return d.registry().size(); })
        .def_static("csv_header", [] { return std::string(DaemonCore::window_csv_header()); })
        // Usage half of a flow's page, as the data path would write it (tests, in-process flows).
        .def("page_address", [](DaemonCore& d, uint32_t id) { return (uintptr_t)d.page(id); })
        .def("report_usage", [](DaemonCore& d, uint32_t id, uint64_t consumed, uint64_t completed, uint64_t backlog) {
            SkyCreditPage* p = d.page(id);
            if (!p) throw py::key_error("unknown flow");
            p->consumed_bytes = consumed; p->completed_bytes = completed; p->backlog_bytes = backlog;
        })
        .def("page_fields", [](DaemonCore& d, uint32_t id) {
            SkyCreditPage* p = d.page(id);
            if (!p) throw py::key_error("unknown flow");
            py::dict o;
            o["granted_bytes"] = p->granted_bytes; o["epoch"] = p->epoch; o["mode"] = p->mode;
            o["unlimited"] = p->unlimited; o["stop"] = p->stop; o["pace_sleep_us"] = p->pace_sleep_us;
            o["budget_per_window"] = p->budget_per_window; o["consumed_bytes"] = p->consumed_bytes;
            o["completed_bytes"] = p->completed_bytes; o["backlog_bytes"] = p->backlog_bytes;
            o["window_ns"] = p->window_ns; o["target_gbps"] = p->target_gbps;
            o["dead_after_windows"] = p->dead_after_windows; o["dead_policy"] = p->dead_policy;
            o["fallback_per_window"] = p->fallback_per_window; o["heartbeat_lost"] = p->heartbeat_lost;
            return o;
        });

    // Native pacer thread for one page given by address (a page of the daemon core, of pinned host memory, of a mapped file).
    py::class_<PagePacer>(m, "PagePacer")
        .def(py::init([](uint64_t page_addr, double rate_gbps, uint64_t window_ns, double burst_windows) {
            return new PagePacer(reinterpret_cast<SkyCreditPage*>(page_addr), rate_gbps, window_ns, burst_windows);
        }), py::arg("page_addr"), py::arg("rate_gbps"), py::arg("window_ns") = 1000000, py::arg("burst_windows") = 2.0)
        .def("start", &PagePacer::start, py::arg("base") = 0)
        .def("stop", &PagePacer::stop, py::call_guard<py::gil_scoped_release>())
        .def_property_readonly("windows", &PagePacer::windows);

    // The heartbeat rule of host-side data paths, callable on a core's page (tests, in-process flows).
    py::class_<SkyHeartbeatWatch>(m, "HeartbeatWatch")
        .def(py::init([]() { return SkyHeartbeatWatch{0, 0, 0}; }))
        .def_readonly("epoch", &SkyHeartbeatWatch::epoch)
        .def_readonly("t_dead_ns", &SkyHeartbeatWatch::t_dead_ns)
        .def("allowance", [](SkyHeartbeatWatch& w, DaemonCore& d, uint32_t id, uint64_t now_ns) {
            SkyCreditPage* p = d.page(id);
            if (!p) throw py::key_error("unknown flow");
            return sky_host_allowance(p, &w, now_ns);
        });

    // ---- signals, with an injectable NVML ----
    py::class_<PcieSample>(m, "PcieSample")
        .def_readonly("tx_gib_s", &PcieSample::tx_gib_s).def_readonly("rx_gib_s", &PcieSample::rx_gib_s)
        .def_readonly("tx_util_pct", &PcieSample::tx_util_pct).def_readonly("rx_util_pct", &PcieSample::rx_util_pct)
        .def_readonly("tx_peak_util_pct", &PcieSample::tx_peak_util_pct)
        .def_readonly("rx_peak_util_pct", &PcieSample::rx_peak_util_pct)
        .def_readonly("valid", &PcieSample::valid)
        .def("csv", [](const PcieSample& s) { return GpuSignals::pcie_csv_row(s); });
    py::class_<HbmSample>(m, "HbmSample")
        .def_readonly("memory_util_pct", &HbmSample::memory_util_pct)
        .def_readonly("estimated_gb_s", &HbmSample::estimated_gb_s)
        .def_readonly("peak_gb_s", &HbmSample::peak_gb_s).def_readonly("gpu_name", &HbmSample::gpu_name)
        .def_readonly("valid", &HbmSample::valid)
        .def("csv", [](const HbmSample& s) { return GpuSignals::hbm_csv_row(s); });
    py::class_<NvlinkSample>(m, "NvlinkSample")
        .def_readonly("tx_gb_s", &NvlinkSample::tx_gb_s).def_readonly("rx_gb_s", &NvlinkSample::rx_gb_s)
        .def_readonly("valid", &NvlinkSample::valid);
    py::class_<GpuSignals>(m, "GpuSignals")
        // fake: dict with keys name, pcie_gen, pcie_width, and callables pcie(counter)->KB/s, util()->(gpu,mem),
        // nvlink()->(tx_kib, rx_kib). None = bind the real NVML.
        .def(py::init([](unsigned index, py::object fake, double hbm_peak) {
            NvmlApi api;
            if (fake.is_none()) api = NvmlApi::load();
            else {
                py::dict d = fake.cast<py::dict>();
                api.init = [] { return 0; };
                api.shutdown = [] { return 0; };
                api.device_by_index = [](unsigned, void** h) { *h = (void*)0x1; return 0; };
                std::string name = d.contains("name") ? d["name"].cast<std::string>() : "Fake GPU";
                unsigned gen = d.contains("pcie_gen") ? d["pcie_gen"].cast<unsigned>() : 5;
                unsigned width = d.contains("pcie_width") ? d["pcie_width"].cast<unsigned>() : 16;
                api.device_name = [name](void*, std::string* s) { *s = name; return 0; };
                api.max_pcie_gen = [gen](void*, unsigned* v) { *v = gen; return 0; };
                api.max_pcie_width = [width](void*, unsigned* v) { *v = width; return 0; };
                if (d.contains("pcie")) {
                    py::object f = d["pcie"];
                    api.pcie_throughput = [f](void*, unsigned c, unsigned* v) {
                        py::gil_scoped_acquire g;
                        py::object r = f(c);
                        if (r.is_none()) return 1;
                        *v = r.cast<unsigned>();
                        return 0;
                    };
                }
                if (d.contains("util")) {
                    py::object f = d["util"];
                    api.utilization = [f](void*, NvmlUtilization* u) {
                        py::gil_scoped_acquire g;
                        auto t = f().cast<std::pair<unsigned, unsigned>>();
                        u->gpu = t.first; u->memory = t.second;
                        return 0;
                    };
                }
                if (d.contains("nvlink")) {
                    py::object f = d["nvlink"];
                    api.nvlink_kib = [f](void*, uint64_t* tx, uint64_t* rx) {
                        py::gil_scoped_acquire g;
                        auto t = f().cast<std::pair<uint64_t, uint64_t>>();
                        *tx = t.first; *rx = t.second;
                        return 0;
                    };
                }
            }
            return std::make_unique<GpuSignals>(std::move(api), index, hbm_peak);
        }), py::arg("gpu_index") = 0, py::arg("fake") = py::none(), py::arg("hbm_peak_gbs") = 0.0)
        .def_property_readonly("available", &GpuSignals::available)
        .def_property_readonly("name", &GpuSignals::name)
        .def_property_readonly("pcie_peak_gib_s", &GpuSignals::pcie_peak_gib_s)
        .def("sample_pcie", &GpuSignals::sample_pcie)
        .def("sample_hbm", &GpuSignals::sample_hbm)
        .def("sample_nvlink", &GpuSignals::sample_nvlink)
        .def_static("pcie_csv_header", [] { return std::string(GpuSignals::pcie_csv_header()); })
        .def_static("hbm_csv_header", [] { return std::string(GpuSignals::hbm_csv_header()); });
}
