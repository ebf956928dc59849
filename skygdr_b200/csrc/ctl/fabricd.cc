// fabricd: the control daemon.
//
//   fabricd --port 7070 [--bind 127.0.0.1] [--policy target_track|weighted_track|ladder|static|none]
//           [--window_us 5000] [--capacity_gbps 64] [--lease_ms 5000] [--log PATH.csv]
//           [--snapshot PATH.json] [--restore PATH.json] [--gpu N --util_source pcie_rx|pcie_tx|sum]
//           [--link NAME=GBPS ...]   more links beside the default one (each a shared capacity with its own policy pass)
//           [--unix PATH]            also listen on a Unix-domain socket (same protocol; for clients on the same host)
//           [--link_signal NAME=GPU:pcie_rx|pcie_tx|nvlink_rx|nvlink_tx ...]   a link's utilisation from that GPU's NVML counters
//                                    (sampled by a thread of its own) instead of the sum over its registered flows
//           [--enter_ratio 0.65 --exit_ratio 0.80 --util_threshold_pct 85 --enter_windows 1 --exit_windows 2]
//
// A TCP line server (one or more commands per connection, each answered by one
// line) in front of DaemonCore, plus a timer thread that runs one
// signal -> policy -> action step per control window. SIGTERM/SIGINT write the
// snapshot file and leave the credit pages in place, so a restarted daemon
// (--restore) picks the same flows up while their kernels keep running on the
// last grant.
//
// The reference's counterpart is a Python process polling CSV files at 10 Hz
// (src/tools/pcie_case_study_controller.py:174-368) and a listener thread
// inside the load generator (src/cpu_client.cc:238-315).
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/select.h>
#include <sys/socket.h>
#include <sys/un.h>

#include <atomic>
#include <cerrno>
#include <map>
#include <mutex>
#include <thread>

#include "daemon_core.hpp"
#include "trace.hpp"
#include "signals.hpp"

using namespace skygdr;

static std::atomic<int> g_stop{0};
static void on_signal(int) { g_stop.store(1); }

static int make_listener(const std::string& ip, int port) {
    int ls = socket(AF_INET, SOCK_STREAM, 0);
    if (ls < 0) return -1;
    int yes = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &yes, sizeof yes);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1) { close(ls); return -1; }
    if (bind(ls, (sockaddr*)&a, sizeof a) != 0 || listen(ls, 64) != 0) { close(ls); return -1; }
    return ls;
}

static int make_unix_listener(const std::string& path) {
    sockaddr_un a{};
    if (path.empty() || path.size() >= sizeof a.sun_path) return -1;
    int ls = socket(AF_UNIX, SOCK_STREAM, 0);
    if (ls < 0) return -1;
    a.sun_family = AF_UNIX;
    memcpy(a.sun_path, path.c_str(), path.size() + 1);
    unlink(path.c_str());                                  // a socket file left by an earlier daemon
    if (bind(ls, (sockaddr*)&a, sizeof a) != 0 || listen(ls, 64) != 0) { close(ls); return -1; }
    return ls;
}

int main(int argc, char** argv) {
    DaemonConfig cfg;
    int port = 7070, gpu = -1;
    std::string bind_ip = "127.0.0.1", log_path, snap_path, restore_path, util_source = "sum";
    std::vector<std::pair<std::string, std::string>> link_defs;
    std::string unix_path;
    struct LinkSignalDef { std::string link, source; int gpu = 0; };
    std::vector<LinkSignalDef> signal_defs;
    for (int i = 1; i < argc; ++i) {
        std::string k = argv[i];
        std::string v;
        size_t eq = k.find('=');
        if (eq != std::string::npos) { v = k.substr(eq + 1); k = k.substr(0, eq); }
        else if (i + 1 < argc) v = argv[++i];
        if (k == "--port") port = atoi(v.c_str());
        else if (k == "--bind") bind_ip = v;
        else if (k == "--policy") cfg.policy = v;
        else if (k == "--window_us") cfg.window_ns = strtoull(v.c_str(), nullptr, 10) * 1000;
        else if (k == "--capacity_gbps") cfg.capacity_gbps = atof(v.c_str());
        else if (k == "--lease_ms") cfg.lease_ns = strtoull(v.c_str(), nullptr, 10) * 1000000;
        else if (k == "--log") log_path = v;
        else if (k == "--snapshot") snap_path = v;
        else if (k == "--restore") restore_path = v;
        else if (k == "--page_dir") cfg.page_dir = v;
        else if (k == "--tag") cfg.tag = v;
        else if (k == "--gpu") gpu = atoi(v.c_str());
        else if (k == "--util_source") util_source = v;
        else if (k == "--enter_ratio") cfg.pcfg.enter_ratio = atof(v.c_str());
        else if (k == "--exit_ratio") cfg.pcfg.exit_ratio = atof(v.c_str());
        else if (k == "--util_threshold_pct") cfg.pcfg.util_threshold_pct = atof(v.c_str());
        else if (k == "--enter_windows") cfg.pcfg.enter_windows = atoi(v.c_str());
        else if (k == "--exit_windows") cfg.pcfg.exit_windows = atoi(v.c_str());
        else if (k == "--low1_fraction") cfg.pcfg.low1_fraction = atof(v.c_str());
        else if (k == "--dead_after_windows") cfg.dead_after_windows = (uint32_t)strtoul(v.c_str(), nullptr, 10);
        else if (k == "--dead_policy") {
            if (v == "stall") cfg.dead_policy = SKY_DEAD_STALL;
            else if (v == "unpaced") cfg.dead_policy = SKY_DEAD_UNPACED;
            else if (v == "static") cfg.dead_policy = SKY_DEAD_STATIC;
            else { fprintf(stderr, "fabricd: --dead_policy is stall, unpaced or static\n"); return 2; }
        }
        else if (k == "--dead_fallback_gbps") cfg.dead_fallback_gbps = atof(v.c_str());
        else if (k == "--unix") unix_path = v;
        else if (k == "--link_signal") {
            const size_t e = v.rfind('='), c = v.rfind(':');
            LinkSignalDef d;
            if (e == std::string::npos || c == std::string::npos || c < e) { fprintf(stderr, "fabricd: --link_signal NAME=GPU:SOURCE\n"); return 2; }
            d.link = v.substr(0, e); d.gpu = atoi(v.substr(e + 1, c - e - 1).c_str()); d.source = v.substr(c + 1);
            if (d.source != "pcie_rx" && d.source != "pcie_tx" && d.source != "nvlink_rx" && d.source != "nvlink_tx") {
                fprintf(stderr, "fabricd: --link_signal source is pcie_rx, pcie_tx, nvlink_rx or nvlink_tx\n");
                return 2;
            }
            signal_defs.push_back(d);
        }
        else if (k == "--link") {
            const size_t e = v.rfind('=');
            if (e == std::string::npos || e == 0) { fprintf(stderr, "fabricd: --link NAME=GBPS\n"); return 2; }
            link_defs.emplace_back(v.substr(0, e), v.substr(e + 1));
        }
        else { fprintf(stderr, "fabricd: unknown flag %s\n", k.c_str()); return 2; }
    }
    if (cfg.window_ns < 100000) { fprintf(stderr, "fabricd: window below 100 us\n"); return 2; }
    cfg.tag += "_" + std::to_string(port);
    cfg.external_util = gpu >= 0 && util_source != "sum";
    DaemonCore core(cfg);
    core.keep_pages_on_exit(!snap_path.empty());
    for (auto& ld : link_defs) {
        const std::string rep = core.handle_line("LINK " + ld.first + " " + ld.second, mono_ns());
        if (rep.compare(0, 2, "OK") != 0) { fprintf(stderr, "fabricd: --link %s=%s: %s", ld.first.c_str(), ld.second.c_str(), rep.c_str()); return 2; }
    }
    if (!restore_path.empty()) {
        std::ifstream in(restore_path);
        std::stringstream ss;
        ss << in.rdbuf();
        if (!core.restore_json(ss.str(), mono_ns())) fprintf(stderr, "fabricd: restore from %s failed\n", restore_path.c_str());
        else fprintf(stderr, "fabricd: restored %zu flows\n", core.registry().size());
    }
    std::unique_ptr<GpuSignals> sigs;
    if (gpu >= 0) sigs = std::make_unique<GpuSignals>(NvmlApi::load(), (unsigned)gpu);

    struct sigaction sa{};
    sa.sa_handler = on_signal;
    sigaction(SIGTERM, &sa, nullptr);
    sigaction(SIGINT, &sa, nullptr);
    signal(SIGPIPE, SIG_IGN);

    int ls = make_listener(bind_ip, port);
    if (ls < 0) { perror("fabricd: listen"); return 1; }
    fprintf(stderr, "fabricd: listening on %s:%d policy=%s window_us=%llu capacity_gbps=%.1f\n", bind_ip.c_str(), port,
            core.policy_name(), (unsigned long long)(cfg.window_ns / 1000), cfg.capacity_gbps);
    if (trace_enabled()) fprintf(stderr, "fabricd: nvtx ranges %s\n", trace_compiled_in() ? "on" : "requested but not compiled in");

    // Measured traffic of the links that have a signal: a sampler thread keeps the latest GB/s per link (the NVML calls
    // average over tens of milliseconds and may block that long, which a control window cannot afford).
    for (auto& d : signal_defs) {
        const std::string rep = core.handle_line("LINK " + d.link, mono_ns());
        if (rep.compare(0, 2, "OK") != 0) { fprintf(stderr, "fabricd: --link_signal names an unknown link %s\n", d.link.c_str()); return 2; }
    }
    std::mutex sig_mu;
    std::map<std::string, double> measured_gbps;
    std::thread sampler;
    if (!signal_defs.empty()) {
        NvmlApi api = NvmlApi::load();
        if (!api.ok()) fprintf(stderr, "fabricd: NVML is not available, --link_signal is ignored\n");
        else sampler = std::thread([&, api] {
            std::map<int, std::unique_ptr<GpuSignals>> gpus;
            for (auto& d : signal_defs)
                if (!gpus.count(d.gpu)) gpus[d.gpu] = std::make_unique<GpuSignals>(api, (unsigned)d.gpu);
            while (!g_stop.load()) {
                for (auto& d : signal_defs) {
                    GpuSignals& gs = *gpus[d.gpu];
                    double gbps = -1;
                    if (d.source.compare(0, 4, "pcie") == 0) {
                        PcieSample s = gs.sample_pcie();
                        if (s.valid) gbps = (d.source == "pcie_tx" ? s.tx_gib_s : s.rx_gib_s) * 1.073741824;
                    } else {
                        NvlinkSample s = gs.sample_nvlink();
                        if (s.valid) gbps = d.source == "nvlink_tx" ? s.tx_gb_s : s.rx_gb_s;
                    }
                    std::lock_guard<std::mutex> g(sig_mu);
                    if (gbps >= 0) measured_gbps[d.link] = gbps; else measured_gbps.erase(d.link);
                }
                std::this_thread::sleep_for(std::chrono::milliseconds(5));
            }
        });
    }

    std::mutex mu;
    FILE* log = log_path.empty() ? nullptr : fopen(log_path.c_str(), "w");
    if (log) { fprintf(log, "%s\n", DaemonCore::window_csv_header()); fflush(log); }

    std::thread timer([&] {
        uint64_t next = mono_ns() + cfg.window_ns;
        uint64_t rows = 0;
        while (!g_stop.load()) {
            uint64_t now = mono_ns();
            if (now < next) { std::this_thread::sleep_for(std::chrono::nanoseconds(std::min<uint64_t>(next - now, 2'000'000))); continue; }
            TraceRange window_range("fabricd.window");
            double util = 0;
            if (sigs && cfg.external_util) {
                TraceRange r("fabricd.signals");
                PcieSample s = sigs->sample_pcie();
                util = util_source == "pcie_tx" ? s.tx_util_pct : s.rx_util_pct;
            }
            std::vector<DaemonCore::WindowLog> logs;
            uint64_t win_ns;
            {
                std::lock_guard<std::mutex> g(mu);
                TraceRange r("fabricd.policy_and_grants");
                std::map<std::string, double> seen;
                if (sampler.joinable()) { std::lock_guard<std::mutex> sg(sig_mu); seen = measured_gbps; }
                logs = core.step_window(now, util, seen.empty() ? nullptr : &seen);
                win_ns = core.config().window_ns;
            }
            if (log) {
                for (auto& w : logs) fprintf(log, "%s\n", DaemonCore::window_csv_row(w).c_str());
                if ((++rows & 63) == 0) fflush(log);
            }
            next += win_ns;
            if (next < now) next = now + win_ns;  // fell behind: do not burst
        }
    });

    auto serve = [&](int c) {
        int yes = 1;
        setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &yes, sizeof yes);
        timeval rto{1, 0};
        setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &rto, sizeof rto);
        std::string acc;
        char buf[1024];
        int idle = 0;
        while (!g_stop.load()) {
            ssize_t n = recv(c, buf, sizeof buf, 0);
            if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK) && ++idle < 30) continue;  // idle persistent client
            if (n <= 0) {
                // Peer closed without a newline: the legacy clients send one bare command.
                if (!acc.empty()) {
                    std::string rep;
                    { std::lock_guard<std::mutex> g(mu); rep = core.handle_line(acc, mono_ns()); }
                    send(c, rep.data(), rep.size(), MSG_NOSIGNAL);
                }
                break;
            }
            idle = 0;
            acc.append(buf, (size_t)n);
            size_t nl;
            bool quit = false;
            while ((nl = acc.find('\n')) != std::string::npos) {
                std::string line = acc.substr(0, nl);
                acc.erase(0, nl + 1);
                if (trim(line) == "QUIT") { quit = true; break; }
                if (trim(line) == "SHUTDOWN") { g_stop.store(1); quit = true; send(c, "OK\n", 3, MSG_NOSIGNAL); break; }
                std::string rep;
                {
                    TraceRange r("fabricd.request");
                    std::lock_guard<std::mutex> g(mu);
                    rep = core.handle_line(line, mono_ns());
                }
                if (send(c, rep.data(), rep.size(), MSG_NOSIGNAL) < 0) { quit = true; break; }
            }
            if (quit) break;
            if (acc.size() > 4096) break;
        }
        close(c);
    };
    std::vector<std::thread> conns;

    int uls = -1;
    if (!unix_path.empty()) {
        uls = make_unix_listener(unix_path);
        if (uls < 0) { perror("fabricd: unix listen"); g_stop.store(1); }
        else fprintf(stderr, "fabricd: also listening on unix:%s\n", unix_path.c_str());
    }
    while (!g_stop.load()) {
        fd_set rf;
        FD_ZERO(&rf);
        FD_SET(ls, &rf);
        if (uls >= 0) FD_SET(uls, &rf);
        timeval tv{0, 200000};
        int r = select(std::max(ls, uls) + 1, &rf, nullptr, nullptr, &tv);
        if (r <= 0) continue;
        for (int l : {ls, uls}) {
            if (l < 0 || !FD_ISSET(l, &rf)) continue;
            int c = accept(l, nullptr, nullptr);
            if (c >= 0) conns.emplace_back(serve, c);
        }
    }
    for (auto& t : conns) t.join();
    timer.join();
    if (sampler.joinable()) sampler.join();
    close(ls);
    if (uls >= 0) { close(uls); unlink(unix_path.c_str()); }
    if (!snap_path.empty()) {
        std::lock_guard<std::mutex> g(mu);
        std::ofstream out(snap_path);
        out << core.snapshot_json() << "\n";
        fprintf(stderr, "fabricd: snapshot written to %s\n", snap_path.c_str());
    }
    if (log) fclose(log);
    return 0;
}
