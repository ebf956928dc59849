// cpu_client: load generator and action end-point of one flow.
//
//   cpu_client <server_ip|-> <tcp_port> <fabric:tcp|sim[:gbps]> <iters> <msg_bytes> <op:write|read> <port> <gid_idx>
//              [qd=64] [span] [pattern:random|seq=random] [align=256] [mtu=1024] [sample=1] [max_samples=0]
//              [ts_ms=0] [ts_out=] [write_ack=1] [read_min_qd=16] [rd_atomic=0] [qps=1]
//
// Command line, environment (SKYGDR_CTRL_PORT, SKYGDR_CTRL_{HIGH,LOW,LOW2,LOW3,LOW4}_SLEEP_US,
// SKYGDR_CTRL_BIND_IP, SKYGDR_READ_MIN_QD, SKYGDR_RD_ATOMIC, SKYGDR_QPS), argument rules, exit codes, the
// per-window CSV and the three final lines follow the reference's client (src/cpu_client.cc:388-545,
// 805-823, 883-941, 1251-1296) so that its sweep and analysis tools keep working. The control port is the
// same one-command-per-connection listener (src/cpu_client.cc:238-315).
//
// What differs: the third argument names a fabric instead of an InfiniBand device. `tcp` moves the payload
// to gpu_server over the session socket; `sim[:gbps]` charges each message its service time on a simulated
// link (server_ip "-" then needs no server at all). And the flow can register with fabricd
// (SKYGDR_DAEMON=host:port, SKYGDR_FLOW_NAME/PRIORITY/TARGET_GBPS/LINK): it then obeys the byte grants of its
// credit page in addition to the legacy sleep pacing, and publishes its progress there.
#include <signal.h>
#include <sys/select.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <thread>
#include <vector>

#include "daemon_core.hpp"
#include "flow_client.hpp"
#include "protocol.hpp"
#include "util.hpp"
#include "wire.hpp"
#include "workload.hpp"

using namespace skygdr;

static std::atomic<int> g_shutdown{0};

static void control_server(ControlState* ctl, std::string bind_ip, int port) {
    int ls = tcp_listen(bind_ip, port, 16);
    if (ls < 0) { perror("[client] control listen"); return; }
    while (!g_shutdown.load()) {
        fd_set rf;
        FD_ZERO(&rf);
        FD_SET(ls, &rf);
        timeval tv{0, 200000};
        if (select(ls + 1, &rf, nullptr, nullptr, &tv) <= 0) continue;
        int c = accept(ls, nullptr, nullptr);
        if (c < 0) continue;
        timeval rto{1, 0};
        setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &rto, sizeof rto);
        char buf[256];
        ssize_t n = recv(c, buf, sizeof buf - 1, 0);
        if (n > 0) {
            buf[n] = 0;
            std::string rep = ctl->handle(buf);
            send_all(c, rep.data(), rep.size());
        }
        close(c);
    }
    close(ls);
}

static uint32_t env_u32(const char* name, uint32_t dflt) {
    const char* v = getenv(name);
    return v && *v ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

int main(int argc, char** argv) {
    if (argc < 9) {
        fprintf(stderr,
                "usage: %s <server_ip|-> <tcp_port> <fabric:tcp|sim[:gbps]> <iters> <msg_bytes> <op:write|read> <port> <gid_idx> "
                "[qd=64] [span] [pattern:random|seq] [align=256] [mtu=1024] [sample=1] [max_samples=0] [ts_ms=0] [ts_out=] "
                "[write_ack=1] [read_min_qd=16] [rd_atomic=0] [qps=1]\n", argv[0]);
        return 1;
    }
    const std::string server_ip = argv[1];
    const int tcp_port = atoi(argv[2]);
    const std::string fabric = argv[3];
    const uint64_t iters = strtoull(argv[4], nullptr, 10);
    uint64_t msg = 0, span = 0;
    if (!parse_size(argv[5], &msg)) { fprintf(stderr, "[client] bad msg_bytes\n"); return 2; }
    const bool is_read = std::string(argv[6]) == "read";
    auto arg = [&](int i, const char* d) { return argc > i ? argv[i] : d; };
    int qd = atoi(arg(9, "64"));
    if (argc > 10 && !parse_size(argv[10], &span)) { fprintf(stderr, "[client] bad span\n"); return 2; }
    const std::string pattern = arg(11, "random");
    uint64_t align = strtoull(arg(12, "256"), nullptr, 10);
    if (align == 0 || (align & (align - 1))) align = 256;
    const uint64_t sample = std::max<uint64_t>(1, strtoull(arg(14, "1"), nullptr, 10));
    const uint64_t max_samples = strtoull(arg(15, "0"), nullptr, 10);
    const int ts_ms = atoi(arg(16, "0"));
    const std::string ts_out = arg(17, "");
    int write_ack = atoi(arg(18, "1"));
    int read_min_qd = (int)env_u32("SKYGDR_READ_MIN_QD", (uint32_t)atoi(arg(19, "16")));
    int qps = (int)env_u32("SKYGDR_QPS", (uint32_t)atoi(arg(21, "1")));
    if (qps < 1) qps = 1;
    if (is_read) write_ack = 0;                          // reads are never acknowledged separately
    if (write_ack && qps > 1) qps = 1;                   // the ack path is single-connection
    if (is_read && qd < read_min_qd) qd = read_min_qd;

    // `sim[:GB/s]`: this process models the link itself (one client, no payload); `link`: the server models a link that all its
    // clients share (gpu_server link:<GB/s>), so this side only exchanges headers and tags; `tcp`: payload over the socket.
    const bool link = fabric.rfind("link", 0) == 0;
    const bool sim = link || fabric.rfind("sim", 0) == 0;
    double sim_gbps = 64.0;
    if (sim && !link && fabric.size() > 4) sim_gbps = atof(fabric.c_str() + 4);
    if (sim_gbps <= 0) sim_gbps = 64.0;

    // ---- control state ----
    ControlState ctl;
    const int ctrl_port = (int)env_u32("SKYGDR_CTRL_PORT", 0);
    {
        const char* l2 = getenv("SKYGDR_CTRL_LOW2_SLEEP_US");
        const char* l3 = getenv("SKYGDR_CTRL_LOW3_SLEEP_US");
        const char* l4 = getenv("SKYGDR_CTRL_LOW4_SLEEP_US");
        ctl.configure(env_u32("SKYGDR_CTRL_HIGH_SLEEP_US", 0), env_u32("SKYGDR_CTRL_LOW_SLEEP_US", 100),
                      l2 ? atol(l2) : -1, l3 ? atol(l3) : -1, l4 ? atol(l4) : -1);
    }
    std::thread ctl_thread;
    if (ctrl_port > 0 && ctrl_port < 65536) {
        ctl.enable();
        const char* bind_ip = getenv("SKYGDR_CTRL_BIND_IP");
        ctl_thread = std::thread(control_server, &ctl, std::string(bind_ip && *bind_ip ? bind_ip : "0.0.0.0"), ctrl_port);
    }
    auto finish = [&](int code) {
        g_shutdown.store(1);
        if (ctl_thread.joinable()) ctl_thread.join();
        return code;
    };

    // ---- session set-up ----
    int s = -1;
    RemoteInfo ri{0, 0, 1ull << 30};
    if (server_ip != "-") {
        s = tcp_connect(server_ip, tcp_port);
        if (s < 0) { perror("[client] connect"); return finish(1); }
        ConnInfo mine{}, peer{};
        mine.qpn = 1;
        ClientParams cp{(uint8_t)(is_read ? 0 : 1), (uint8_t)write_ack, 0, (uint32_t)qd, (uint32_t)qps};
        char ready = 0;
        bool ok = send_all(s, &mine, sizeof mine) && recv_all(s, &peer, sizeof peer) && recv_all(s, &ri, sizeof ri) &&
                  send_all(s, &cp, sizeof cp);
        for (int q = 1; ok && q < qps; ++q) ok = send_all(s, &mine, sizeof mine) && recv_all(s, &peer, sizeof peer);
        ok = ok && recv_all(s, &ready, 1);
        if (!ok) { fprintf(stderr, "[client] handshake failed\n"); return finish(1); }
    } else if (!sim) {
        fprintf(stderr, "[client] server_ip '-' needs the sim fabric\n");
        return finish(1);
    }
    if (msg == 0 || msg > ri.len) { fprintf(stderr, "[client] msg_bytes=%llu does not fit the remote region (%llu)\n",
                                            (unsigned long long)msg, (unsigned long long)ri.len); return finish(2); }
    if (span == 0 || span > ri.len) span = ri.len;
    if (span < msg) span = msg;

    // ---- optional registration with the daemon ----
    FlowClient fabric_client;
    SkyCreditPage* page = nullptr;
    if (const char* d = getenv("SKYGDR_DAEMON")) {
        if (fabric_client.connect(d)) {
            const char* nm = getenv("SKYGDR_FLOW_NAME");
            const char* pr = getenv("SKYGDR_FLOW_PRIORITY");
            const char* tg = getenv("SKYGDR_FLOW_TARGET_GBPS");
            std::string reply;
            const char* lk = getenv("SKYGDR_FLOW_LINK");
            if (fabric_client.register_flow(nm ? nm : "kv_offload", pr ? pr : "besteffort", tg ? atof(tg) : 0.0, "", &reply, lk ? lk : "")) {
                page = fabric_client.page();
                fprintf(stderr, "[client] registered with fabricd: %s", reply.c_str());
            } else {
                fprintf(stderr, "[client] registration refused: %s", reply.empty() ? "no answer\n" : reply.c_str());
            }
        } else {
            fprintf(stderr, "[client] SKYGDR_DAEMON=%s not reachable; running unregistered\n", d);
        }
    }

    // ---- buffers, samples, time series ----
    std::vector<unsigned char> buf(sim ? 0 : msg, 0x5a);
    std::vector<double> lat_us, lat_win;
    FILE* ts_fp = nullptr;
    if (ts_ms > 0) {
        ts_fp = (!ts_out.empty() && ts_out != "-") ? fopen(ts_out.c_str(), "w") : stdout;
        if (ts_fp) {
            fprintf(ts_fp, "ts_unix_ms,window_ms,window_us,ops,ops_per_s,throughput_gib_s,p50_us,p90_us,p99_us,p999_us,min_us,max_us,"
                           "samples,control_mode,pace_sleep_us,control_commands\n");
            fflush(ts_fp);
        } else fprintf(stderr, "[client] failed to open ts_out=%s\n", ts_out.c_str());
    }
    uint64_t completed = 0, win_completed0 = 0, seen = 0, seq_off = 0, consumed = 0;
    Rng rng(mono_ns() ^ (uint64_t)getpid());
    uint64_t t_start = mono_ns(), win_start = t_start;
    auto flush_window = [&](bool force) {
        if (!ts_fp) return;
        uint64_t now = mono_ns();
        uint64_t dt_us = (now - win_start) / 1000;
        if (!force && dt_us < (uint64_t)ts_ms * 1000) return;
        uint64_t ops = completed - win_completed0;
        if (ops == 0 && lat_win.empty()) { win_start = now; return; }
        std::sort(lat_win.begin(), lat_win.end());
        double sec = dt_us * 1e-6;
        fprintf(ts_fp, "%llu,%llu,%llu,%llu,%.6f,%.6f,%.3f,%.3f,%.3f,%.3f,%.3f,%.3f,%zu,%s,%u,%llu\n", (unsigned long long)unix_ms(),
                (unsigned long long)(dt_us / 1000), (unsigned long long)dt_us, (unsigned long long)ops, sec > 0 ? ops / sec : 0.0,
                sec > 0 ? double(ops) * double(msg) / kGiB / sec : 0.0, percentile_sorted(lat_win, 0.5), percentile_sorted(lat_win, 0.9),
                percentile_sorted(lat_win, 0.99), percentile_sorted(lat_win, 0.999), lat_win.empty() ? 0.0 : lat_win.front(),
                lat_win.empty() ? 0.0 : lat_win.back(), lat_win.size(), mode_name(ctl.mode()), ctl.sleep_us(),
                (unsigned long long)ctl.commands());
        fflush(ts_fp);
        lat_win.clear();
        win_start = now;
        win_completed0 = completed;
    };

    // ---- data loop ----
    // Two shapes, as in the reference: acknowledged writes keep one message in flight and wait for its ACK tag
    // (src/cpu_client.cc:1088-1249); reads and unacknowledged writes keep `qd` messages in flight per queue pair and
    // repost as completions come back (the steady-queue-depth loop, src/cpu_client.cc:943-1087). On the simulated
    // fabric the link serves one message at a time at its rate, so latency grows with the depth while throughput
    // stays at the link rate; over TCP the requests are pipelined on the connection.
    int rc = 0;
    SkyHeartbeatWatch heartbeat = {0, 0, 0};
    struct InFlight { uint64_t t_post, t_link_done, len; uint32_t tag; };
    std::deque<InFlight> in_flight;
    const size_t depth = write_ack ? 1 : (size_t)std::max(1, qd) * (size_t)qps;
    uint64_t link_free = mono_ns(), bytes_done = 0;
    auto account = [&](const InFlight& f, uint64_t t_done) {
        ++completed;
        bytes_done += f.len;
        if (page) { page->completed_bytes += f.len; page->last_ts_ns = t_done; }
        if ((seen++ % sample) == 0) {
            double us = (t_done - f.t_post) * 1e-3;
            if (max_samples == 0 || lat_us.size() < max_samples) lat_us.push_back(us);
            lat_win.push_back(us);
        }
    };
    auto complete_oldest = [&]() -> bool {
        InFlight f = in_flight.front();
        in_flight.pop_front();
        if (s >= 0) {
            if (is_read && !sim) { if (!recv_all(s, buf.data(), f.len)) { rc = 4; return false; } }
            else if (is_read || write_ack) {
                uint32_t tag = 0;
                if (!recv_all(s, &tag, 4)) { rc = 4; return false; }
                if (write_ack && tag != f.tag) { fprintf(stderr, "[client] unexpected ACK tag %u (want %u)\n", tag, f.tag); rc = 4; return false; }
            }
        }
        if (sim && !link) while (mono_ns() < f.t_link_done) { /* the link is still busy with this message */ }
        account(f, mono_ns());
        return true;
    };
    // One message of `len` bytes: credit gate, queue depth, post, (ACK), legacy pacing, window flush, lease renewal.
    auto issue = [&](uint64_t i, uint64_t len) -> bool {
        uint64_t off;
        if (pattern == "seq") { off = seq_off; seq_off += len; if (seq_off + len > span) seq_off = 0; }
        else off = span > len ? (uint64_t)(rng.uniform() * double(span - len)) : 0;
        off &= ~(align - 1);
        if (page) {                                      // byte grant of the flow, if it has one
            while (consumed + len > sky_host_allowance(page, &heartbeat, mono_ns()) && !page->stop && !ctl.stop_requested())
                std::this_thread::sleep_for(std::chrono::microseconds(50));
            if (page->stop) return false;
            consumed += len;
            page->consumed_bytes = consumed;
        }
        while (in_flight.size() >= depth && rc == 0) complete_oldest();
        if (rc) return false;
        InFlight f{mono_ns(), 0, len, (uint32_t)i};
        if (sim && !link) {
            const uint64_t service_ns = (uint64_t)(double(len) / (sim_gbps * 1e9) * 1e9);
            f.t_link_done = std::max(f.t_post, link_free) + service_ns;
            link_free = f.t_link_done;
        }
        if (s >= 0) {
            MsgHeader h{off, (uint32_t)len, (uint32_t)i, is_read ? 1u : 0u, 0};
            if (!send_all(s, &h, sizeof h)) { rc = 3; return false; }
            if (!sim && !is_read && !send_all(s, buf.data(), len)) { rc = 3; return false; }   // the payload of a write travels with it
        }
        in_flight.push_back(f);
        if (write_ack && !complete_oldest()) return false;   // acknowledged writes: wait for this one before the next
        uint32_t pace = ctl.sleep_us();                  // legacy pacing: sleep after each post
        if (pace) std::this_thread::sleep_for(std::chrono::microseconds(pace));
        flush_window(false);
        fabric_client.renew_if_due(mono_ns());
        return true;
    };

    // SKYGDR_REQUESTS=rate_per_s:lo_bytes:hi_bytes:seed:duration_s turns the flow into a request stream: Poisson arrivals of
    // requests with uniform sizes, each sent as messages of at most msg_bytes in arrival order; the flow time of a request
    // runs from its arrival to its last completion. Without it the flow is backlogged for `iters` messages, as in the reference.
    std::vector<double> flow_ms;
    size_t n_requests = 0, unfinished = 0;
    const char* req_env = getenv("SKYGDR_REQUESTS");
    if (req_env && *req_env) {
        double rate = 20, lo = 50e6, hi = 500e6, dur = 10;
        unsigned long long seed = 0;
        if (sscanf(req_env, "%lf:%lf:%lf:%llu:%lf", &rate, &lo, &hi, &seed, &dur) < 5 || rate <= 0 || hi < lo || dur <= 0) {
            fprintf(stderr, "[client] SKYGDR_REQUESTS wants rate:lo_bytes:hi_bytes:seed:duration_s\n");
            return finish(2);
        }
        const std::vector<Arrival> arr = poisson_uniform(seed, rate, dur, lo, hi);
        n_requests = arr.size();
        struct Req { uint64_t remaining, t_arrival; };
        std::deque<Req> q;
        size_t next = 0;
        uint64_t i = 0, backlog = 0;
        const uint64_t t_base = mono_ns();
        while (!ctl.stop_requested() && rc == 0) {
            const uint64_t now = mono_ns();
            while (next < arr.size() && t_base + (uint64_t)(arr[next].t_s * 1e9) <= now) {
                q.push_back({arr[next].bytes, t_base + (uint64_t)(arr[next].t_s * 1e9)});
                backlog += arr[next].bytes;
                ++next;
            }
            if (page) page->backlog_bytes = backlog;
            if (q.empty()) {
                if (next >= arr.size()) break;
                const uint64_t wait_ns = t_base + (uint64_t)(arr[next].t_s * 1e9) - now;
                std::this_thread::sleep_for(std::chrono::nanoseconds(std::min<uint64_t>(wait_ns, 200000)));
                continue;
            }
            const uint64_t len = std::min<uint64_t>(msg, q.front().remaining);
            if (!issue(i++, len)) break;
            while (!in_flight.empty() && rc == 0 && q.front().remaining <= len) complete_oldest();   // the request ends with this message
            q.front().remaining -= len;
            backlog -= len;
            if (q.front().remaining == 0) {
                flow_ms.push_back((mono_ns() - q.front().t_arrival) * 1e-6);
                q.pop_front();
            }
        }
        unfinished = q.size() + (arr.size() - next);
        if (page) page->backlog_bytes = 0;
    } else {
        for (uint64_t i = 0; i < iters && !ctl.stop_requested() && rc == 0; ++i) {
            if (page) page->backlog_bytes = (iters - i) * msg;
            if (!issue(i, msg)) break;
        }
        if (page) page->backlog_bytes = 0;
    }
    while (!in_flight.empty() && rc == 0) complete_oldest();       // drain what is still in flight
    double sec = (mono_ns() - t_start) * 1e-9;
    flush_window(true);
    if (ts_fp && ts_fp != stdout) fclose(ts_fp);
    printf("[client] done: iters=%llu msg=%llu qd=%d qps=%d span=%llu pattern=%s\n", (unsigned long long)iters, (unsigned long long)msg, qd,
           qps, (unsigned long long)span, pattern.c_str());
    printf("[client] elapsed=%.3f s  ops=%.0f ops/s  throughput=%.2f GiB/s\n", sec, sec > 0 ? completed / sec : 0.0,
           sec > 0 ? double(bytes_done) / kGiB / sec : 0.0);
    if (n_requests) {
        std::sort(flow_ms.begin(), flow_ms.end());
        double mean = 0;
        for (double v : flow_ms) mean += v;
        printf("[client] requests=%zu finished=%zu unfinished=%zu flow_time_ms p50=%.3f p99=%.3f mean=%.3f\n", n_requests, flow_ms.size(),
               unfinished, percentile_sorted(flow_ms, 0.5), percentile_sorted(flow_ms, 0.99), flow_ms.empty() ? 0.0 : mean / flow_ms.size());
    }
    if (ctl.stop_requested()) printf("[client] control_stop=1 mode=%s pace_sleep_us=%u\n", mode_name(ctl.mode()), ctl.sleep_us());
    if (!lat_us.empty()) {
        std::sort(lat_us.begin(), lat_us.end());
        printf("[client] latency_us samples=%zu p50=%.3f p90=%.3f p99=%.3f p999=%.3f min=%.3f max=%.3f\n", lat_us.size(),
               percentile_sorted(lat_us, 0.5), percentile_sorted(lat_us, 0.9), percentile_sorted(lat_us, 0.99),
               percentile_sorted(lat_us, 0.999), lat_us.front(), lat_us.back());
    } else printf("[client] latency_us samples=0\n");
    fflush(stdout);
    if (s >= 0) { MsgHeader h{0, 0, 0, 2, 0}; send_all(s, &h, sizeof h); close(s); }
    fabric_client.unregister();
    page = nullptr;
    fabric_client.close();
    return finish(rc);
}
