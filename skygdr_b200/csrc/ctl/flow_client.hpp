// Flow registration for native data paths: connect to fabricd, register a flow with a priority and a bandwidth goal,
// map its credit page, renew the lease, unregister. This is the client half of the protocol in daemon_core.hpp
// (REGISTER / RENEW / UNREGISTER); a data path then obeys the page: sky_host_allowance() on the host,
// credit_acquire() in a kernel (the page address must be registered with the CUDA runtime for that).
//
// The reference has no registration: a flow is whatever process listens on a control port
// (src/cpu_client.cc:238-315), and its goal lives in the policy script's flags
// (src/tools/pcie_case_study_controller.py:134-171).
#pragma once
#include <string>

#include "credit_page.h"
#include "daemon_core.hpp"
#include "wire.hpp"

namespace skygdr {

class FlowClient {
public:
    FlowClient() = default;
    FlowClient(const FlowClient&) = delete;
    FlowClient& operator=(const FlowClient&) = delete;
    ~FlowClient() { close(); }

    // "host:port" of fabricd. False when it cannot be reached.
    bool connect(const std::string& host_port) {
        const size_t colon = host_port.rfind(':');
        if (colon == std::string::npos) return false;
        sock_ = tcp_connect(host_port.substr(0, colon), atoi(host_port.c_str() + colon + 1));
        return sock_ >= 0;
    }
    bool connected() const { return sock_ >= 0; }

    // Registers the flow; on success flow_id() is set and page() is the mapped credit page (nullptr when the daemon keeps
    // its pages on the heap). `reply` receives the daemon's answer line either way.
    // `link` names the shared capacity the flow competes on (a link defined at the daemon); empty = the default link.
    bool register_flow(const std::string& name, const std::string& priority, double target_gbps, const std::string& kind, std::string* reply,
                       const std::string& link = "") {
        char line[320];
        const int n = snprintf(line, sizeof line, "REGISTER %s %s %g %s%s%s\n", name.c_str(), priority.c_str(), target_gbps,
                               kind.empty() ? name.c_str() : kind.c_str(), link.empty() ? "" : " link=", link.c_str());
        std::string rep;
        if (!request(std::string(line, (size_t)n), &rep)) return false;
        if (reply) *reply = rep;
        if (rep.rfind("OK", 0) != 0) return false;
        const size_t p1 = rep.find("flow_id="), p2 = rep.find("page="), p3 = rep.find("lease_ms="), p4 = rep.find("window_us=");
        if (p1 == std::string::npos) return false;
        flow_id_ = (uint32_t)strtoul(rep.c_str() + p1 + 8, nullptr, 10);
        if (p3 != std::string::npos) lease_ms_ = strtoull(rep.c_str() + p3 + 9, nullptr, 10);
        if (p4 != std::string::npos) window_us_ = strtoull(rep.c_str() + p4 + 10, nullptr, 10);
        if (p2 != std::string::npos) {
            const std::string path = rep.substr(p2 + 5, rep.find(' ', p2) - p2 - 5);
            if (path != "-") page_ = map_credit_page(path, false);
        }
        return true;
    }
    bool renew() {
        char line[64];
        const int n = snprintf(line, sizeof line, "RENEW %u\n", flow_id_);
        std::string rep;
        return flow_id_ && request(std::string(line, (size_t)n), &rep) && rep.rfind("OK", 0) == 0;
    }
    // Renews when a third of the lease has passed since the last renewal; cheap enough to call per message.
    void renew_if_due(uint64_t now_ns) {
        const uint64_t every = lease_ms_ ? lease_ms_ * 1000000ull / 3 : 500000000ull;
        if (sock_ >= 0 && now_ns - renewed_ns_ > every) { renew(); renewed_ns_ = now_ns; }
    }
    void unregister() {
        if (sock_ >= 0 && flow_id_) {
            char line[64];
            const int n = snprintf(line, sizeof line, "UNREGISTER %u\nQUIT\n", flow_id_);
            send_all(sock_, line, (size_t)n);
        }
        flow_id_ = 0;
    }
    void close() {
        if (page_) { unmap_credit_page(page_); page_ = nullptr; }
        if (sock_ >= 0) { ::close(sock_); sock_ = -1; }
    }
    uint32_t flow_id() const { return flow_id_; }
    SkyCreditPage* page() const { return page_; }
    uint64_t lease_ms() const { return lease_ms_; }
    uint64_t window_us() const { return window_us_; }

private:
    bool request(const std::string& line, std::string* reply) {
        if (sock_ < 0 || !send_all(sock_, line.data(), line.size())) return false;
        reply->clear();
        char c;
        while (reply->size() < 1024) {                 // one answer line
            const ssize_t k = recv(sock_, &c, 1, 0);
            if (k <= 0) return false;
            reply->push_back(c);
            if (c == '\n') return true;
        }
        return false;
    }
    int sock_ = -1;
    uint32_t flow_id_ = 0;
    uint64_t lease_ms_ = 0, window_us_ = 0, renewed_ns_ = 0;
    SkyCreditPage* page_ = nullptr;
};

}  // namespace skygdr
