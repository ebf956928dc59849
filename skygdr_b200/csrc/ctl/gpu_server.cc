// gpu_server: the target end of a flow. Exposes a memory region, serves clients one after another,
// and acknowledges a write only after its bytes are in place.
//
//   gpu_server <fabric:tcp|gpu[:device]|sim|link:GB/s> <mr_size> <tcp_port> <port> <gid_idx> [mtu=1024]
//
// Same command line and session order as the reference's server (src/gpu_server.cu:8,215-530:
// handshake, region info, client parameters, ready byte, then either idle until "done" or the
// write-with-ack loop with a 4-byte ACK per tag). The reference registers cudaMalloc'd memory with
// an RNIC and must flush GPUDirect writes before the ACK (:54-80,426-436); here the first argument
// names the fabric instead of an InfiniBand device: `tcp` receives the payload on the session socket
// into the region (the ACK follows the last byte, so it has the same meaning), `sim` moves no payload.
// `gpu[:device]` is `tcp` with the region in that GPU's memory, as in the reference: the payload arrives in pinned staging
// buffers and goes on with asynchronous copies (one chunk in flight while the next is received), and the ACK is sent only
// after the stream has drained, that is, once the bytes are visible in device memory: the counterpart of the reference's
// cudaDeviceFlushGPUDirectRDMAWrites before its ACK. Reads come back the same way. The CUDA runtime is bound at run time
// (cuda_rt.hpp), so the program still builds and runs its other fabrics without one.
// `link:<GB/s>` is the shared-link form used by the CPU-only control-loop experiment: clients are served at the same
// time (a thread each) and every message occupies one simulated link of that rate for len / rate, first come first
// served, before its tag goes back, so concurrent flows really take bandwidth from one another.
// GPU-resident pools between processes are exposed by skygdr_b200.parallel.symm (CUDA IPC) instead.
#include <signal.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <thread>
#include <vector>

#include "cuda_rt.hpp"
#include "util.hpp"
#include "wire.hpp"

using namespace skygdr;

static volatile sig_atomic_t g_stop = 0;
static void on_sig(int) { g_stop = 1; }

int main(int argc, char** argv) {
    if (argc < 6) {
        fprintf(stderr, "usage: %s <fabric:tcp|gpu[:device]|sim|link:GB/s> <mr_size> <tcp_port> <port> <gid_idx> [mtu=1024]\n", argv[0]);
        return 1;
    }
    std::string fabric = argv[1];
    uint64_t mr_size = 0;
    if (!parse_size(argv[2], &mr_size) || mr_size == 0) { fprintf(stderr, "[server] bad mr_size\n"); return 2; }
    int tcp_port = atoi(argv[3]);
    bool sim = fabric.rfind("sim", 0) == 0 || fabric.rfind("link", 0) == 0;
    const bool gpu = fabric.rfind("gpu", 0) == 0;
    std::vector<unsigned char> region;
    if (!sim && !gpu) region.resize(mr_size);
    // gpu fabric: device region, two pinned staging buffers, one stream
    CudaRt rt;
    unsigned char* d_region = nullptr;
    unsigned char* stage[2] = {nullptr, nullptr};
    void* stream = nullptr;
    const size_t kStage = 4u << 20;
    if (gpu) {
        const int device = fabric.size() > 4 ? atoi(fabric.c_str() + 4) : 0;
        const std::string why = rt.load();
        if (!why.empty()) { fprintf(stderr, "[server] gpu fabric unavailable: %s\n", why.c_str()); return 1; }
        int e = rt.SetDevice(device);
        if (!e) e = rt.Malloc((void**)&d_region, mr_size);
        for (int i = 0; i < 2 && !e; ++i) e = rt.HostAlloc((void**)&stage[i], kStage, 0);
        if (!e) e = rt.StreamCreateWithFlags(&stream, 1 /* non-blocking */);
        if (e) { fprintf(stderr, "[server] gpu fabric set-up failed on device %d: %s\n", device, rt.err(e).c_str()); return 1; }
    }
    // Both return false on a socket or CUDA error. A staging buffer is reused every other chunk, so the stream is drained
    // before a buffer's second use; the final drain is what the ACK waits for.
    auto recv_to_device = [&](int c, uint64_t off, uint32_t len) {
        int k = 0;
        for (uint32_t done = 0; done < len; ++k) {
            const uint32_t n = (uint32_t)std::min<uint64_t>(kStage, len - done);
            if (k >= 2 && rt.StreamSynchronize(stream)) return false;
            if (!recv_all(c, stage[k & 1], n)) return false;
            if (rt.MemcpyAsync(d_region + off + done, stage[k & 1], n, CudaRt::kHostToDevice, stream)) return false;
            done += n;
        }
        return rt.StreamSynchronize(stream) == 0;
    };
    auto send_from_device = [&](int c, uint64_t off, uint32_t len) {
        for (uint32_t done = 0; done < len;) {
            const uint32_t n = (uint32_t)std::min<uint64_t>(kStage, len - done);
            if (rt.MemcpyAsync(stage[0], d_region + off + done, n, CudaRt::kDeviceToHost, stream) || rt.StreamSynchronize(stream)) return false;
            if (!send_all(c, stage[0], n)) return false;
            done += n;
        }
        return true;
    };
    struct sigaction sa{};
    sa.sa_handler = on_sig;
    sigaction(SIGINT, &sa, nullptr);
    sigaction(SIGTERM, &sa, nullptr);
    signal(SIGPIPE, SIG_IGN);
    int ls = tcp_listen("0.0.0.0", tcp_port, 1);
    if (ls < 0) { perror("[server] listen"); return 1; }
    printf("[server] fabric=%s mr_size=%llu listening on %d\n", fabric.c_str(), (unsigned long long)mr_size, tcp_port);
    fflush(stdout);
    std::atomic<uint32_t> serial{1};
    std::mutex link_mu;
    uint64_t link_free_ns = 0;
    const bool link = fabric.rfind("link", 0) == 0;
    double link_gbps = 64.0;
    if (link && fabric.size() > 5) link_gbps = atof(fabric.c_str() + 5);
    if (link_gbps <= 0) link_gbps = 64.0;
    auto occupy_link = [&](uint32_t len) {               // first come first served; returns when the message has left the link
        uint64_t t_done;
        {
            std::lock_guard<std::mutex> g(link_mu);
            const uint64_t now = mono_ns();
            t_done = std::max(now, link_free_ns) + (uint64_t)(double(len) / (link_gbps * 1e9) * 1e9);
            link_free_ns = t_done;
        }
        for (;;) {
            const uint64_t now = mono_ns();
            if (now >= t_done) break;
            if (t_done - now > 200000) std::this_thread::sleep_for(std::chrono::nanoseconds(t_done - now - 100000));
        }
    };
    auto serve = [&](int c) {
        int yes = 1;
        setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &yes, sizeof yes);
        ConnInfo peer{}, mine{};
        mine.qpn = serial++;
        RemoteInfo ri{0x5359u, 0, mr_size};
        ClientParams cp{};
        char ready = 1;
        bool ok = recv_all(c, &peer, sizeof peer) && send_all(c, &mine, sizeof mine) && send_all(c, &ri, sizeof ri) &&
                  recv_all(c, &cp, sizeof cp);
        for (uint32_t q = 1; ok && q < cp.qps; ++q) ok = recv_all(c, &peer, sizeof peer) && send_all(c, &mine, sizeof mine);
        ok = ok && send_all(c, &ready, 1);
        uint64_t msgs = 0, bytes = 0;
        while (ok && !g_stop) {
            MsgHeader h;
            if (!recv_all(c, &h, sizeof h)) break;
            if (h.kind == 2) break;                                  // client is done
            if (h.offset + h.len > mr_size) { fprintf(stderr, "[server] access outside the region\n"); break; }
            if (link) occupy_link(h.len);
            if (h.kind == 0) {                                       // write (+ optional ack)
                if (gpu) { if (!recv_to_device(c, h.offset, h.len)) break; }
                else if (!sim) { if (!recv_all(c, region.data() + h.offset, h.len)) break; }
                ++msgs; bytes += h.len;
                if (cp.write_ack) { uint32_t tag = h.tag; if (!send_all(c, &tag, 4)) break; }
            } else if (h.kind == 1) {                                // read: send the bytes back
                if (gpu) { if (!send_from_device(c, h.offset, h.len)) break; }
                else if (!sim) { if (!send_all(c, region.data() + h.offset, h.len)) break; }
                else { uint32_t tag = h.tag; if (!send_all(c, &tag, 4)) break; }
                ++msgs; bytes += h.len;
            }
        }
        printf("[server] session closed: msgs=%llu bytes=%llu op=%s write_ack=%u qd=%u qps=%u\n", (unsigned long long)msgs,
               (unsigned long long)bytes, cp.op ? "write" : "read", cp.write_ack, cp.qd, cp.qps);
        fflush(stdout);
        close(c);
    };
    while (!g_stop) {
        int c = accept(ls, nullptr, nullptr);
        if (c < 0) { if (g_stop) break; continue; }
        if (link) std::thread(serve, c).detach();        // shared link: clients at the same time
        else serve(c);                                   // the reference's order: one client after the other
    }
    close(ls);
    if (gpu) {
        rt.StreamDestroy(stream);
        rt.FreeHost(stage[0]);
        rt.FreeHost(stage[1]);
        rt.Free(d_region);
    }
    return 0;
}
