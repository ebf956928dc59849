// Wire structs of the flow set-up handshake and socket helpers, shared by cpu_client and gpu_server.
//
// The three fixed structs are the reference's (src/cpu_client.cc:317-324, 646-651, 722-729 and the
// identical definitions in src/gpu_server.cu:123-139, 317-322); the client always sends first. Over
// RDMA they carried QP numbers, GIDs and an rkey; on the TCP and simulated fabrics of this build the
// same bytes are exchanged (qpn = a connection serial, gid = zero, rkey = a session key), so a tool
// that speaks the reference's handshake finds the same sizes and order.
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>

namespace skygdr {

struct ConnInfo { uint32_t qpn; uint8_t gid[16]; uint8_t port; uint8_t gid_idx; uint16_t pad; };
struct RemoteInfo { uint32_t rkey; uint64_t addr; uint64_t len; };          // naturally aligned: 24 bytes
struct ClientParams { uint8_t op; uint8_t write_ack; uint16_t pad; uint32_t qd; uint32_t qps; };
static_assert(sizeof(ConnInfo) == 24 && sizeof(RemoteInfo) == 24 && sizeof(ClientParams) == 12, "wire layout");

// Per-message header on the TCP fabric: what an RDMA work request carries (remote offset, length,
// immediate). kind: 0 = write, 1 = read request, 2 = done.
struct MsgHeader { uint64_t offset; uint32_t len; uint32_t tag; uint32_t kind; uint32_t pad; };

inline bool send_all(int fd, const void* p, size_t n) {
    const char* c = (const char*)p;
    while (n) {
        ssize_t k = send(fd, c, n, MSG_NOSIGNAL);
        if (k <= 0) return false;
        c += k; n -= (size_t)k;
    }
    return true;
}
inline bool recv_all(int fd, void* p, size_t n) {
    char* c = (char*)p;
    while (n) {
        ssize_t k = recv(fd, c, n, 0);
        if (k <= 0) return false;
        c += k; n -= (size_t)k;
    }
    return true;
}
inline int tcp_connect(const std::string& ip, int port) {
    int s = socket(AF_INET, SOCK_STREAM, 0);
    if (s < 0) return -1;
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1 || connect(s, (sockaddr*)&a, sizeof a) != 0) { close(s); return -1; }
    int yes = 1;
    setsockopt(s, IPPROTO_TCP, TCP_NODELAY, &yes, sizeof yes);
    return s;
}
inline int tcp_listen(const std::string& ip, int port, int backlog) {
    int ls = socket(AF_INET, SOCK_STREAM, 0);
    if (ls < 0) return -1;
    int yes = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &yes, sizeof yes);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1) { close(ls); return -1; }
    if (bind(ls, (sockaddr*)&a, sizeof a) != 0 || listen(ls, backlog) != 0) { close(ls); return -1; }
    return ls;
}

}  // namespace skygdr
