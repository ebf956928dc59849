// NVLink multicast region: one physical allocation on each GPU of a team, every one of them bound to a single
// multicast object. A store through the multicast address (`multimem.st`) leaves the issuing GPU once and NVSwitch
// delivers it into every member's allocation at the same offset; the unicast addresses reach one member's copy.
// The reference has no fan-out; its transfers are one cudaMemcpyPeerAsync per destination
// (llm_problem_analysis/kv_nvlink_transfer.cu:122).
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace sky {

struct MulticastRegion {
    std::vector<int> devices;                      // the team, in the caller's order
    size_t bytes = 0;                              // rounded up to the multicast granularity
    size_t granularity = 0;
    unsigned long long mc_handle = 0;
    std::vector<unsigned long long> mem_handles;   // per member
    std::vector<unsigned long long> unicast;       // address of member i's copy, readable and writable from every member
    unsigned long long multicast = 0;              // address whose stores land in every member's copy
    std::vector<char> bound;                       // per member: bound to the multicast object
};

// False with a reason when the driver or the device has no multicast support (no NVSwitch, old driver).
bool multicast_supported(int device, std::string* why);
// Single-process team: the calling process must be able to open every listed device. Throws std::runtime_error with the
// failing driver call's name and error string; what was built up to that point is taken down again first.
MulticastRegion* multicast_create(const std::vector<int>& devices, size_t bytes);
// Synchronises every member, then unmaps, unbinds and releases in that order. Safe on a partly built region.
void multicast_destroy(MulticastRegion* r);

}  // namespace sky
