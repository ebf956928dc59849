// Definitions shared by device code and by host code that never sees nvcc.
#pragma once

namespace sky {

// Per-launch status block in device memory. The host sets it to "unset"
// (status 0, cursor and t_start all ones) before a launch and reads it after.
struct LaunchStatus {
    unsigned int status;            // SkyStatus; first non-OK code wins
    unsigned int detail;            // code-specific (chunk index low bits, barrier id, ...)
    unsigned long long cursor;      // smallest chunk index NOT done; ~0ull = everything done
    unsigned long long chunks_done;
    unsigned long long bytes_done;
    unsigned long long stall_ns;    // summed over CTAs: time waiting for credit
    unsigned long long t_start_ns;  // globaltimer of the first CTA to start
    unsigned long long t_end_ns;    // globaltimer of the last CTA to finish
    unsigned int ctas_done;
    unsigned int work_counter;      // dynamic chunk scheduler
};

}  // namespace sky
