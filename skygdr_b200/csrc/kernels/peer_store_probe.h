// Store-only probe of the SM write path into peer (or multicast) memory; see peer_store_probe.cu.
#pragma once
#include <cuda_runtime.h>

namespace sky {
// Writes `total_bytes` (rounded down to whole units per CTA) of `dst` `iters` times. mode 0: st.global.v4; mode 1:
// cp.async.bulk of `store_bytes` with `inflight` (1, 2, 4 or 8) groups outstanding per CTA; mode 2: multimem.st.v4 (dst is a
// multicast address). Returns after the launch; time it with events on `stream`.
cudaError_t launch_peer_store_probe(void* dst, unsigned long long total_bytes, int mode, unsigned store_bytes, int inflight, int ctas,
                                    int iters, cudaStream_t stream);
}  // namespace sky
