// Device-side building blocks shared by all sm_100a kernels: timers, bounded
// waits, system-scope loads/stores, mbarrier / TMA / tcgen05 wrappers.
//
// Every wait here is bounded. A wait that runs out returns false; the caller
// records a status word and returns normally, so a late or dead peer never
// leaves a kernel spinning on a shared GPU.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "common_host.h"
#include "credit_page.h"

namespace sky {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u32(unsigned int* p, unsigned int v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Arrival without its own fence. Use after ONE __threadfence_system() when several peers are notified: a release
// per peer would serialise one system-scope fence (a round trip over NVLink) per arrival.
__device__ __forceinline__ void red_relaxed_sys_add_u32(unsigned int* p, unsigned int v) {
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 16-byte streaming load that does not pollute L1, and plain 16-byte store.
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 16-byte store through a multicast address: NVSwitch writes it into every bound GPU's memory.
__device__ __forceinline__ void multimem_st_v4(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_cs_v4(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Waits until *flag >= want (acquire, system scope) or `timeout_ns` passes.
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int want, unsigned long long timeout_ns) {
    // Poll relaxed; once the value is there, read it once more with acquire semantics. That load is what orders the reads
    // that follow behind the producer's release, and unlike a system-scope fence it does not have to wait for this SM's own
    // outstanding writes.
    // The first look is the acquire load itself: when the value is already there (the common case for a kernel that starts
    // after its producers), one round trip instead of two.
    if ((int)(ld_acquire_sys_u32(flag) - want) >= 0) return true;
    unsigned long long t0 = globaltimer_ns();
    unsigned ns = 32;
    for (;;) {
        if ((int)(ld_sys_u32(flag) - want) >= 0) return (int)(ld_acquire_sys_u32(flag) - want) >= 0;
        if (globaltimer_ns() - t0 > timeout_ns) return false;
        __nanosleep(ns);
        if (ns < 256) ns <<= 1;
    }
}

__device__ __forceinline__ void set_status(LaunchStatus* st, unsigned code, unsigned detail) {
    if (atomicCAS(&st->status, 0u, code) == 0u) st->detail = detail;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched with launch_pdl() may begin while the kernel before
// it in the stream is still draining; pdl_wait() blocks until that kernel has completed and its writes
// are visible, so it must come before the first read of anything an earlier kernel produced and before
// the first global write. pdl_trigger() lets the NEXT kernel's CTAs start as soon as every CTA of this
// kernel has called it (or exited); it does not publish any data.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Credit gate. One thread per CTA calls this per chunk.
//
// `need` is the cumulative byte count the flow will have consumed once this
// chunk is sent. The grant is read from the flow's credit page, which lives in
// mapped host memory and is written by the control side; the last value read is
// cached in *cache so that an unpaced or generously paced flow touches host
// memory only once in a while. Returns false when the deadline passed or the
// page's stop flag is set (then *stopped tells which).
constexpr unsigned long long SKY_UNLIMITED_RECHECK_BYTES = 256ull << 20;

__device__ __forceinline__ bool credit_acquire(const SkyCreditPage* page, unsigned long long need,
                                               unsigned long long* cache, unsigned long long max_wait_ns,
                                               unsigned long long* stall_ns, bool* stopped, bool* control_lost = nullptr) {
    *stopped = false;
    if (control_lost) *control_lost = false;
    if (page == nullptr) return true;
    if (need <= *cache) return true;
    unsigned long long t0 = globaltimer_ns();
    unsigned ns = 64;
    // Heartbeat: the control side bumps `epoch` every window. If it stays put for dead_after_windows windows while this
    // thread is waiting for credit, the control side is taken for dead and the page's dead_policy applies.
    const unsigned dead_windows = ld_sys_u32(&page->dead_after_windows);
    const unsigned long long dead_ns = dead_windows ? (unsigned long long)dead_windows * ld_sys_u64((const unsigned long long*)&page->window_ns) : 0ull;
    unsigned long long epoch0 = dead_ns ? ld_sys_u64((const unsigned long long*)&page->epoch) : 0ull, t_epoch = t0, t_dead = 0;
    // An earlier wait (this CTA's or another's) may have found the heartbeat stale at this very epoch already.
    bool dead = dead_ns && ld_sys_u64((const unsigned long long*)&page->heartbeat_lost) == epoch0 + 1;
    if (dead) t_dead = ld_sys_u64((const unsigned long long*)&page->heartbeat_lost_ns);
    for (;;) {
        if (ld_sys_u32(&page->stop)) { *stopped = true; *stall_ns += globaltimer_ns() - t0; return false; }
        // "unlimited" is not cached for the rest of the launch: the control side may start pacing this flow at any window, and a
        // launch can last many windows. The page is read again after SKY_UNLIMITED_RECHECK_BYTES more of the flow's bytes
        // (a fraction of a millisecond at link rate), which costs an unpaced flow one host-memory read per few chunks per CTA.
        if (ld_sys_u32(&page->unlimited)) { *cache = need + SKY_UNLIMITED_RECHECK_BYTES; break; }
        unsigned long long g = ld_sys_u64((const unsigned long long*)&page->granted_bytes);
        *cache = g;
        if (need <= g) break;
        const unsigned long long now = globaltimer_ns();
        if (dead_ns) {
            const unsigned long long e = ld_sys_u64((const unsigned long long*)&page->epoch);
            if (e != epoch0) { epoch0 = e; t_epoch = now; dead = false; }
            else if (!dead && now - t_epoch > dead_ns) {
                dead = true;
                t_dead = now;
                SkyCreditPage* w = const_cast<SkyCreditPage*>(page);
                st_sys_u64((unsigned long long*)&w->heartbeat_lost_ns, now);
                st_sys_u64((unsigned long long*)&w->heartbeat_lost, e + 1);
            }
            if (dead) {
                if (control_lost) *control_lost = true;
                const unsigned policy = ld_sys_u32(&page->dead_policy);
                if (policy == SKY_DEAD_UNPACED) { *cache = ~0ull; break; }
                if (policy == SKY_DEAD_STATIC) {
                    const unsigned long long w = max(1ull, ld_sys_u64((const unsigned long long*)&page->window_ns));
                    const unsigned long long self = g + (now > t_dead ? (now - t_dead) / w : 0ull) * ld_sys_u64((const unsigned long long*)&page->fallback_per_window);
                    if (need <= self) break;         // not cached: the next chunk asks again
                } else {
                    *stall_ns += now - t0;
                    return false;                    // SKY_DEAD_STALL
                }
            }
        }
        if (now - t0 > max_wait_ns) { *stall_ns += now - t0; return false; }
        __nanosleep(ns);
        if (ns < 8192) ns <<= 1;      // the page is in host memory: poll it gently
    }
    *stall_ns += globaltimer_ns() - t0;
    return true;
}

// ---------------------------------------------------------------------------
// mbarrier, TMA, tcgen05.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up once `timeout_ns` of wall time has passed (checked every 32 polls;
// a failed try_wait itself may block for a hardware-defined slice). Returns false on give-up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long timeout_ns = 200000000ull) {
    for (int i = 0; i < 32; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > timeout_ns) return false;
    }
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 2-D tiled TMA load, global -> shared, completion on an mbarrier. No cluster
// broadcast: one CTA, one destination.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const void* tmap, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate. One thread issues.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with A taken from TMEM: lane = row of A, 16-bit elements packed two per 32-bit column, K along the columns.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 consecutive fp32 columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile whose rows are 64
// elements (128 bytes) wide and stored with the 128-byte swizzle that a TMA
// box of inner extent 64 x bf16 produces: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                               // 128-byte swizzle
    return d;
}

// The same with a caller-given distance between the 8-row groups (tiles whose groups are not packed back to back).
__device__ __forceinline__ uint64_t umma_desc_k_sw128_sbo(uint32_t smem_addr, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Byte offset of element (row, col) in a [rows][64] bf16 tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128_off(int row, int col) {
    const int chunk = (col >> 3) ^ (row & 7);
    return (uint32_t)(row * 128 + chunk * 16 + (col & 7) * 2);
}

// MN-major operand, 128-byte swizzle: 64 contiguous elements along M per row, rows (K index) 128 bytes apart,
// 8-row groups `sbo` bytes apart, the next 64 elements of M `lbo` bytes away.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_x4(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr) : "memory");
}

// Split-KV combine of one output element: log-sum-exp merge of `n` partial results (running maximum m, sum l, value o),
// eight partials at a time so that their loads are in flight together (one L2 round trip per eight splits instead of
// one per split and array). part_o points at this thread's column of the first partial; partials are `o_pitch` floats apart.
__device__ __forceinline__ float combine_splits(const float* part_m, const float* part_l, const float* part_o, long long o_pitch, int n) {
    float mm = -INFINITY, ll = 0.f, oo = 0.f;
    for (int s0 = 0; s0 < n; s0 += 8) {
        float m8[8], l8[8], o8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool in = s0 + i < n;
            m8[i] = in ? __ldcg(part_m + s0 + i) : -INFINITY;
            l8[i] = in ? __ldcg(part_l + s0 + i) : 0.f;
            o8[i] = in ? __ldcg(part_o + (long long)(s0 + i) * o_pitch) : 0.f;
        }
        float cm = m8[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) cm = fmaxf(cm, m8[i]);
        const float nm = fmaxf(mm, cm);
        const float keep = mm == -INFINITY ? 0.f : exp2f(mm - nm);
        ll *= keep;
        oo *= keep;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float r = m8[i] == -INFINITY ? 0.f : exp2f(m8[i] - nm);
            ll += l8[i] * r;
            oo += o8[i] * r;
        }
        mm = nm;
    }
    return ll > 0.f ? oo / ll : 0.f;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}


// Host: launch with the programmatic-stream-serialization attribute (set SKYGDR_PDL=0 to launch plainly).
bool pdl_enabled();
// cluster_z > 1 launches thread-block clusters of that many CTAs along the grid's z dimension (gridDim.z must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    return launch_pdl_cluster(kernel, grid, block, smem, stream, 0, std::forward<Args>(args)...);
}

// Raises a kernel's dynamic shared memory limit once per device: the attribute belongs to the (function, device) pair, and one
// process may drive several GPUs. `done_mask` is a per-kernel static, one bit per device ordinal.
inline cudaError_t set_max_dynamic_smem_once(const void* func, int bytes, unsigned long long* done_mask) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (*done_mask & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) *done_mask |= bit;
    return e;
}

}  // namespace sky
