// Device side of the row-sharded output exchange: stores into every rank's gather buffer and the
// publish / bounded-wait protocol on the ranks' control blocks (see ShardDev in kernels.h).
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace ullm {

__device__ __forceinline__ unsigned long long shard_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Relaxed system-scope accesses to the step words; the ordering comes from ONE system-scope fence before the
// stores of a publication and one after the last load of a wait (a release store / acquire load per word would
// each carry a fence of its own: one per rank, in series, on the step's critical path).
__device__ __forceinline__ unsigned shard_ld_relaxed_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void shard_st_relaxed_sys(unsigned *p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One value to the same place in every rank's gather buffer (`addr` is the place in this rank's).
// Plain stores: the peers' buffers are mapped into this GPU's address space; nothing is read remotely.
__device__ __forceinline__ void shard_store_all(const ShardDev &sh, float *addr, float v) {
    for (int r = 0; r < sh.world; ++r) *(float *)((char *)addr + sh.delta[r]) = v;
}

// Waits until every rank has published exchange `step` (wrap-around safe); false when the time limit ran out.
__device__ __forceinline__ bool shard_wait_all(const ShardDev &sh, unsigned step) {
    const unsigned long long t0 = shard_now_ns();
    for (int r = 0; r < sh.world; ++r) {
        const unsigned *f = sh.ctl + r * SHARD_CTL_STRIDE;
        for (;;) {
            if ((int)(shard_ld_relaxed_sys(f) - step) >= 0) break;
            asm volatile("nanosleep.u32 32;" ::: "memory");
            if (shard_now_ns() - t0 > sh.timeout_ns) return false;
        }
    }
    __threadfence_system(); // acquire: the ranks' rows, stored before their publications, are visible from here on
    return true;
}

// Called by ONE thread of the launch, once every store of the exchange happens-before it (see
// shard_cta_done): counts the exchange, tells every rank, and waits for theirs when asked to.
// Returns false when the wait ran out of time.
__device__ __forceinline__ bool shard_publish(const ShardDev &sh) {
    // System-scope fence: the other CTAs' stores into the peers' buffers were ordered before their
    // arrival (gpu scope), this thread has observed every arrival, and fences are cumulative - so all
    // of those stores are ordered before the release stores below, as seen from the other GPUs.
    unsigned *stepw = sh.ctl + SHARD_CTL_STEP;
    const unsigned step = *(volatile unsigned *)stepw + 1u; // touched by one thread per launch; launches are stream-ordered
    __threadfence_system();                                 // (the load above is in flight while the fence drains)
    *(volatile unsigned *)stepw = step;
    for (int r = 0; r < sh.world; ++r) shard_st_relaxed_sys(sh.peer_flag[r], step);
    return sh.wait ? shard_wait_all(sh, step) : true;
}

// Called by one thread per CTA once the CTA's stores have been issued and a CTA-wide barrier has
// passed.  The last CTA of the grid to arrive publishes.  `aborted`: this CTA gave up on a bounded
// wait, its rows are missing, so the exchange must not be published.  One atomic per CTA: the low
// 16 bits of the word count arrivals, the high bits count aborted CTAs.
// Returns false only in the publishing thread, when its wait for the other ranks ran out of time.
__device__ __forceinline__ bool shard_cta_done(const ShardDev &sh, bool aborted) {
    unsigned *done = sh.ctl + SHARD_CTL_DONE;
    __threadfence(); // this CTA's stores (the barrier made them this thread's business) before its arrival
    const unsigned old = atomicAdd(done, aborted ? 0x10001u : 1u);
    if ((old & 0xffffu) != gridDim.x * gridDim.y * gridDim.z - 1) return true;
    *(volatile unsigned *)done = 0u; // for the next launch, which the stream orders after this one
    if ((old >> 16) != 0u || aborted || !sh.signal) return true;
    return shard_publish(sh);
}

// ---- tagged exchange (see ShardDev::tagged) ----
// An aligned 8-byte store / load is one access, so a pair is never seen half written (what NCCL's LL protocol
// relies on as well); volatile keeps both out of the L1.
__device__ __forceinline__ void shard_st_pair(uint2 *p, float v, unsigned step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(step) : "memory");
}
__device__ __forceinline__ uint2 shard_ld_pair(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// The step this launch belongs to: one more than the rank has completed.  Read by every thread that needs it
// before its CTA arrives; the word changes only after every CTA of the launch has arrived.
__device__ __forceinline__ unsigned shard_this_step(const ShardDev &sh) { return *(volatile unsigned *)(sh.ctl + SHARD_CTL_STEP) + 1u; }
// Polls (bounded) the pair of gather-buffer float e for `step`; false when the time limit ran out.
__device__ __forceinline__ bool shard_take_pair(const ShardDev &sh, unsigned step, size_t e, unsigned long long t0) {
    const uint2 *slot = sh.pairs + (size_t)(step & 1u) * sh.pair_floats + e;
    for (unsigned spin = 0;; ++spin) {
        const uint2 v = shard_ld_pair(slot);
        if (v.y == step) {
            sh.ybase[e] = __uint_as_float(v.x);
            return true;
        }
        if ((spin & 63u) == 63u && shard_now_ns() - t0 > sh.timeout_ns) return false;
    }
}
// End of a tagged launch, one thread per CTA after a CTA-wide barrier: counts the CTA in; the last one completes
// the step (step word, and the ranks' flag words so that the flag protocol of other entry points stays in
// step).  `failed`: this CTA gave up on a bounded wait: the step is not completed.
__device__ __forceinline__ void shard_cta_done_tagged(const ShardDev &sh, unsigned step, bool failed) {
    unsigned *done = sh.ctl + SHARD_CTL_DONE;
    const unsigned old = atomicAdd(done, failed ? 0x10001u : 1u);
    if ((old & 0xffffu) != gridDim.x * gridDim.y * gridDim.z - 1) return;
    *(volatile unsigned *)done = 0u;
    if ((old >> 16) != 0u || failed) return;
    *(volatile unsigned *)(sh.ctl + SHARD_CTL_STEP) = step;
    for (int r = 0; r < sh.world; ++r) shard_st_relaxed_sys(sh.peer_flag[r], step);
}

} // namespace ullm
