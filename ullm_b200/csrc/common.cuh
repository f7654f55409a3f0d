// Shared definitions for the sm_100a kernels: block geometry of the on-disk
// formats, small device helpers, and the TMA-bulk / mbarrier wrappers (every
// wait is bounded: after a fixed number of polls the kernel records a status
// word and leaves instead of spinning forever).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ullm {

// Block geometry (crates/ullm-core/src/dtype.rs:55-82).
constexpr int QK_K = 256;
constexpr int Q4K_BYTES = 144; // f16 d @0, f16 dmin @2, u8 scales[12] @4, u8 qs[128] @16
constexpr int Q6K_BYTES = 210; // u8 ql[128] @0, u8 qh[64] @128, i8 scales[16] @192, f16 d @208

// FMT_Q6KR is the prepared form of Q6_K used by resident weight objects: the same
// 210 bytes per super-block, re-ordered per row so that every access is an aligned
// 128-bit load and three of every four 6-bit values need one mask (prepare.cu).
enum Fmt : int { FMT_Q4K = 0, FMT_Q6K = 1, FMT_MLX4 = 2, FMT_Q6KR = 3 };

// Device-side status word values (kept in a per-context int in global memory).
constexpr int DEV_OK = 0;
constexpr int DEV_TIMEOUT = 1;

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }

// The 6-bit (scale, min) pair j of a k-quant super-block
// (crates/ullm-core/src/dequant.rs:41-49).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier + 1-D bulk (TMA) copies --------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller must leave) when the phase did
// not complete within the poll limit.  try_wait itself blocks for a
// hardware-defined slice, so the limit corresponds to far more than any
// legitimate wait here (a DRAM read of a few KB).
constexpr uint32_t MBAR_POLL_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < MBAR_POLL_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Global -> shared bulk copy, completion counted in bytes on `bar`.  Source,
// destination and size must all be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Asks the L2 to fetch `bytes` (a multiple of 16, 16-byte aligned) from global memory: no destination, no completion.
// (The tile ring in shared memory holds two to three tiles, which bounds the bytes a CTA can have in flight from
// DRAM; prefetching the tiles after those into the L2 is the obvious way around that bound - see the note at its
// one use for what it measured.)
__device__ __forceinline__ void bulk_prefetch_l2(const void *gsrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}

// Programmatic dependent launch: lets the next kernel in the stream start its
// prologue early / wait for the previous kernel's results.
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int dp4a_su(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a_u8x4, uint32_t b_u8x4, int c) {
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_u8x4), "r"(c));
    return d;
}

} // namespace ullm
