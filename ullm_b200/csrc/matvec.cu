// Batch-1 quantized matvec  y[o] = sum_i W[o,i] * x[i]  for GGUF Q4_K / Q6_K
// super-blocks and MLX 4-bit affine groups, weights kept in their on-disk bytes
// (CPU form: crates/ullm-model/src/math.rs:9-33; GPU surface:
// crates/ullm-metal/src/forward.rs:639-673).
//
// Two kernels per format:
//
//  * streamed (the hot path).  A persistent CTA per SM walks row tiles.  One
//    producer thread streams each tile — R whole rows, a flat, contiguous,
//    16-byte-aligned byte range of the matrix — into a shared-memory ring with
//    1-D bulk (TMA) copies that complete on mbarriers, so tens of KB per SM stay
//    in flight without holding registers.  Consumer warps own a fixed column
//    group for the whole kernel: at start-up each lane re-expresses the slice of
//    x it will ever touch as 16-bit fixed point (lane-local scale = max|x| of the
//    8..32 values sharing one weight scale, split in a signed high and an
//    unsigned low byte plane) and keeps it in registers.  Per weight the inner
//    loop is then a mask and two dp4a: integer dot products are exact, and each
//    sub-block's integer sum is scaled by (weight scale * x scale) and
//    accumulated in fp32, min/bias terms use the exact fp32 sum of x.  The only
//    approximation is the 2^-16 relative rounding of x inside its group.
//    Rows are reduced with warp shuffles (transposed when a warp owns several
//    rows) and across column groups through shared memory.
//
//  * generic (fallback for shapes the streamed layout rules exclude): one warp
//    per row, direct global loads, fp32 FMA.
//
// Every wait on an mbarrier is bounded; on expiry the kernel sets the status
// word, stops computing and still walks its barriers so no warp is left behind.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>
#include <cmath>

namespace ullm {

// ---------------------------------------------------------------------------
// Shared unpack helpers
// ---------------------------------------------------------------------------

// Scale / min bytes of sub-blocks 2c and 2c+1 from the 12 packed bytes given as
// three little-endian words (same mapping as dequant.rs:41-49).
__device__ __forceinline__ void q4k_pair(uint32_t u0, uint32_t u1, uint32_t u2, int c, int &scA, int &mA, int &scB,
                                         int &mB) {
    uint32_t scw, mw;
    if (c < 2) {
        scw = u0 & 0x3f3f3f3fu;
        mw = u1 & 0x3f3f3f3fu;
    } else {
        scw = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
        mw = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
    }
    int sh = (c & 1) * 16;
    scA = (scw >> sh) & 0xff;
    scB = (scw >> (sh + 8)) & 0xff;
    mA = (mw >> sh) & 0xff;
    mB = (mw >> (sh + 8)) & 0xff;
}

template <typename T> __device__ __forceinline__ float tbl_load(const T *p);
template <> __device__ __forceinline__ float tbl_load<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float tbl_load<uint16_t>(const uint16_t *p) { return bf16_bits_to_f32(*p); }

// ---------------------------------------------------------------------------
// Generic kernels: one warp per row, fp32 math, no alignment demands beyond the
// natural one of each format (4 bytes for Q4_K / MLX words, 2 bytes for Q6_K).
// ---------------------------------------------------------------------------
template <int FMT, typename TBL>
__global__ void __launch_bounds__(256) matvec_generic_kernel(const uint8_t *__restrict__ w,
                                                            const TBL *__restrict__ scales,
                                                            const TBL *__restrict__ biases, int group,
                                                            const float *__restrict__ x, float *__restrict__ y,
                                                            size_t row0, size_t out_dim, size_t in_dim) {
    const int lane = threadIdx.x & 31;
    const size_t o = row0 + (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= out_dim) return;
    float acc = 0.f;
    if constexpr (FMT == FMT_Q4K) {
        const int nb = (int)(in_dim / QK_K);
        const uint8_t *row = w + o * (size_t)nb * Q4K_BYTES;
        const int c = lane >> 3;
        for (int b = 0; b < nb; ++b) {
            const uint32_t *blk = (const uint32_t *)(row + (size_t)b * Q4K_BYTES);
            uint32_t h0 = blk[0];
            float d = f16_bits_to_f32((uint16_t)(h0 & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(h0 >> 16));
            int scA, mA, scB, mB;
            q4k_pair(blk[1], blk[2], blk[3], c, scA, mA, scB, mB);
            uint32_t q = blk[4 + lane];
            const float *xp = x + (size_t)b * QK_K + 64 * c + 4 * (lane & 7);
            float4 xa = *(const float4 *)xp, xb = *(const float4 *)(xp + 32);
            float sa = (float)(q & 15) * xa.x + (float)((q >> 8) & 15) * xa.y + (float)((q >> 16) & 15) * xa.z +
                       (float)((q >> 24) & 15) * xa.w;
            float sb = (float)((q >> 4) & 15) * xb.x + (float)((q >> 12) & 15) * xb.y +
                       (float)((q >> 20) & 15) * xb.z + (float)(q >> 28) * xb.w;
            acc += d * ((float)scA * sa + (float)scB * sb) -
                   dmin * ((float)mA * (xa.x + xa.y + xa.z + xa.w) + (float)mB * (xb.x + xb.y + xb.z + xb.w));
        }
    } else if constexpr (FMT == FMT_Q6K) {
        const int nb = (int)(in_dim / QK_K);
        const uint8_t *row = w + o * (size_t)nb * Q6K_BYTES;
        const int sub = lane >> 4, r = lane & 15, nh = r >> 3, t = r & 7;
        for (int b0 = 0; b0 < nb; b0 += 2) {
            int b = b0 + sub;
            if (b >= nb) break;
            const uint8_t *blk = row + (size_t)b * Q6K_BYTES;
            const uint16_t *pa = (const uint16_t *)(blk + 64 * nh + 4 * t);
            const uint16_t *pb = (const uint16_t *)(blk + 64 * nh + 32 + 4 * t);
            const uint16_t *ph = (const uint16_t *)(blk + 128 + 32 * nh + 4 * t);
            uint32_t A = pa[0] | ((uint32_t)pa[1] << 16), B = pb[0] | ((uint32_t)pb[1] << 16),
                     H = ph[0] | ((uint32_t)ph[1] << 16);
            const int8_t *sc = (const int8_t *)(blk + 192) + 8 * nh + (t >> 2);
            float d = f16_bits_to_f32(*(const uint16_t *)(blk + 208));
            const float *xp = x + (size_t)b * QK_K + 128 * nh + 4 * t;
            float s = 0.f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t lo = (g & 1) ? B : A;
                if (g >= 2) lo >>= 4;
                uint32_t hi = (H >> (2 * g)) & 0x03030303u;
                uint32_t qv = (lo & 0x0f0f0f0fu) | (hi << 4);
                float4 xv = *(const float4 *)(xp + 32 * g);
                float part = (float)((int)(qv & 0xff) - 32) * xv.x + (float)((int)((qv >> 8) & 0xff) - 32) * xv.y +
                             (float)((int)((qv >> 16) & 0xff) - 32) * xv.z + (float)((int)(qv >> 24) - 32) * xv.w;
                s += (float)sc[2 * g] * part;
            }
            acc += d * s;
        }
    } else {
        const size_t words = in_dim / 8, groups = in_dim / (size_t)group;
        const uint32_t *row = (const uint32_t *)w + o * words;
        for (size_t wi = lane; wi < words; wi += 32) {
            uint32_t q = row[wi];
            size_t g = (wi * 8) / (size_t)group;
            float s = tbl_load<TBL>(scales + o * groups + g), bi = tbl_load<TBL>(biases + o * groups + g);
            const float *xp = x + wi * 8;
            float4 xa = *(const float4 *)xp, xb = *(const float4 *)(xp + 4);
            float dot = (float)(q & 15) * xa.x + (float)((q >> 4) & 15) * xa.y + (float)((q >> 8) & 15) * xa.z +
                        (float)((q >> 12) & 15) * xa.w + (float)((q >> 16) & 15) * xb.x +
                        (float)((q >> 20) & 15) * xb.y + (float)((q >> 24) & 15) * xb.z + (float)(q >> 28) * xb.w;
            acc += s * dot + bi * (xa.x + xa.y + xa.z + xa.w + xb.x + xb.y + xb.z + xb.w);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[o] = acc;
}

// ---------------------------------------------------------------------------
// Streamed kernels
// ---------------------------------------------------------------------------
constexpr int XREGS_Q4K = 36, XREGS_Q6K = 24, XREGS_MLX = 18;
template <int FMT> struct FmtTraits;
template <> struct FmtTraits<FMT_Q4K> { static constexpr int XREGS = XREGS_Q4K, CG_ELEMS = 2048; };
template <> struct FmtTraits<FMT_Q6K> { static constexpr int XREGS = XREGS_Q6K, CG_ELEMS = 1024; };
template <> struct FmtTraits<FMT_MLX4> { static constexpr int XREGS = XREGS_MLX, CG_ELEMS = 1024; };

struct StreamParams {
    const uint8_t *w;
    const uint8_t *scales, *biases; // MLX tables (bytes), else null
    const float *x;
    float *y;
    int *status;
    uint32_t out_dim, in_dim, group;
    uint32_t row_bytes, tbl_row_bytes;
    uint32_t R, WC, WR, NW, S;
    uint32_t w_stage_bytes, tbl_stage_bytes, stage_bytes; // regions inside one stage (128-B multiples)
    uint32_t ntiles, ncg;
    uint32_t off_part, off_prep, off_ring; // byte offsets in dynamic smem
};

// 16-bit fixed point of up to 32 values sharing one scale.  X = rint(v/s) with
// s = max|v|/32767; returned as byte planes: hi = X >> 8 (signed), lo = X & 255.
__device__ __forceinline__ int quant16(float v, float inv) {
    int q = __float2int_rn(v * inv);
    return max(-32767, min(32767, q));
}

// Fills the persistent register image of (column group cg, lane ln) at
// slot[k * 32] (k = 0..XREGS-1; the caller passes slot already offset by lane).
template <int FMT>
__device__ __forceinline__ void prep_slot(const float *__restrict__ x, uint32_t in_dim, uint32_t cg, uint32_t ln,
                                          uint32_t *slot) {
    constexpr int XR = FmtTraits<FMT>::XREGS;
    if constexpr (FMT == FMT_Q4K) {
        // lane: block 8cg + ln/4, chunk c = ln%4: low nibbles = elements [64c,64c+32),
        // high nibbles = [64c+32, 64c+64)   (dequant.rs:200-214)
        uint32_t e0 = cg * 2048u + (ln >> 2) * 256u + (ln & 3) * 64u;
        if (e0 >= in_dim) {
#pragma unroll
            for (int k = 0; k < XR; ++k) slot[k * 32] = 0u;
            return;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float v[32];
            const float4 *xp = (const float4 *)(x + e0 + 32 * half);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 t = __ldg(xp + i);
                v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
            }
            float mx = 0.f, sum = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(v[i])), sum += v[i];
            float inv = mx > 0.f ? 32767.f / mx : 0.f, s = mx * (1.f / 32767.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    int q = quant16(v[4 * j + k], inv);
                    hi |= (uint32_t)((q >> 8) & 0xff) << (8 * k);
                    lo |= (uint32_t)(q & 0xff) << (8 * k);
                }
                slot[(16 * half + j) * 32] = hi;
                slot[(16 * half + 8 + j) * 32] = lo;
            }
            // high nibbles are used in place (value * 16): fold the 1/16 here
            slot[(32 + half) * 32] = __float_as_uint(half ? s * 0.0625f : s);
            slot[(34 + half) * 32] = __float_as_uint(sum);
        }
    } else if constexpr (FMT == FMT_Q6K) {
        // lane: block 4cg + ln/8, half nh = (ln%8)/4, l0 = 8*(ln%4); group g = 0..3 is
        // the element range 128nh + 32g + l0 + [0,8)   (dequant.rs:264-279)
        uint32_t r = ln & 7;
        uint32_t e0 = cg * 1024u + (ln >> 3) * 256u + (r >> 2) * 128u + (r & 3) * 8u;
        if (e0 >= in_dim) {
#pragma unroll
            for (int k = 0; k < XR; ++k) slot[k * 32] = 0u;
            return;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float v[8];
            const float4 *xp = (const float4 *)(x + e0 + 32 * g);
            float4 t0 = __ldg(xp), t1 = __ldg(xp + 1);
            v[0] = t0.x, v[1] = t0.y, v[2] = t0.z, v[3] = t0.w, v[4] = t1.x, v[5] = t1.y, v[6] = t1.z, v[7] = t1.w;
            float mx = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[i]));
            float inv = mx > 0.f ? 32767.f / mx : 0.f, s = mx * (1.f / 32767.f);
            int isum = 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    int q = quant16(v[4 * j + k], inv);
                    isum += q;
                    hi |= (uint32_t)((q >> 8) & 0xff) << (8 * k);
                    lo |= (uint32_t)(q & 0xff) << (8 * k);
                }
                slot[(4 * g + j) * 32] = hi;
                slot[(4 * g + 2 + j) * 32] = lo;
            }
            slot[(16 + g) * 32] = __float_as_uint(s);
            slot[(20 + g) * 32] = (uint32_t)(32 * isum); // sum (q-32) X = sum q X - 32 sum X
        }
    } else {
        // lane: words 4*(32cg+ln) .. +3 = elements 32*(32cg+ln) + [0,32); nibble k of
        // word j is element 8j+k (dequant.rs:310-311).  Even nibbles are taken with
        // the mask 0x0f0f0f0f, odd ones in place (value*16) with 0xf0f0f0f0.
        uint32_t e0 = (cg * 32u + ln) * 32u;
        if (e0 >= in_dim) {
#pragma unroll
            for (int k = 0; k < XR; ++k) slot[k * 32] = 0u;
            return;
        }
        float v[32];
        const float4 *xp = (const float4 *)(x + e0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4 t = __ldg(xp + i);
            v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
        }
        float mx = 0.f, sum = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(v[i])), sum += v[i];
        float inv = mx > 0.f ? 32767.f / mx : 0.f, s = mx * (1.f / 32767.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t he = 0, le = 0, ho = 0, lo = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int qe = quant16(v[8 * j + 2 * k], inv), qo = quant16(v[8 * j + 2 * k + 1], inv);
                he |= (uint32_t)((qe >> 8) & 0xff) << (8 * k);
                le |= (uint32_t)(qe & 0xff) << (8 * k);
                ho |= (uint32_t)((qo >> 8) & 0xff) << (8 * k);
                lo |= (uint32_t)(qo & 0xff) << (8 * k);
            }
            slot[j * 32] = he, slot[(4 + j) * 32] = le, slot[(8 + j) * 32] = ho, slot[(12 + j) * 32] = lo;
        }
        slot[16 * 32] = __float_as_uint(s * 0.0625f);
        slot[17 * 32] = __float_as_uint(sum);
    }
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Partial dot product of one row with the lane's column slice.
//   row_addr : shared-memory byte address of the row inside the stage
//   X        : the lane's persistent register image (see prep_slot)
//   tbl_s/b  : MLX only — shared-memory byte addresses of this row's tables
template <int FMT, typename TBL>
__device__ __forceinline__ float row_partial(uint32_t row_addr, const uint32_t (&X)[FmtTraits<FMT>::XREGS], uint32_t cg,
                                             uint32_t ln, uint32_t tbl_s, uint32_t tbl_b, uint32_t group) {
    if constexpr (FMT == FMT_Q4K) {
        const uint32_t blk = row_addr + (cg * 8u + (ln >> 2)) * Q4K_BYTES;
        const int c = ln & 3;
        uint4 hdr = lds128(blk);
        uint4 qa = lds128(blk + 16 + 32 * c), qb = lds128(blk + 32 + 32 * c);
        const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        int ah = 0, al = 0, bh = 0, bl = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t lo = q[j] & 0x0f0f0f0fu, hi = q[j] & 0xf0f0f0f0u;
            ah = dp4a_su(lo, X[j], ah);
            al = dp4a_uu(lo, X[8 + j], al);
            bh = dp4a_su(hi, X[16 + j], bh);
            bl = dp4a_uu(hi, X[24 + j], bl);
        }
        int scA, mA, scB, mB;
        q4k_pair(hdr.y, hdr.z, hdr.w, c, scA, mA, scB, mB);
        float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
        float ia = (float)(ah * 256 + al), ib = (float)(bh * 256 + bl);
        float pos = (float)scA * __uint_as_float(X[32]) * ia + (float)scB * __uint_as_float(X[33]) * ib;
        float neg = (float)mA * __uint_as_float(X[34]) + (float)mB * __uint_as_float(X[35]);
        return d * pos - dmin * neg;
    } else if constexpr (FMT == FMT_Q6K) {
        const uint32_t blk = row_addr + (cg * 4u + (ln >> 3)) * Q6K_BYTES; // 2-byte aligned only
        const uint32_t r = ln & 7, nh = r >> 2, t = r & 3;
        const uint32_t sh = (blk & 2u) * 8u; // 0 or 16
        const uint32_t base = blk & ~3u;
        // three 8-byte streams, each read as three aligned words and funnel-shifted
        uint32_t pa = base + 64 * nh + 8 * t, pb = pa + 32, ph = base + 128 + 32 * nh + 8 * t;
        uint32_t a0 = lds32(pa), a1 = lds32(pa + 4), a2 = lds32(pa + 8);
        uint32_t b0 = lds32(pb), b1 = lds32(pb + 4), b2 = lds32(pb + 8);
        uint32_t h0 = lds32(ph), h1 = lds32(ph + 4), h2 = lds32(ph + 8);
        uint32_t A[2] = {__funnelshift_r(a0, a1, sh), __funnelshift_r(a1, a2, sh)};
        uint32_t B[2] = {__funnelshift_r(b0, b1, sh), __funnelshift_r(b1, b2, sh)};
        uint32_t H[2] = {__funnelshift_r(h0, h1, sh), __funnelshift_r(h1, h2, sh)};
        int acc_h[4] = {0, 0, 0, 0}, acc_l[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t q0 = (A[j] & 0x0f0f0f0fu) | ((H[j] << 4) & 0x30303030u);
            uint32_t q1 = (B[j] & 0x0f0f0f0fu) | ((H[j] << 2) & 0x30303030u);
            uint32_t q2 = ((A[j] >> 4) & 0x0f0f0f0fu) | (H[j] & 0x30303030u);
            uint32_t q3 = ((B[j] >> 4) & 0x0f0f0f0fu) | ((H[j] >> 2) & 0x30303030u);
            acc_h[0] = dp4a_su(q0, X[0 + j], acc_h[0]), acc_l[0] = dp4a_uu(q0, X[2 + j], acc_l[0]);
            acc_h[1] = dp4a_su(q1, X[4 + j], acc_h[1]), acc_l[1] = dp4a_uu(q1, X[6 + j], acc_l[1]);
            acc_h[2] = dp4a_su(q2, X[8 + j], acc_h[2]), acc_l[2] = dp4a_uu(q2, X[10 + j], acc_l[2]);
            acc_h[3] = dp4a_su(q3, X[12 + j], acc_h[3]), acc_l[3] = dp4a_uu(q3, X[14 + j], acc_l[3]);
        }
        // int8 scales 8nh + t/2 + 2g (dequant.rs:267, :275-278) and the f16 d at +208
        const uint32_t sca = blk + 192 + 8 * nh + (t >> 1);
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            int sc;
            asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sc) : "r"(sca + 2 * g));
            int isum = acc_h[g] * 256 + acc_l[g] - (int)X[20 + g];
            s += (float)sc * __uint_as_float(X[16 + g]) * (float)isum;
        }
        uint32_t dbits;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits) : "r"(blk + 208));
        return f16_bits_to_f32((uint16_t)dbits) * s;
    } else {
        const uint32_t widx = cg * 32u + ln; // 16-byte unit inside the row
        uint4 qw = lds128(row_addr + widx * 16u);
        const uint32_t q[4] = {qw.x, qw.y, qw.z, qw.w};
        int eh = 0, el = 0, oh = 0, ol = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t ev = q[j] & 0x0f0f0f0fu, od = q[j] & 0xf0f0f0f0u;
            eh = dp4a_su(ev, X[j], eh);
            el = dp4a_uu(ev, X[4 + j], el);
            oh = dp4a_su(od, X[8 + j], oh);
            ol = dp4a_uu(od, X[12 + j], ol);
        }
        int isum16 = 16 * (eh * 256 + el) + (oh * 256 + ol);
        uint32_t g = (widx * 32u) / group;
        float sc, bi;
        if constexpr (sizeof(TBL) == 4) {
            sc = __uint_as_float(lds32(tbl_s + 4 * g));
            bi = __uint_as_float(lds32(tbl_b + 4 * g));
        } else {
            uint32_t sb, bb;
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sb) : "r"(tbl_s + 2 * g));
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(bb) : "r"(tbl_b + 2 * g));
            sc = bf16_bits_to_f32((uint16_t)sb);
            bi = bf16_bits_to_f32((uint16_t)bb);
        }
        return sc * __uint_as_float(X[16]) * (float)isum16 + bi * __uint_as_float(X[17]);
    }
}

// Sums v[i] over the warp for i = 0..N-1 with a transposed butterfly: after the
// call every lane holds the complete sum of row `row_of_lane` (N=1: row 0;
// N=2: bit 4 of lane; N=4: bits 4,3 -> 2*b4 + b3).
template <int N> __device__ __forceinline__ float warp_reduce_rows(float (&v)[N], uint32_t lane, uint32_t &row_of_lane) {
    static_assert(N == 1 || N == 2 || N == 4, "rows per warp");
    float r;
    if constexpr (N == 1) {
        r = v[0];
        row_of_lane = 0;
        r += __shfl_xor_sync(0xffffffffu, r, 16);
        r += __shfl_xor_sync(0xffffffffu, r, 8);
    } else if constexpr (N == 2) {
        bool up = lane & 16;
        float send = up ? v[0] : v[1], keep = up ? v[1] : v[0];
        r = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        row_of_lane = up ? 1 : 0;
        r += __shfl_xor_sync(0xffffffffu, r, 8);
    } else {
        bool up = lane & 16;
        float s0 = up ? v[0] : v[2], s1 = up ? v[1] : v[3];
        float k0 = up ? v[2] : v[0], k1 = up ? v[3] : v[1];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
        k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
        bool up2 = lane & 8;
        float send = up2 ? k0 : k1, keep = up2 ? k1 : k0;
        r = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        row_of_lane = (up ? 2 : 0) + (up2 ? 1 : 0);
    }
    r += __shfl_xor_sync(0xffffffffu, r, 4);
    r += __shfl_xor_sync(0xffffffffu, r, 2);
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    return r;
}

__device__ __forceinline__ bool wait_or_timeout(uint64_t *bar, uint32_t parity) {
    // ~2^31 cycles (about a second) of polling before giving up
    long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) return false;
    }
}

template <int FMT, int RW, int G, typename TBL>
__global__ void __launch_bounds__(544, 1) matvec_stream_kernel(const StreamParams p) {
    constexpr int XR = FmtTraits<FMT>::XREGS;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + p.S;
    float *part = (float *)(smem + p.off_part);
    uint32_t *prep = (uint32_t *)(smem + p.off_prep);
    uint8_t *ring = smem + p.off_ring;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == p.NW;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    auto issue = [&](uint32_t tile, uint32_t s) {
        uint32_t r0 = tile * p.R;
        uint32_t rows = min(p.R, p.out_dim - r0);
        uint32_t wb = rows * p.row_bytes, tb = rows * p.tbl_row_bytes;
        uint8_t *dst = ring + (size_t)s * p.stage_bytes;
        mbar_arrive_expect_tx(&full[s], wb + 2 * tb);
        bulk_g2s(dst, p.w + (size_t)r0 * p.row_bytes, wb, &full[s]);
        if (FMT == FMT_MLX4) {
            bulk_g2s(dst + p.w_stage_bytes, p.scales + (size_t)r0 * p.tbl_row_bytes, tb, &full[s]);
            bulk_g2s(dst + p.w_stage_bytes + p.tbl_stage_bytes, p.biases + (size_t)r0 * p.tbl_row_bytes, tb, &full[s]);
        }
    };

    // Weights do not depend on the previous kernel in the stream: start the first
    // S tiles now, before waiting for it.
    if (producer && lane == 0) {
        uint32_t k = 0;
        for (uint32_t tile = blockIdx.x; tile < p.ntiles && k < p.S; tile += gridDim.x, ++k) issue(tile, k);
    }
    pdl_wait_prior();

    // x -> fixed-point register images, built once per CTA in shared memory
    for (uint32_t sl = tid; sl < p.ncg * 32u; sl += blockDim.x)
        prep_slot<FMT>(p.x, p.in_dim, sl >> 5, sl & 31u, prep + (size_t)(sl >> 5) * XR * 32 + (sl & 31u));
    __syncthreads();

    if (producer) {
        if (lane == 0) {
            uint32_t k = 0;
            for (uint32_t tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++k) {
                if (k < p.S) continue;
                uint32_t s = k % p.S;
                if (!wait_or_timeout(&empty[s], ((k / p.S) - 1) & 1)) {
                    *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                issue(tile, s);
            }
        }
        return;
    }

    const uint32_t rs = warp / p.WC, cgw = warp % p.WC;
    uint32_t X[G][XR];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        uint32_t cg = cgw + g * p.WC;
#pragma unroll
        for (int k = 0; k < XR; ++k) X[g][k] = cg < p.ncg ? prep[((size_t)cg * XR + k) * 32 + lane] : 0u;
    }

    bool aborted = false;
    uint32_t k = 0;
    for (uint32_t tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++k) {
        const uint32_t s = k % p.S;
        if (!aborted && !wait_or_timeout(&full[s], (k / p.S) & 1)) aborted = true;
        const uint32_t stage = smem_u32(ring + (size_t)s * p.stage_bytes);
        const uint32_t r0 = tile * p.R;
        float v[RW];
#pragma unroll
        for (int rr = 0; rr < RW; ++rr) {
            v[rr] = 0.f;
            const uint32_t rl = rs * RW + rr;
            if (!aborted && r0 + rl < p.out_dim) {
                const uint32_t row_addr = stage + rl * p.row_bytes;
                const uint32_t ts = stage + p.w_stage_bytes + rl * p.tbl_row_bytes;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const uint32_t cg = cgw + g * p.WC;
                    // lanes past the end of the row hold a zero register image but must
                    // not read beyond the stage
                    bool live = cg < p.ncg;
                    if (FMT == FMT_Q4K) live = live && (cg * 8u + (lane >> 2)) * QK_K < p.in_dim;
                    if (FMT == FMT_Q6K) live = live && (cg * 4u + (lane >> 3)) * QK_K < p.in_dim;
                    if (FMT == FMT_MLX4) live = live && (cg * 32u + lane) * 32u < p.in_dim;
                    if (live) v[rr] += row_partial<FMT, TBL>(row_addr, X[g], cg, lane, ts, ts + p.tbl_stage_bytes, p.group);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]); // stage may be refilled

        uint32_t myrow;
        float r = warp_reduce_rows<RW>(v, lane, myrow);
        const uint32_t rl = rs * RW + myrow;
        if (p.WC == 1) {
            if ((lane & 7) == 0 && (RW == 4 || (lane & 8) == 0) && r0 + rl < p.out_dim && !aborted) p.y[r0 + rl] = r;
        } else {
            float *pt = part + (size_t)(k & 1) * p.R * p.WC;
            if ((lane & 7) == 0 && (RW == 4 || (lane & 8) == 0)) pt[rl * p.WC + cgw] = r;
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rs), "r"(p.WC * 32) : "memory");
            const uint32_t sl = cgw * 32 + lane;
            if (sl < RW) {
                const uint32_t row = rs * RW + sl;
                float acc = 0.f;
                for (uint32_t c = 0; c < p.WC; ++c) acc += pt[row * p.WC + c];
                if (r0 + row < p.out_dim && !aborted) p.y[r0 + row] = acc;
            }
        }
    }
    if (aborted && lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
}

// ---------------------------------------------------------------------------
// Host side: shape rules, tile plan, dispatch
// ---------------------------------------------------------------------------
const char *matvec_shape_error(int fmt, size_t out_dim, size_t in_dim, size_t group) {
    if (out_dim == 0 || in_dim == 0) return "empty matrix";
    if (out_dim > 0x7fffffffull || in_dim > 0x7fffffffull) return "dimension too large";
    if (fmt == FMT_Q4K || fmt == FMT_Q6K) {
        if (in_dim % QK_K) return "in_dim is not a multiple of the 256-element super-block";
    } else if (fmt == FMT_MLX4) {
        if (in_dim % 8) return "in_dim is not a multiple of 8 (one packed word)";
        if (group == 0 || in_dim % group) return "in_dim is not a multiple of the MLX group size";
        if (group % 8) return "MLX group size is not a multiple of 8";
    } else {
        return "no kernel for this weight type";
    }
    return nullptr;
}

static inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

struct Plan {
    bool ok = false;
    StreamParams p{};
    int rw = 1, g = 1, grid = 0, threads = 0;
    uint32_t smem = 0;
    double score = 0;
};

static Plan plan_stream(const DeviceInfo &dev, int fmt, size_t out_dim, size_t in_dim, size_t group, int tbl_bytes) {
    Plan best;
    const uint32_t cg_elems = fmt == FMT_Q4K ? 2048u : 1024u;
    const uint32_t xregs = fmt == FMT_Q4K ? XREGS_Q4K : (fmt == FMT_Q6K ? XREGS_Q6K : XREGS_MLX);
    uint32_t row_bytes, tbl_row_bytes = 0;
    if (fmt == FMT_MLX4) {
        if (in_dim % 32 || group % 32) return best; // a lane owns 32 consecutive weights of one group
        row_bytes = (uint32_t)(in_dim / 2);
        tbl_row_bytes = (uint32_t)(in_dim / group) * tbl_bytes;
    } else {
        row_bytes = (uint32_t)(in_dim / QK_K) * (fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
    }
    const uint32_t ncg = (uint32_t)((in_dim + cg_elems - 1) / cg_elems);
    const uint32_t gmax = 2;
    const uint32_t G = (ncg + 15) / 16;
    if (G > gmax) return best;
    const uint32_t WC = (ncg + G - 1) / G;
    const int budget = dev.max_smem_optin - 1024;
    for (uint32_t WR = 1; WR <= 16; WR *= 2) {
        if (WC * WR > 16) break;
        if (WC > 1 && WR > 8) break; // named barriers 1..8
        for (uint32_t RW = 1; RW <= 4; RW *= 2) {
            const uint32_t R = WR * RW;
            if ((R * row_bytes) % 16 || (R * tbl_row_bytes) % 16) continue;
            if (out_dim % R && ((row_bytes % 16) || (tbl_row_bytes % 16))) continue;
            const uint32_t wst = align_up(R * row_bytes, 128), tst = align_up(R * tbl_row_bytes, 128);
            const uint32_t stage = wst + 2 * tst;
            if (stage > 48 * 1024) continue;
            const uint32_t ntiles = (uint32_t)((out_dim + R - 1) / R);
            const uint32_t grid = std::min<uint32_t>((uint32_t)dev.sm_count, ntiles);
            const uint32_t per = (ntiles + grid - 1) / grid;
            const uint32_t off_part = 128;
            const uint32_t off_prep = align_up(off_part + 2 * R * WC * 4, 128);
            const uint32_t off_ring = align_up(off_prep + ncg * xregs * 32 * 4, 128);
            if ((int)off_ring + 2 * (int)stage > budget) continue;
            uint32_t S = std::min<uint32_t>(8, (budget - off_ring) / stage);
            S = std::min(S, std::max(2u, per));
            const double eff = (double)ntiles / ((double)per * grid);
            const double fill = std::min(1.0, (double)(S * stage) / 49152.0);
            const double score = eff * std::pow(std::min(1.0, stage / 8192.0), 0.25) *
                                 std::sqrt(std::min(1.0, WC * WR / 8.0)) * (1.0 + 0.03 * std::log2((double)RW)) *
                                 (0.5 + 0.5 * fill);
            if (score > best.score) {
                best.ok = true;
                best.score = score;
                best.rw = (int)RW;
                best.g = (int)G;
                best.grid = (int)grid;
                best.threads = (int)(WC * WR + 1) * 32;
                best.smem = off_ring + S * stage;
                StreamParams &p = best.p;
                p.out_dim = (uint32_t)out_dim, p.in_dim = (uint32_t)in_dim, p.group = (uint32_t)group;
                p.row_bytes = row_bytes, p.tbl_row_bytes = tbl_row_bytes;
                p.R = R, p.WC = WC, p.WR = WR, p.NW = WC * WR, p.S = S;
                p.w_stage_bytes = wst, p.tbl_stage_bytes = tst, p.stage_bytes = stage;
                p.ntiles = ntiles, p.ncg = ncg;
                p.off_part = off_part, p.off_prep = off_prep, p.off_ring = off_ring;
            }
        }
    }
    return best;
}

template <int FMT, int RW, int G, typename TBL>
static cudaError_t launch_stream_t(const Plan &pl, cudaStream_t st, bool pdl) {
    auto kfn = matvec_stream_kernel<FMT, RW, G, TBL>;
    static bool attr_set[64] = {};
    int devid = 0;
    cudaGetDevice(&devid);
    if (devid < 64 && !attr_set[devid]) {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[devid] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid), cfg.blockDim = dim3(pl.threads), cfg.dynamicSmemBytes = pl.smem, cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kfn, pl.p);
}

template <int FMT, typename TBL> static cudaError_t launch_stream_f(const Plan &pl, cudaStream_t st, bool pdl) {
#define ULLM_CASE(RWv, Gv) \
    if (pl.rw == RWv && pl.g == Gv) return launch_stream_t<FMT, RWv, Gv, TBL>(pl, st, pdl);
    ULLM_CASE(1, 1) ULLM_CASE(2, 1) ULLM_CASE(4, 1) ULLM_CASE(1, 2) ULLM_CASE(2, 2) ULLM_CASE(4, 2)
#undef ULLM_CASE
    return cudaErrorInvalidConfiguration;
}

template <int FMT, typename TBL>
static cudaError_t launch_generic_t(const void *d_w, const MlxTables &tb, const float *d_x, float *d_y, size_t row0,
                                    size_t out_dim, size_t in_dim, cudaStream_t st) {
    if (row0 >= out_dim) return cudaSuccess;
    const unsigned rows_per_cta = 8;
    unsigned grid = (unsigned)((out_dim - row0 + rows_per_cta - 1) / rows_per_cta);
    matvec_generic_kernel<FMT, TBL><<<grid, rows_per_cta * 32, 0, st>>>((const uint8_t *)d_w, (const TBL *)tb.scales,
                                                                        (const TBL *)tb.biases, (int)tb.group, d_x, d_y,
                                                                        row0, out_dim, in_dim);
    return cudaGetLastError();
}

cudaError_t launch_matvec(const DeviceInfo &dev, int fmt, const void *d_w, const MlxTables &tb, const float *d_x,
                          float *d_y, size_t out_dim, size_t in_dim, int *d_status, cudaStream_t st, bool force_generic,
                          bool pdl, MatvecPlan *plan_out) {
    Plan pl;
    const bool aligned = ((uintptr_t)d_w % 16 == 0) && ((uintptr_t)d_x % 16 == 0) &&
                         (fmt != FMT_MLX4 || ((uintptr_t)tb.scales % 16 == 0 && (uintptr_t)tb.biases % 16 == 0));
    if (!force_generic && aligned) pl = plan_stream(dev, fmt, out_dim, in_dim, tb.group, tb.elem_bytes);
    if (plan_out) {
        plan_out->streamed = pl.ok;
        plan_out->rows_per_tile = pl.ok ? (int)pl.p.R : 8;
        plan_out->warps = pl.ok ? (int)pl.p.NW : 8;
        plan_out->stages = pl.ok ? (int)pl.p.S : 0;
        plan_out->smem_bytes = pl.ok ? (int)pl.smem : 0;
        plan_out->grid = pl.ok ? pl.grid : (int)((out_dim + 7) / 8);
    }
    if (pl.ok) {
        pl.p.w = (const uint8_t *)d_w, pl.p.scales = (const uint8_t *)tb.scales, pl.p.biases = (const uint8_t *)tb.biases;
        pl.p.x = d_x, pl.p.y = d_y, pl.p.status = d_status;
        if (fmt == FMT_Q4K) return launch_stream_f<FMT_Q4K, float>(pl, st, pdl);
        if (fmt == FMT_Q6K) return launch_stream_f<FMT_Q6K, float>(pl, st, pdl);
        if (tb.elem_bytes == 2) return launch_stream_f<FMT_MLX4, uint16_t>(pl, st, pdl);
        return launch_stream_f<FMT_MLX4, float>(pl, st, pdl);
    }
    if (fmt == FMT_Q4K) return launch_generic_t<FMT_Q4K, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    if (fmt == FMT_Q6K) return launch_generic_t<FMT_Q6K, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    if (fmt == FMT_MLX4) {
        if (tb.elem_bytes == 2) return launch_generic_t<FMT_MLX4, uint16_t>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
        return launch_generic_t<FMT_MLX4, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    }
    return cudaErrorInvalidValue;
}

} // namespace ullm
