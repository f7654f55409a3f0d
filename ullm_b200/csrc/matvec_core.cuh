// Device code shared by the streamed matvec and MoE kernels: format unpack
// helpers, the fixed-point register image of x, and the per-row partial dot
// product on a row staged in shared memory.
#pragma once

#include "common.cuh"

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

constexpr int XREGS_Q4K = 36, XREGS_Q6K = 24, XREGS_MLX = 18;
template <int FMT> struct FmtTraits;
template <> struct FmtTraits<FMT_Q4K> { static constexpr int XREGS = XREGS_Q4K, CG_ELEMS = 2048; };
template <> struct FmtTraits<FMT_Q6K> { static constexpr int XREGS = XREGS_Q6K, CG_ELEMS = 1024; };
template <> struct FmtTraits<FMT_MLX4> { static constexpr int XREGS = XREGS_MLX, CG_ELEMS = 1024; };


// 16-bit fixed point of up to 32 values sharing one scale.  X = rint(v/s) with
// s = max|v|/32767; returned as byte planes: hi = X >> 8 (signed), lo = X & 255.
__device__ __forceinline__ int quant16(float v, float inv) {
    int q = __float2int_rn(v * inv);
    return max(-32767, min(32767, q));
}

// Fills the persistent register image of (column group cg, lane ln) at
// slot[k * 32] (k = 0..XREGS-1; the caller passes slot already offset by lane).
// The vector a matvec consumes: x itself, or rmsnorm(x) = x[i] * inv * norm_w[i]
// (crates/ullm-model/src/math.rs:82-86) when norm_w is given.
struct ActSrc {
    const float *x;
    const float *norm_w; // may be null
    float inv;           // 1 / sqrt(mean(x^2) + eps) when norm_w is set
};
__device__ __forceinline__ float4 act_load4(const ActSrc &a, uint32_t i) {
    float4 t = __ldg((const float4 *)(a.x + i));
    if (a.norm_w) {
        float4 w = __ldg((const float4 *)(a.norm_w + i));
        t.x = t.x * a.inv * w.x, t.y = t.y * a.inv * w.y, t.z = t.z * a.inv * w.z, t.w = t.w * a.inv * w.w;
    }
    return t;
}

template <int FMT>
__device__ __forceinline__ void prep_slot(const ActSrc &src, uint32_t in_dim, uint32_t cg, uint32_t ln, uint32_t *slot) {
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
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 t = act_load4(src, e0 + 32 * half + 4 * i);
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
            float4 t0 = act_load4(src, e0 + 32 * g), t1 = act_load4(src, e0 + 32 * g + 4);
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
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4 t = act_load4(src, e0 + 4 * i);
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


} // namespace ullm
