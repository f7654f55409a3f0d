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

constexpr int XREGS_Q4K = 36, XREGS_Q6K = 24, XREGS_MLX = 18, XREGS_Q6KR = 37;
template <int FMT> struct FmtTraits;
template <> struct FmtTraits<FMT_Q4K> { static constexpr int XREGS = XREGS_Q4K, CG_ELEMS = 2048; };
template <> struct FmtTraits<FMT_Q6K> { static constexpr int XREGS = XREGS_Q6K, CG_ELEMS = 1024; };
template <> struct FmtTraits<FMT_MLX4> { static constexpr int XREGS = XREGS_MLX, CG_ELEMS = 1024; };
template <> struct FmtTraits<FMT_Q6KR> { static constexpr int XREGS = XREGS_Q6KR, CG_ELEMS = 2048; };


// 16-bit fixed point of up to 32 values sharing one scale.  X = rint(v/s) with
// s = max|v|/32767; returned as byte planes: hi = X >> 8 (signed), lo = X & 255.
// max(|a|, |b|) that keeps a NaN once it has seen one (fmaxf drops NaNs): a group that holds a NaN gets a NaN
// scale, so the NaN reaches every output row the way it does in the reference's f32 product
// (crates/ullm-model/src/math.rs:17) instead of being rounded to an integer.
__device__ __forceinline__ float absmax_nan(float mx, float v) {
    const float a = fabsf(v);
    return (a > mx || a != a) ? a : mx;
}
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

// Builds the persistent register images of one activation vector in shared
// memory: img[(cg * XREGS + k) * 32 + lane] is register k of (column group cg,
// lane).  Work is split in tasks of 8 consecutive elements so that all `nthr`
// threads take part (blockDim-uniform loop; nthr must be a multiple of 32 and all
// threads of the participating warps must call this).
//
// Register image layouts (what row_partial expects):
//  Q4_K  lane (cg, ln): block 8cg + ln/4, chunk c = ln%4.  Low nibbles are elements
//        [64c, 64c+32) of the block, high nibbles [64c+32, 64c+64) (dequant.rs:200-214).
//        k = 16*half + j: high byte plane of word j (elements 4j..4j+3) of that half,
//        16*half + 8 + j: low byte plane, 32+half: x scale (half 1 carries 1/16 because
//        high nibbles are used in place), 34+half: fp32 sum of the 32 x values.
//  Q6_K  lane (cg, ln): block 4cg + ln/8, nh = (ln%8)/4, l0 = 8*(ln%4); group g = 0..3 is
//        elements 128nh + 32g + l0 + [0,8) (dequant.rs:264-279).  k = 4g + j: high plane of
//        word j, 4g + 2 + j: low plane, 16+g: x scale, 20+g: 32 * sum of the fixed-point x
//        (folds the -32 offset of the 6-bit values).
//  Q6KR  lane (cg, ln): block 8cg + ln/4, nh = (ln/2)%2, t' = ln%2: the 16 positions
//        l = 16t' .. 16t'+15 of half nh in all four groups g (elements 128nh + 32g + l).
//        One x scale for the 64 values.  k = 8g + j: high plane of word j (l = 16t'+4j..+3)
//        of group g, 8g + 4 + j: low plane, 32: x scale, 33+g: -32 * sum of the fixed-point
//        x of group g (the accumulator's start value: folds the -32 offset).
//  MLX4  lane (cg, ln): words 4*(32cg+ln)..+3 = elements 32*(32cg+ln) + [0,32); nibble n of
//        word j is element 8j+n (dequant.rs:310-311).  k = j: high plane of the even
//        nibbles of word j, 4+j: their low plane, 8+j / 12+j: the odd nibbles (used in
//        place, value*16), 16: x scale / 16, 17: fp32 sum of the 32 x values.
// Raw x values a thread fetched early (before the weight stream was started, so that
// these small loads do not queue behind megabytes of weight traffic): pass ps of the
// task loop below, i.e. elements 8 * (ps * nthr + tid) .. +7.
constexpr int PREP_NPRE = 3;
struct PrepPre {
    float4 x[PREP_NPRE][2];
    float4 w0[2]; // norm weights of pass 0
    bool valid = false;
};
__device__ __forceinline__ void prep_preload(PrepPre &pre, const float *x, const float *norm_w, uint32_t in_dim, uint32_t tid,
                                             uint32_t nthr) {
    const uint32_t ntasks = in_dim >> 3;
#pragma unroll
    for (int ps = 0; ps < PREP_NPRE; ++ps) {
        const uint32_t t = ps * nthr + tid;
        const uint32_t e = (t < ntasks ? t : 0u) << 3;
        pre.x[ps][0] = __ldg((const float4 *)(x + e));
        pre.x[ps][1] = __ldg((const float4 *)(x + e + 4));
    }
    if (norm_w) {
        const uint32_t e = (tid < ntasks ? tid : 0u) << 3;
        pre.w0[0] = __ldg((const float4 *)(norm_w + e));
        pre.w0[1] = __ldg((const float4 *)(norm_w + e + 4));
    }
    pre.valid = true;
}
__device__ __forceinline__ float4 norm4(float4 t, float inv, float4 w) {
    t.x = t.x * inv * w.x, t.y = t.y * inv * w.y, t.z = t.z * inv * w.z, t.w = t.w * inv * w.w;
    return t;
}

template <int FMT>
__device__ __forceinline__ void prep_image(const ActSrc &src, uint32_t in_dim, uint32_t *img, uint32_t tid, uint32_t nthr,
                                           const PrepPre *pre = nullptr) {
    constexpr int XR = FmtTraits<FMT>::XREGS;
    const uint32_t ntasks = in_dim >> 3;
    int pass = 0;
    for (uint32_t base = 0; base < ntasks; base += nthr, ++pass) {
        const uint32_t t = base + tid;
        const bool act = t < ntasks;
        const uint32_t e = (act ? t : 0u) << 3;
        float4 t0, t1;
        if (pre && pass < PREP_NPRE) {
            t0 = pass == 0 ? pre->x[0][0] : (pass == 1 ? pre->x[1][0] : pre->x[2][0]);
            t1 = pass == 0 ? pre->x[0][1] : (pass == 1 ? pre->x[1][1] : pre->x[2][1]);
            if (src.norm_w) {
                float4 w0 = pass == 0 ? pre->w0[0] : __ldg((const float4 *)(src.norm_w + e));
                float4 w1 = pass == 0 ? pre->w0[1] : __ldg((const float4 *)(src.norm_w + e + 4));
                t0 = norm4(t0, src.inv, w0), t1 = norm4(t1, src.inv, w1);
            }
        } else {
            t0 = act_load4(src, e), t1 = act_load4(src, e + 4);
        }
        const float v[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        float mx = 0.f, sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = absmax_nan(mx, v[i]), sum += v[i];
        if (FMT == FMT_Q6KR) { // 64 values share a scale: task bits 0 (8 of 16), 2-3 (group)
            mx = absmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = absmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = absmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        } else if (FMT != FMT_Q6K) { // 32 values share a scale: four neighbouring tasks
            mx = absmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = absmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        }
        const float inv = mx > 0.f ? 32767.f / mx : 0.f, sc = mx * (1.f / 32767.f);
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = quant16(v[i], inv);
        int isum8 = 0;
        if (FMT == FMT_Q6KR) {
#pragma unroll
            for (int i = 0; i < 8; ++i) isum8 += q[i];
            isum8 += __shfl_xor_sync(0xffffffffu, isum8, 1); // the 16 positions of this group
        }
        if (!act) continue;
        if constexpr (FMT == FMT_Q4K) {
            const uint32_t b = e >> 8, r = e & 255u, c = r >> 6, half = (r >> 5) & 1u, sub = (r >> 3) & 3u;
            uint32_t *slot = img + ((b >> 3) * XR) * 32 + (((b & 7u) << 2) | c);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    hi |= (uint32_t)((q[4 * j + k] >> 8) & 0xff) << (8 * k);
                    lo |= (uint32_t)(q[4 * j + k] & 0xff) << (8 * k);
                }
                slot[(16 * half + 2 * sub + j) * 32] = hi;
                slot[(16 * half + 8 + 2 * sub + j) * 32] = lo;
            }
            if (sub == 0) {
                slot[(32 + half) * 32] = __float_as_uint(half ? sc * 0.0625f : sc);
                slot[(34 + half) * 32] = __float_as_uint(sum);
            }
        } else if constexpr (FMT == FMT_Q6K) {
            const uint32_t b = e >> 8, r = e & 255u, nh = r >> 7, g = (r >> 5) & 3u, tt = (r >> 3) & 3u;
            uint32_t *slot = img + ((b >> 2) * XR) * 32 + (((b & 3u) << 3) | (nh << 2) | tt);
            int isum = 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    isum += q[4 * j + k];
                    hi |= (uint32_t)((q[4 * j + k] >> 8) & 0xff) << (8 * k);
                    lo |= (uint32_t)(q[4 * j + k] & 0xff) << (8 * k);
                }
                slot[(4 * g + j) * 32] = hi;
                slot[(4 * g + 2 + j) * 32] = lo;
            }
            slot[(16 + g) * 32] = __float_as_uint(sc);
            slot[(20 + g) * 32] = (uint32_t)(32 * isum);
        } else if constexpr (FMT == FMT_Q6KR) {
            const uint32_t b = e >> 8, r = e & 255u, nh = r >> 7, g = (r >> 5) & 3u, l8 = (r >> 3) & 3u;
            const uint32_t tp = l8 >> 1, jj = (l8 & 1u) * 2u;
            uint32_t *slot = img + ((b >> 3) * XR) * 32 + (((b & 7u) << 2) | (nh << 1) | tp);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    hi |= (uint32_t)((q[4 * j + k] >> 8) & 0xff) << (8 * k);
                    lo |= (uint32_t)(q[4 * j + k] & 0xff) << (8 * k);
                }
                slot[(8 * g + jj + j) * 32] = hi;
                slot[(8 * g + 4 + jj + j) * 32] = lo;
            }
            if ((l8 & 1u) == 0) slot[(33 + g) * 32] = (uint32_t)(-32 * isum8);
            if (g == 0 && (l8 & 1u) == 0) slot[32 * 32] = __float_as_uint(sc);
        } else {
            const uint32_t widx = e >> 5, j = (e >> 3) & 3u;
            uint32_t *slot = img + ((widx >> 5) * XR) * 32 + (widx & 31u);
            uint32_t he = 0, le = 0, ho = 0, lo = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                he |= (uint32_t)((q[2 * k] >> 8) & 0xff) << (8 * k);
                le |= (uint32_t)(q[2 * k] & 0xff) << (8 * k);
                ho |= (uint32_t)((q[2 * k + 1] >> 8) & 0xff) << (8 * k);
                lo |= (uint32_t)(q[2 * k + 1] & 0xff) << (8 * k);
            }
            slot[j * 32] = he, slot[(4 + j) * 32] = le, slot[(8 + j) * 32] = ho, slot[(12 + j) * 32] = lo;
            if (j == 0) {
                slot[16 * 32] = __float_as_uint(sc * 0.0625f);
                slot[17 * 32] = __float_as_uint(sum);
            }
        }
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
    } else if constexpr (FMT == FMT_Q6KR) {
        // prepared row: [records 48 B x 4 x nb][scales 4 B x 4 x nb][d 2 B x nb];
        // tbl_s / tbl_b carry the addresses of the scale and d planes of this row
        const uint32_t ri = cg * 32u + ln; // record = (block, nh, t')
        const uint32_t rec = row_addr + ri * 48u;
        const uint4 w1 = lds128(rec), w2 = lds128(rec + 16), w3 = lds128(rec + 32);
        const uint32_t sc4 = lds32(tbl_s + ri * 4u);
        uint32_t dbits;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits) : "r"(tbl_b + (ri >> 2) * 2u));
        const uint32_t a1[4] = {w1.x, w1.y, w1.z, w1.w}, a2[4] = {w2.x, w2.y, w2.z, w2.w}, a3[4] = {w3.x, w3.y, w3.z, w3.w};
        int ah[4] = {0, 0, 0, 0};
        int al[4] = {(int)X[33], (int)X[34], (int)X[35], (int)X[36]};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t q0 = a1[j] & 0x3f3f3f3fu, q3 = a3[j] & 0x3f3f3f3fu;
            const uint32_t q1 = (a2[j] & 0x0f0f0f0fu) | ((a1[j] >> 2) & 0x30303030u);
            const uint32_t q2 = ((a2[j] >> 4) & 0x0f0f0f0fu) | ((a3[j] >> 2) & 0x30303030u);
            ah[0] = dp4a_su(q0, X[j], ah[0]), al[0] = dp4a_uu(q0, X[4 + j], al[0]);
            ah[1] = dp4a_su(q1, X[8 + j], ah[1]), al[1] = dp4a_uu(q1, X[12 + j], al[1]);
            ah[2] = dp4a_su(q2, X[16 + j], ah[2]), al[2] = dp4a_uu(q2, X[20 + j], al[2]);
            ah[3] = dp4a_su(q3, X[24 + j], ah[3]), al[3] = dp4a_uu(q3, X[28 + j], al[3]);
        }
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int sc = (int)(sc4 << (24 - 8 * g)) >> 24; // int8 scale of group g
            s += (float)sc * (float)(ah[g] * 256 + al[g]);
        }
        return f16_bits_to_f32((uint16_t)dbits) * __uint_as_float(X[32]) * s;
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
        // group sizes are powers of two in every MLX checkpoint (32, 64, 128): a shift, not a division, per row
        const uint32_t g = (group & (group - 1u)) == 0u ? (widx * 32u) >> (31 - __clz((int)group)) : (widx * 32u) / group;
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
    if (mbar_try_wait(bar, parity)) return true; // already complete: no timer needed
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
