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
#include "kernels.h"
#include "matvec_core.cuh"

#include <algorithm>
#include <cmath>

namespace ullm {

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
struct StreamParams {
    const uint8_t *w;
    const uint8_t *scales, *biases; // MLX tables (bytes), else null
    const float *x;
    float *y;
    int *status;
    const float *norm_w; // prologue: x <- rmsnorm(x, norm_w, eps) when set
    float eps;
    int epi;             // EPI_STORE / EPI_RESIDUAL / EPI_SWIGLU
    const float *res;    // EPI_RESIDUAL: y[o] = res[o] + (W x)[o]  (res may alias y)
    uint32_t out_dim, in_dim, group;
    uint32_t row_bytes, tbl_row_bytes;
    uint32_t gran;       // CTA row ranges start at multiples of this many rows (16-byte alignment)
    uint32_t R, WC, WR, NW, S;
    uint32_t NSL;        // barrier slices per tile: WR (one per row slice of RW rows) or 1 (whole tile)
    uint32_t w_stage_bytes, tbl_stage_bytes, stage_bytes; // regions inside one stage (128-B multiples)
    uint32_t ncg;
    uint32_t off_part, off_prep, off_ring; // byte offsets in dynamic smem
    int pdl;                   // launched with programmatic stream serialization
    uint32_t chunk;            // bytes per bulk copy (multiple of 16)
};
static int g_stream_chunk = 4096;
void matvec_stream_set_chunk(int bytes) { g_stream_chunk = bytes >= 1024 ? bytes / 16 * 16 : 4096; }

constexpr int STREAM_MAX_THREADS = 800; // 24 consumer warps + the producer warp

template <int FMT, int RW, int G, typename TBL>
__global__ void __launch_bounds__(STREAM_MAX_THREADS, 1) matvec_stream_kernel(const StreamParams p) {
    constexpr int XR = FmtTraits<FMT>::XREGS;
    extern __shared__ __align__(128) uint8_t smem[];
    // full / empty mbarriers, one pair per (stage, slice): a row slice (the RW rows of one warp row) is
    // handed over as soon as its own bytes are in, and refilled as soon as its own warps are done with it,
    // so a 90 KB tile does not have to land completely before the first row is computed.
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + p.S * p.NSL;
    float *part = (float *)(smem + p.off_part);
    uint32_t *prep = (uint32_t *)(smem + p.off_prep);
    uint8_t *ring = smem + p.off_ring;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == p.NW;

    // Rows are dealt to the CTAs as contiguous, balanced ranges (to within `gran`
    // rows); each CTA walks its range in tiles of R rows, the last one ragged.
    const uint32_t units = p.out_dim / p.gran;
    const uint32_t rbeg = (uint32_t)(((uint64_t)units * blockIdx.x) / gridDim.x) * p.gran;
    const uint32_t rend = blockIdx.x + 1 == gridDim.x ? p.out_dim
                                                      : (uint32_t)(((uint64_t)units * (blockIdx.x + 1)) / gridDim.x) * p.gran;
    const uint32_t ntiles = (rend - rbeg + p.R - 1) / p.R;

    // Under programmatic dependent launch the next kernel may be scheduled as soon
    // as SMs free up; it only prefetches its own weights until this grid is done.
    pdl_launch_dependents();
    // Without a programmatic dependency x is ready now: fetch it before the weight
    // stream starts, or these few KB wait behind megabytes of queued weight traffic.
    const uint32_t nthr_c = p.NW * 32; // consumer threads
    PrepPre pre;
    if (!p.pdl && !producer) prep_preload(pre, p.x, p.norm_w, p.in_dim, tid, nthr_c);
    if (tid == 0) {
        for (uint32_t s = 0; s < p.S * p.NSL; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.NW / p.NSL);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (producer) {
        // One tile = one contiguous byte range (plus two table ranges for MLX), requested slice by
        // slice (one slice = the whole tile unless the plan asks for one per warp row).  The whole
        // producer warp issues a slice, in chunks of p.chunk bytes spread over the lanes; all chunks
        // complete on the slice's barrier.  Weights do not depend on the previous kernel in the
        // stream, so the stream starts at once.  The first ring revolution is staggered (tile k is
        // requested when tile k-1 has landed): requested together, all S tiles would arrive together
        // and the first row could only be computed when most of the ring had been filled.
        const uint32_t srows = p.R / p.NSL; // rows per slice
        uint32_t s = 0, ph = 0;             // stage and the phase of its previous use, carried along
        bool ok = true;
        for (uint32_t k = 0; k < ntiles && ok; ++k) {
            const uint32_t r0 = rbeg + k * p.R;
            const uint32_t rows = min(p.R, rend - r0);
            uint8_t *dst = ring + (size_t)s * p.stage_bytes;
            for (uint32_t j = 0; j < p.NSL; ++j) {
                uint64_t *fb = &full[s * p.NSL + j];
                if (lane == 0) {
                    if (k >= p.S) ok = wait_or_timeout(&empty[s * p.NSL + j], ph ^ 1u);
                    else if (k > 0 && j == 0) ok = wait_or_timeout(&full[(k - 1) * p.NSL + p.NSL - 1], 0);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                const uint32_t row0 = j * srows;
                const uint32_t nrows = rows > row0 ? min(srows, rows - row0) : 0u; // 0: a slice past the ragged end
                const uint32_t wb = nrows * p.row_bytes, tb = nrows * p.tbl_row_bytes;
                if (lane == 0) mbar_arrive_expect_tx(fb, wb + 2 * tb);
                __syncwarp();
                const uint8_t *src = p.w + (size_t)(r0 + row0) * p.row_bytes;
                uint8_t *d = dst + (size_t)row0 * p.row_bytes;
                for (uint32_t off = lane * p.chunk; off < wb; off += 32 * p.chunk)
                    bulk_g2s(d + off, src + off, min(p.chunk, wb - off), fb);
                if (FMT == FMT_MLX4 && lane < 2 && tb) {
                    const uint8_t *t = (lane ? p.biases : p.scales) + (size_t)(r0 + row0) * p.tbl_row_bytes;
                    bulk_g2s(dst + p.w_stage_bytes + lane * p.tbl_stage_bytes + (size_t)row0 * p.tbl_row_bytes, t, tb, fb);
                }
            }
            if (++s == p.S) s = 0, ph ^= 1u;
        }
        return;
    }

    // ---- consumer warps (named barrier 2 = all of them) ----
    pdl_wait_prior();
    if (p.pdl) prep_preload(pre, p.x, p.norm_w, p.in_dim, tid, nthr_c);

    // Optional fused RMSNorm of the input (crates/ullm-model/src/math.rs:82-86):
    // every CTA recomputes the mean square of x (a few KB from L2).
    ActSrc src{p.x, p.norm_w, 0.f};
    if (p.norm_w) {
        float ss = 0.f;
        const uint32_t ntasks = p.in_dim >> 3;
#pragma unroll
        for (int ps = 0; ps < PREP_NPRE; ++ps)
            if (ps * nthr_c + tid < ntasks) {
                const float4 a = pre.x[ps][0], b = pre.x[ps][1];
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
            }
        for (uint32_t t = PREP_NPRE * nthr_c + tid; t < ntasks; t += nthr_c) {
            const float4 a = __ldg((const float4 *)(p.x + 8 * t)), b = __ldg((const float4 *)(p.x + 8 * t + 4));
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) part[warp] = ss;
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
        float tot = 0.f;
        for (uint32_t w = 0; w < p.NW; ++w) tot += part[w];
        src.inv = 1.0f / sqrtf(tot / (float)p.in_dim + p.eps);
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory"); // part is reused by the row reduction below
    }
    // x -> fixed-point register images, built once per CTA in shared memory
    prep_image<FMT>(src, p.in_dim, prep, tid, nthr_c, &pre);
    asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");

    const uint32_t rs = warp / p.WC, cgw = warp % p.WC;
    uint32_t X[G][XR];
    bool live[G]; // lanes past the end of the row must not read beyond the stage
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint32_t cg = cgw + g * p.WC;
        live[g] = cg < p.ncg;
        if (FMT == FMT_Q4K || FMT == FMT_Q6KR) live[g] = live[g] && (cg * 8u + (lane >> 2)) * QK_K < p.in_dim;
        if (FMT == FMT_Q6K) live[g] = live[g] && (cg * 4u + (lane >> 3)) * QK_K < p.in_dim;
        if (FMT == FMT_MLX4) live[g] = live[g] && (cg * 32u + lane) * 32u < p.in_dim;
#pragma unroll
        for (int k = 0; k < XR; ++k) X[g][k] = live[g] ? prep[((size_t)cg * XR + k) * 32 + lane] : 0u;
    }
    const uint32_t nb = p.in_dim / QK_K;

    bool aborted = false;
    // Sums the per-column-group partials of tile kt and writes its rows.  Run by the
    // first warp of each row slice, one tile-ring revolution late: by then every
    // warp has released the tile's stage (and written its partials before doing
    // so), so no barrier between the warps of a slice is needed per tile.
    // `slot` = kt mod 2S names the tile's partial area (the tile loop keeps it without dividing).
    auto flush = [&](uint32_t kt, uint32_t slot) {
        if (cgw != 0 || lane >= RW) return;
        const float *pt = part + ((size_t)slot * p.R) * p.WC;
        const uint32_t row = rs * RW + lane, gr = rbeg + kt * p.R + row;
        if (gr >= rend || aborted) return;
        float acc = 0.f;
        for (uint32_t c = 0; c < p.WC; ++c) acc += pt[row * p.WC + c];
        if (p.epi == EPI_STORE) p.y[gr] = acc;
        else if (p.epi == EPI_RESIDUAL) p.y[gr] = p.res[gr] + acc;
        else if ((lane & 1) == 0) {
            float up = 0.f;
            for (uint32_t c = 0; c < p.WC; ++c) up += pt[(row + 1) * p.WC + c];
            p.y[gr >> 1] = acc / (1.0f + expf(-acc)) * up;
        }
    };
    const uint32_t bslice = p.NSL > 1 ? rs : 0u; // the barrier pair of this warp's rows
    uint32_t slot = 0; // k mod 2S: stage s = slot mod S, mbarrier phase = slot / S
    for (uint32_t k = 0; k < ntiles; ++k, slot = slot + 1 == 2 * p.S ? 0 : slot + 1) {
        const uint32_t ph = slot >= p.S ? 1u : 0u, s = slot - ph * p.S;
            if (!aborted && !wait_or_timeout(&full[s * p.NSL + bslice], ph)) aborted = true;
            if (p.WC > 1 && k >= p.S) flush(k - p.S, ph ? s : s + p.S);
        const uint32_t stage = smem_u32(ring + (size_t)s * p.stage_bytes);
        const uint32_t r0 = rbeg + k * p.R;
        float v[RW];
#pragma unroll
        for (int rr = 0; rr < RW; ++rr) {
            v[rr] = 0.f;
            const uint32_t rl = rs * RW + rr;
            if (!aborted && r0 + rl < rend) {
                const uint32_t row_addr = stage + rl * p.row_bytes;
                uint32_t ts, tb2;
                if (FMT == FMT_Q6KR) ts = row_addr + 192u * nb, tb2 = row_addr + 208u * nb;
                else ts = stage + p.w_stage_bytes + rl * p.tbl_row_bytes, tb2 = ts + p.tbl_stage_bytes;
#pragma unroll
                for (int g = 0; g < G; ++g)
                    if (live[g]) v[rr] += row_partial<FMT, TBL>(row_addr, X[g], cgw + g * p.WC, lane, ts, tb2, p.group);
            }
        }
        uint32_t myrow;
        float r = warp_reduce_rows<RW>(v, lane, myrow);
        const uint32_t rl = rs * RW + myrow;
        if (p.WC == 1) {
            // SwiGLU on interleaved rows: even row = gate, odd row = up, held by the
            // lane group that differs in the lowest row bit
            float other = 0.f;
            if (RW >= 2) other = __shfl_xor_sync(0xffffffffu, r, RW == 2 ? 16 : 8);
            const bool writer = (lane & 7) == 0 && (RW == 4 || (lane & 8) == 0) && (RW > 1 || lane == 0);
            if (writer && r0 + rl < rend && !aborted) {
                if (p.epi == EPI_STORE) p.y[r0 + rl] = r;
                else if (p.epi == EPI_RESIDUAL) p.y[r0 + rl] = p.res[r0 + rl] + r;
                else if ((myrow & 1) == 0) p.y[(r0 + rl) >> 1] = r / (1.0f + expf(-r)) * other;
            }
        } else {
            float *pt = part + ((size_t)slot * p.R) * p.WC;
            if ((lane & 7) == 0 && (RW == 4 || (lane & 8) == 0)) pt[rl * p.WC + cgw] = r;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s * p.NSL + bslice]); // partials written, the slice may be refilled
    }
    if (p.WC > 1) {
        asm volatile("bar.sync 1, %0;" ::"r"(p.NW * 32) : "memory"); // all partials of the last tiles are in
        for (uint32_t kt = ntiles > p.S ? ntiles - p.S : 0; kt < ntiles; ++kt) flush(kt, kt % (2 * p.S));
    }
    if (aborted && lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
}

// ---------------------------------------------------------------------------
// Host side: shape rules, tile plan, dispatch
// ---------------------------------------------------------------------------
const char *matvec_shape_error(int fmt, size_t out_dim, size_t in_dim, size_t group) {
    if (out_dim == 0 || in_dim == 0) return "empty matrix";
    if (out_dim > 0x7fffffffull || in_dim > 0x7fffffffull) return "dimension too large";
    if (fmt == FMT_Q4K || fmt == FMT_Q6K || fmt == FMT_Q6KR) {
        if (in_dim % QK_K) return "in_dim is not a multiple of the 256-element super-block";
        if (fmt == FMT_Q6KR && in_dim % 2048) return "prepared Q6_K rows need in_dim to be a multiple of 2048";
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
static inline uint32_t gcd_u32(uint32_t a, uint32_t b) {
    while (b) {
        uint32_t t = a % b;
        a = b, b = t;
    }
    return a;
}

struct Plan {
    bool ok = false;
    StreamParams p{};
    int rw = 1, g = 1, grid = 0, threads = 0;
    uint32_t smem = 0;
    double score = 0;
};

// force_wr / force_rw / force_stages: the caller's plan override (tests), 0 = choose automatically.
static Plan plan_stream(const DeviceInfo &dev, int fmt, size_t out_dim, size_t in_dim, size_t group, int tbl_bytes,
                        int epi, int force_wr = 0, int force_rw = 0, int force_stages = 0) {
    Plan best;
    const uint32_t cg_elems = (fmt == FMT_Q4K || fmt == FMT_Q6KR) ? 2048u : 1024u;
    const uint32_t xregs = fmt == FMT_Q4K ? XREGS_Q4K : (fmt == FMT_Q6K ? XREGS_Q6K : (fmt == FMT_Q6KR ? XREGS_Q6KR : XREGS_MLX));
    uint32_t row_bytes, tbl_row_bytes = 0;
    if (fmt == FMT_MLX4) {
        if (in_dim % 32 || group % 32) return best; // a lane owns 32 consecutive weights of one group
        row_bytes = (uint32_t)(in_dim / 2);
        tbl_row_bytes = (uint32_t)(in_dim / group) * tbl_bytes;
    } else {
        row_bytes = (uint32_t)(in_dim / QK_K) * (fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
    }
    if (fmt == FMT_Q6KR && in_dim % 2048) return best;
    // rows at which a 16-byte aligned copy may start
    uint32_t gran = 16 / gcd_u32(row_bytes, 16);
    if (tbl_row_bytes) gran = std::max(gran, 16 / gcd_u32(tbl_row_bytes, 16)); // both powers of two
    if (epi == EPI_SWIGLU) gran = std::max(gran, 2u);
    if (out_dim % gran) return best;
    const uint32_t ncg = (uint32_t)((in_dim + cg_elems - 1) / cg_elems);
    const uint32_t cpsm = 1u; // one CTA per SM
    const uint32_t max_warps = 24;
    const uint32_t G = (ncg + 15) / 16;
    if (G > 2) return best;
    const uint32_t WC = (ncg + G - 1) / G;
    if (WC > max_warps) return best;
    const int budget = dev.max_smem_optin - 1024;
    const uint32_t units = (uint32_t)(out_dim / gran);
    const uint32_t grid = std::min<uint32_t>((uint32_t)dev.sm_count * cpsm, units);
    const uint32_t rows_cta = ((units + grid - 1) / grid) * gran; // the largest range
    for (uint32_t WR = 1; WR <= 15; ++WR) {
        if (WC * WR > max_warps) break;
        if (WC == 1 && WR > 24) break;
        if (force_wr && (int)WR != force_wr) continue;
        for (uint32_t RW = (epi == EPI_SWIGLU ? 2 : 1); RW <= 4; RW *= 2) {
            if (force_rw && (int)RW != force_rw) continue;
            const uint32_t R = WR * RW;
            if (R % gran) continue;
            const uint32_t wst = align_up(R * row_bytes, 128), tst = align_up(R * tbl_row_bytes, 128);
            const uint32_t stage = wst + 2 * tst;
            if (stage > 100 * 1024) continue;
            // one barrier pair per row slice when the slices are large (measured: slices of 47 KB, [4096,14336]
            // Q6_K, 13.7 -> 13.0 us; slices of 13-18 KB lose 10-20 %) and start 16-byte aligned, else one per tile
            const uint32_t NSL = (WR > 1 && RW * row_bytes >= 32768 && (RW * row_bytes) % 16 == 0 &&
                                  (RW * tbl_row_bytes) % 16 == 0) ? WR : 1u;
            const uint32_t off_part = align_up(2 * 8 * NSL * 8, 128); // up to 8 stages x NSL slices x (full, empty)
            const uint32_t off_prep = align_up(off_part + std::max(2 * 8 * R * WC * 4, 128u), 128);
            const uint32_t off_ring = align_up(off_prep + ncg * xregs * 32 * 4, 128);
            if ((int)off_ring + 2 * (int)stage > budget) continue;
            const uint32_t tiles = (rows_cta + R - 1) / R;
            uint32_t S = std::min<uint32_t>(8, (budget - off_ring) / stage);
            S = std::min(S, std::max(2u, tiles));
            if (force_stages) S = std::min<uint32_t>(S, (uint32_t)force_stages);
            // Measured on B200 (plan sweeps on [28672,8192] and [8192,8192] Q4_K, [14336,4096] and [4096,14336]
            // Q6_K): the kernels are bound by instruction issue, not by HBM (about 200 warp instructions per
            // 2048 weights; streaming alone runs at 5.2 TB/s where the full kernel reached 3.9), so four rows per
            // warp beat two (the register image of x and the per-tile bookkeeping are shared by more rows, and
            // the transposed reduction costs less per row), as many warps as the tile allows beat fewer, and two
            // stages of 70-95 KB are enough when that is what four rows per warp cost.
            const double eff = (double)rows_cta / ((double)tiles * R); // idle warps in the ragged tile
            const double f_warps = std::sqrt(std::min(1.0, (WC * WR) / 14.0));
            const double f_rw = RW == 1 ? 0.75 : (RW == 2 ? 0.84 : 1.0);
            const double f_stage = std::sqrt(std::min(1.0, stage / 45056.0));
            const double f_depth = (S >= 3 || tiles <= S) ? 1.0 : 0.97;
            const double score = eff * f_warps * f_rw * f_stage * f_depth;
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
                p.row_bytes = row_bytes, p.tbl_row_bytes = tbl_row_bytes, p.gran = gran;
                p.R = R, p.WC = WC, p.WR = WR, p.NW = WC * WR, p.S = S, p.NSL = NSL;
                p.w_stage_bytes = wst, p.tbl_stage_bytes = tst, p.stage_bytes = stage;
                p.ncg = ncg;
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
                          float *d_y, size_t out_dim, size_t in_dim, int *d_status, cudaStream_t st,
                          const MatvecOpts &o) {
    Plan pl;
    const bool fused = o.norm_w || o.epi != EPI_STORE;
    const bool aligned = ((uintptr_t)d_w % 16 == 0) && ((uintptr_t)d_x % 16 == 0) &&
                         (!o.norm_w || (uintptr_t)o.norm_w % 16 == 0) &&
                         (fmt != FMT_MLX4 || ((uintptr_t)tb.scales % 16 == 0 && (uintptr_t)tb.biases % 16 == 0));
    if (o.epi == EPI_SWIGLU && (out_dim & 1)) return cudaErrorInvalidValue;
    if (!o.force_generic && aligned) pl = plan_stream(dev, fmt, out_dim, in_dim, tb.group, tb.elem_bytes, o.epi, o.plan_wr, o.plan_rw, o.plan_stages);
    if (o.plan_out) {
        o.plan_out->streamed = pl.ok;
        o.plan_out->rows_per_tile = pl.ok ? (int)pl.p.R : 8;
        o.plan_out->warps = pl.ok ? (int)pl.p.NW : 8;
        o.plan_out->stages = pl.ok ? (int)pl.p.S : 0;
        o.plan_out->smem_bytes = pl.ok ? (int)pl.smem : 0;
        o.plan_out->grid = pl.ok ? pl.grid : (int)((out_dim + 7) / 8);
    }
    if (pl.ok) {
        pl.p.w = (const uint8_t *)d_w, pl.p.scales = (const uint8_t *)tb.scales, pl.p.biases = (const uint8_t *)tb.biases;
        pl.p.x = d_x, pl.p.y = d_y, pl.p.status = d_status;
        pl.p.norm_w = o.norm_w, pl.p.eps = o.eps, pl.p.epi = o.epi, pl.p.res = o.res;
        pl.p.pdl = o.pdl ? 1 : 0;
        pl.p.chunk = (uint32_t)g_stream_chunk;
        if (fmt == FMT_Q4K) return launch_stream_f<FMT_Q4K, float>(pl, st, o.pdl);
        if (fmt == FMT_Q6K) return launch_stream_f<FMT_Q6K, float>(pl, st, o.pdl);
        if (fmt == FMT_Q6KR) return launch_stream_f<FMT_Q6KR, float>(pl, st, o.pdl);
        if (tb.elem_bytes == 2) return launch_stream_f<FMT_MLX4, uint16_t>(pl, st, o.pdl);
        return launch_stream_f<FMT_MLX4, float>(pl, st, o.pdl);
    }
    if (fused || fmt == FMT_Q6KR) return cudaErrorNotSupported; // the plain kernel has no fused prologue / epilogue
    if (fmt == FMT_Q4K) return launch_generic_t<FMT_Q4K, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    if (fmt == FMT_Q6K) return launch_generic_t<FMT_Q6K, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    if (fmt == FMT_MLX4) {
        if (tb.elem_bytes == 2) return launch_generic_t<FMT_MLX4, uint16_t>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
        return launch_generic_t<FMT_MLX4, float>(d_w, tb, d_x, d_y, 0, out_dim, in_dim, st);
    }
    return cudaErrorInvalidValue;
}

bool matvec_is_streamed(const DeviceInfo &dev, int fmt, size_t out_dim, size_t in_dim, size_t group, int tbl_bytes,
                        int epi) {
    return plan_stream(dev, fmt, out_dim, in_dim, group, tbl_bytes, epi).ok;
}

} // namespace ullm
