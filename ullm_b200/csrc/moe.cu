// Mixture-of-experts SwiGLU FFN on MLX 4-bit stacked experts, for a few tokens
// at once (CPU form: crates/ullm-model/src/lib.rs:1453-1488; GPU form:
// crates/ullm-metal/src/forward.rs:484-494 with shader.metal:301-444).
//
// Four launches:
//   1. route   : per token, top-k experts by descending router logit (ties: lower
//                index first) and softmax over the selected logits; then the
//                (token, slot) pairs are grouped by expert so each distinct
//                expert's weights are read from HBM once for all tokens that
//                picked it.
//   2. gate_up : expert-gathered  hidden[pair] = silu(W_gate[e] x_t) * (W_up[e] x_t)
//   3. down    : expert-gathered  down[pair]   = W_down[e] hidden[pair]
//   4. combine : y[t] = sum over slots, in descending-logit order, of w * down
//                (the order the reference accumulates in, lib.rs:1479-1488).  A launch of its own on purpose:
//                folded into the down kernel's epilogue (a counter per token and row tile, the CTA that
//                finishes a token's last slot sums the k rows in slot order) it was measured slower on
//                B200, 90 us against 63 us for the benchmark's 8-token step, because every (expert, row tile)
//                unit then pays two CTA barriers and an atomic round trip.
// Kernels 2 and 3 are streamed like the dense matvec: persistent CTAs, each
// owning a contiguous range of (expert, row-tile) units so that it meets one or
// two experts only, weights and group tables arriving through a TMA-bulk ring;
// activations are re-expressed as 16-bit fixed point in shared memory per CTA
// and the products are integer dp4a sums scaled in fp32 (see matvec.cu).
// A plain gather kernel covers shapes the streamed layout rules exclude.
#include "kernels.h"
#include "matvec_core.cuh"

#include <algorithm>
#include <climits>

namespace ullm {

constexpr int MOE_MAX_TOK = 8;   // tokens per launch group
constexpr int MOE_MAX_K = 16;    // experts per token (reference kernel cap, shader.metal:310)
constexpr int MOE_MAX_EXPERTS = 1024;

// Layout of the routing scratch (ints): [0] D = number of distinct experts,
// [1 .. 1+E) expert ids ascending, [1+E .. 2+2E) pair offsets, then pair ids.
__host__ __device__ inline int route_off_list() { return 1; }
__host__ __device__ inline int route_off_offs(int E) { return 1 + E; }
__host__ __device__ inline int route_off_pairs(int E) { return 2 + 2 * E; }

// ---------------------------------------------------------------------------
// 1. routing
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_route_kernel(const float *__restrict__ logits, int n_tok, int n_exp, int k,
                                                       uint32_t *__restrict__ idx, float *__restrict__ wts,
                                                       int *__restrict__ route) {
    __shared__ __align__(16) float lg[MOE_MAX_TOK][MOE_MAX_EXPERTS];
    __shared__ int sel[MOE_MAX_TOK * MOE_MAX_K];
    __shared__ int cnt[MOE_MAX_EXPERTS];
    __shared__ int offs_s[MOE_MAX_EXPERTS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait_prior();
    // one warp per token (n_tok <= 8 = warps of the block)
    if (warp < n_tok) {
        const int t = warp;
        float *l = lg[t];
        for (int i = lane; i < n_exp; i += 32) l[i] = logits[(size_t)t * n_exp + i];
        __syncwarp();
        float mx = 0.f, wsum = 0.f, mine = 0.f;
        // Experts are ranked by the total order on f32 bit patterns (descending, lower index first among equal
        // patterns): the order the reference sorts by (total_cmp, lib.rs:1457).  It also ranks NaN, so a token
        // whose logits are all NaN still selects k distinct experts in range; its weights come out NaN, as in
        // the reference.  `taken` marks this lane's experts (bit m = expert lane + 32 m) already selected.
        uint32_t taken = 0u;
        for (int j = 0; j < k; ++j) {
            int bk = INT_MIN, bi = 0x7fffffff;
            for (int i = lane, m = 0; i < n_exp; i += 32, ++m) {
                if ((taken >> m) & 1u) continue;
                int key = __float_as_int(l[i]);
                key ^= (key >> 31) & 0x7fffffff;
                if (key > bk || (key == bk && i < bi)) bk = key, bi = i;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ok > bk || (ok == bk && oi < bi)) bk = ok, bi = oi;
            }
            // k <= n_exp (checked on the host), so an untaken expert always exists and bi is in range
            if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
            const float bv = l[bi];
            // softmax over the k selected logits (lib.rs:1460-1475): the first is the max
            if (j == 0) mx = bv;
            const float e = expf(bv - mx);
            wsum += e; // summed in selection order, identically in every lane
            if (lane == j) mine = e;
            if (lane == 0) sel[t * k + j] = bi;
        }
        __syncwarp();
        if (lane < k) {
            wts[t * k + lane] = mine / wsum;
            idx[t * k + lane] = (uint32_t)sel[t * k + lane];
        }
    }
    __syncthreads();
    // group the pairs by expert (ascending expert id, pairs in (token, slot) order): every pair sets its bit in
    // its expert's 128-bit mask; an expert's count is the mask's population and its pairs are the set bits in
    // ascending order, so nothing depends on the order in which the bits were set
    const int npairs = n_tok * k;
    unsigned long long(*mask)[2] = reinterpret_cast<unsigned long long(*)[2]>(&lg[0][0]); // the logits are spent: their 32 KB hold the masks
    for (int e = threadIdx.x; e < n_exp; e += blockDim.x) mask[e][0] = 0ull, mask[e][1] = 0ull;
    __syncthreads();
    for (int p = threadIdx.x; p < npairs; p += blockDim.x) atomicOr(&mask[sel[p]][p >> 6], 1ull << (p & 63));
    __syncthreads();
    for (int e = threadIdx.x; e < n_exp; e += blockDim.x) cnt[e] = __popcll(mask[e][0]) + __popcll(mask[e][1]);
    __syncthreads();
    int *list = route + route_off_list(), *offs = route + route_off_offs(n_exp), *pairs = route + route_off_pairs(n_exp);
    if (warp == 0) {
        // exclusive scan of the counts and of the "used" flags, 32 experts at a time
        int base_off = 0, base_d = 0;
        for (int e0 = 0; e0 < n_exp; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < n_exp ? cnt[e] : 0, u = c > 0;
            int so = c, sd = u;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int a = __shfl_up_sync(0xffffffffu, so, o), b2 = __shfl_up_sync(0xffffffffu, sd, o);
                if (lane >= o) so += a, sd += b2;
            }
            if (u) {
                const int d = base_d + sd - 1;
                list[d] = e;
                offs[d] = base_off + so - c;
                offs_s[e] = base_off + so - c;
            }
            base_off += __shfl_sync(0xffffffffu, so, 31);
            base_d += __shfl_sync(0xffffffffu, sd, 31);
        }
        if (lane == 0) {
            offs[base_d] = base_off;
            route[0] = base_d;
        }
    }
    __syncthreads();
    // each used expert writes its pairs, in (token, slot) order
    for (int e = threadIdx.x; e < n_exp; e += blockDim.x) {
        if (!cnt[e]) continue;
        int o = offs_s[e];
        for (int h = 0; h < 2; ++h)
            for (unsigned long long m = mask[e][h]; m; m &= m - 1) pairs[o++] = 64 * h + __ffsll((long long)m) - 1;
    }
}

// ---------------------------------------------------------------------------
// 2/3. streamed expert-gathered kernels
// ---------------------------------------------------------------------------
struct MoeStreamParams {
    // matrices of this launch: NM = 2 (gate, up) or 1 (down); stacked over experts
    const uint8_t *w[2], *sc[2], *bi[2];
    const float *act;  // gate_up: x [n_tok, in]; down: hidden [n_pairs, in]
    const float *norm_w; // gate_up only, may be null: RMSNorm weight applied to x first (x * inv * w, math.rs:82-86)
    float eps;
    float *out;        // gate_up: hidden [n_pairs, rows]; down: down_out [n_pairs, rows]
    const int *route;
    int *status;
    uint32_t n_exp, k, n_tok;
    uint32_t rows, in_dim, group; // per-expert matrix [rows, in_dim]
    uint32_t row_bytes, tbl_row_bytes;
    uint32_t R, NW, S, tiles_per_expert, ncg;
    uint32_t w_stage_bytes, tbl_stage_bytes, stage_bytes; // one matrix' regions; stage = NM * (w + 2 tbl)
    uint32_t off_route, off_q, off_ring; // byte offsets in dynamic shared memory
};

// GATE_UP: two matrices, x indexed by token, epilogue silu(g)*u.
// RW = rows per warp and tile (p.R / p.NW), a template parameter so that the per-row sums of a tile are reduced
// over the warp together (transposed butterfly) instead of one after the other.
template <bool GATE_UP, int G, typename TBL, int RW>
__global__ void __launch_bounds__(544, 1) moe_stream_kernel(const MoeStreamParams p) {
    constexpr int XR = XREGS_MLX, NM = GATE_UP ? 2 : 1;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + p.S;
    uint32_t *qimg = (uint32_t *)(smem + p.off_q); // [vec][cg][XR][32]
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
    pdl_launch_dependents();
    pdl_wait_prior(); // the routing table and the activations come from earlier kernels

    // The routing table goes to shared memory in one sweep (one round trip to L2 instead of one per
    // entry looked at): [0] D, expert ids, pair offsets, pair ids, then this CTA's first / end unit.
    int *rt_s = (int *)(smem + p.off_route);
    int *ex_list = rt_s + route_off_list(), *ex_off = rt_s + route_off_offs(p.n_exp), *pairs = rt_s + route_off_pairs(p.n_exp);
    const uint32_t n_route = (uint32_t)route_off_pairs(p.n_exp) + p.n_tok * p.k;
    uint32_t *u_s = (uint32_t *)(rt_s + route_off_pairs(p.n_exp) + MOE_MAX_TOK * MOE_MAX_K);
    for (uint32_t i = tid; i < n_route; i += blockDim.x) rt_s[i] = p.route[i];
    __syncthreads();
    const int D = rt_s[0];
    // Units (expert d, row tile rt), in that order, are dealt to the CTAs by COST, not by count: a
    // tile of an expert picked by np pairs costs np row passes (the arithmetic per pair is about
    // what the tile's transfer takes, so popular experts are compute-bound).  Unit (d, rt) sits at
    // cost position ex_off[d] * T + rt * np(d); CTA b owns the units whose position falls in its
    // equal share of the total npairs * T.  The first expert whose last tile lies at or beyond a cost
    // is found by a ballot over the experts (the bound grows with d); warps 0 and 1 do one end each.
    const uint32_t T = p.tiles_per_expert;
    if (warp < 2) {
        const uint64_t C = (uint64_t)ex_off[D] * T, c = C * (blockIdx.x + warp) / gridDim.x;
        uint32_t unit = (uint32_t)D * T;
        for (int d0 = 0; d0 < D; d0 += 32) {
            const int d = d0 + (int)lane;
            uint64_t base = 0, np = 1;
            bool hit = false;
            if (d < D) {
                base = (uint64_t)ex_off[d] * T, np = (uint64_t)(ex_off[d + 1] - ex_off[d]);
                hit = c <= base + (T - 1) * np;
            }
            const uint32_t m = __ballot_sync(0xffffffffu, hit);
            if (m) {
                const int first = __ffs(m) - 1;
                const uint32_t mine = (uint32_t)d * T + (c <= base ? 0u : (uint32_t)((c - base + np - 1) / np));
                unit = __shfl_sync(0xffffffffu, mine, first);
                break;
            }
        }
        if (lane == 0) u_s[warp] = unit;
    }
    __syncthreads();
    const uint32_t u0 = u_s[0], u1 = u_s[1];

    if (producer) {
        if (lane == 0) {
            uint32_t kk = 0;
            for (uint32_t u = u0; u < u1; ++u, ++kk) {
                const uint32_t s = kk % p.S;
                if (kk >= p.S && !wait_or_timeout(&empty[s], ((kk / p.S) - 1) & 1)) {
                    *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                const uint32_t d = u / p.tiles_per_expert, rt = u % p.tiles_per_expert;
                const uint32_t e = (uint32_t)ex_list[d], r0 = rt * p.R;
                const uint32_t nrows = min(p.R, p.rows - r0);
                const uint32_t wb = nrows * p.row_bytes, tb = nrows * p.tbl_row_bytes;
                const size_t grow = (size_t)e * p.rows + r0;
                uint8_t *dst = ring + (size_t)s * p.stage_bytes;
                mbar_arrive_expect_tx(&full[s], NM * (wb + 2 * tb));
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    uint8_t *dm = dst + m * (p.w_stage_bytes + 2 * p.tbl_stage_bytes);
                    bulk_g2s(dm, p.w[m] + grow * p.row_bytes, wb, &full[s]);
                    bulk_g2s(dm + p.w_stage_bytes, p.sc[m] + grow * p.tbl_row_bytes, tb, &full[s]);
                    bulk_g2s(dm + p.w_stage_bytes + p.tbl_stage_bytes, p.bi[m] + grow * p.tbl_row_bytes, tb, &full[s]);
                }
            }
        }
        return;
    }

    const uint32_t nthr_c = p.NW * 32; // consumer threads (named barrier 1)
    // Fixed-point images of several activation vectors are built side by side, one group of warps per
    // vector, so that their loads are in flight together.
    const uint32_t pg_thr = max(32u, (nthr_c / max(1u, GATE_UP ? p.n_tok : 4u)) & ~31u), pg_n = nthr_c / pg_thr;
    const uint32_t pg = tid / pg_thr, pg_tid = tid % pg_thr; // pg >= pg_n: a leftover warp, idle here
    if (GATE_UP) {
        // every token's x, once per CTA; with a norm weight the vector is RMS-normalised on the way (every CTA
        // recomputes the few KB's mean square, which saves a kernel in front of this one)
        float *ss_s = (float *)(u_s + 2); // 32 floats behind the unit bounds
        if (p.norm_w) {
            float ss = 0.f;
            for (uint32_t t = pg; t < p.n_tok && pg < pg_n; t += pg_n) { // n_tok <= pg_n: at most one token per group
                const float4 *xv = (const float4 *)(p.act + (size_t)t * p.in_dim);
                for (uint32_t i = pg_tid; i < p.in_dim / 4; i += pg_thr) {
                    const float4 a = __ldg(xv + i);
                    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) ss_s[warp] = ss;
            asm volatile("bar.sync 1, %0;" ::"r"(nthr_c) : "memory");
        }
        for (uint32_t t = pg; t < p.n_tok && pg < pg_n; t += pg_n) {
            float inv = 0.f;
            if (p.norm_w) {
                float tot = 0.f;
                for (uint32_t w = pg * (pg_thr / 32); w < (pg + 1) * (pg_thr / 32); ++w) tot += ss_s[w];
                inv = 1.0f / sqrtf(tot / (float)p.in_dim + p.eps);
            }
            prep_image<FMT_MLX4>(ActSrc{p.act + (size_t)t * p.in_dim, p.norm_w, inv}, p.in_dim, qimg + (size_t)t * p.ncg * XR * 32, pg_tid,
                                 pg_thr);
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthr_c) : "memory");
    }

    bool aborted = false;
    int cur_d = -1;
    uint32_t kk = 0;
    const int kshift = (p.k & (p.k - 1u)) == 0u ? 31 - __clz((int)p.k) : -1; // experts per token is usually a power of two
    // The register image of the current activation vector survives from tile to tile: most experts
    // are picked by a single pair, and then all row tiles of the expert use the same vector.
    uint32_t X[G][XR];
    int loaded_vec = -1;
    // the tile loop divides nothing: stage, mbarrier phase, expert and row tile are carried along
    uint32_t s = 0, ph = 0, d = u0 / p.tiles_per_expert, rt = u0 % p.tiles_per_expert;
    for (uint32_t u = u0; u < u1; ++u, ++kk, s = s + 1 == p.S ? 0 : s + 1, ph ^= (s == 0), rt = rt + 1 == p.tiles_per_expert ? 0 : rt + 1, d += (rt == 0)) {
        const uint32_t r0 = rt * p.R;
        const int pb = ex_off[d], np = ex_off[d + 1] - pb;
        if (!GATE_UP && (int)d != cur_d) {
            // new expert: fixed-point images of the hidden vectors of its pairs
            asm volatile("bar.sync 1, %0;" ::"r"(nthr_c) : "memory"); // everyone done with the previous images
            for (int j = (int)pg; j < np && pg < pg_n; j += (int)pg_n)
                prep_image<FMT_MLX4>(ActSrc{p.act + (size_t)pairs[pb + j] * p.in_dim, nullptr, 0.f}, p.in_dim,
                                     qimg + (size_t)j * p.ncg * XR * 32, pg_tid, pg_thr);
            asm volatile("bar.sync 1, %0;" ::"r"(nthr_c) : "memory");
            loaded_vec = -1; // the images were rebuilt
        }
        cur_d = (int)d;
        if (!aborted && !wait_or_timeout(&full[s], ph)) aborted = true;
        const uint32_t stage = smem_u32(ring + (size_t)s * p.stage_bytes);
        const uint32_t mstride = p.w_stage_bytes + 2 * p.tbl_stage_bytes;
        for (int j = 0; j < np && !aborted; ++j) {
            const int pair = pairs[pb + j];
            const uint32_t vec = GATE_UP ? (kshift >= 0 ? (uint32_t)pair >> kshift : (uint32_t)pair / p.k) : (uint32_t)j; // the pair's token
            if ((int)vec != loaded_vec) {
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int q = 0; q < XR; ++q)
                        X[g][q] = (uint32_t)g < p.ncg ? qimg[((size_t)(vec * p.ncg + g) * XR + q) * 32 + lane] : 0u;
                loaded_vec = (int)vec;
            }
            constexpr int NV = RW * NM; // partial sums of this warp's rows (gate and up of a row side by side)
            float v[NV];
#pragma unroll
            for (int rr = 0; rr < RW; ++rr) {
                const uint32_t rl = warp * RW + rr;
#pragma unroll
                for (int m = 0; m < NM; ++m) {
                    float a = 0.f;
                    if (r0 + rl < p.rows) {
                        const uint32_t base = stage + m * mstride;
                        const uint32_t ts = base + p.w_stage_bytes + rl * p.tbl_row_bytes;
#pragma unroll
                        for (int g = 0; g < G; ++g)
                            if ((uint32_t)g < p.ncg && (g * 32u + lane) * 32u < p.in_dim)
                                a += row_partial<FMT_MLX4, TBL>(base + rl * p.row_bytes, X[g], g, lane, ts, ts + p.tbl_stage_bytes, p.group);
                    }
                    v[rr * NM + m] = a;
                }
            }
            if constexpr (NV <= 4) {
                // after the call the lanes with (bit 4, bit 3) = (i / 2, i % 2) [NV = 4] or bit 4 = i [NV = 2] hold sum i
                uint32_t idx;
                const float r = warp_reduce_rows<NV>(v, lane, idx);
                const float other = GATE_UP ? __shfl_xor_sync(0xffffffffu, r, NV == 4 ? 8 : 16) : 0.f; // the row's up sum
                const uint32_t rr = GATE_UP ? idx >> 1 : idx, rl = warp * RW + rr;
                const bool writer = (lane & (NV == 4 ? 7 : 15)) == 0 && (NV > 1 || lane == 0) && (!GATE_UP || (idx & 1) == 0);
                if (writer && r0 + rl < p.rows)
                    p.out[(size_t)pair * p.rows + r0 + rl] = GATE_UP ? r / (1.0f + expf(-r)) * other : r; // math.rs:103-105, lib.rs:1482
            } else {
#pragma unroll
                for (int rr = 0; rr < RW; ++rr) {
                    const float g0 = warp_sum(v[rr * NM]), u0 = NM > 1 ? warp_sum(v[rr * NM + NM - 1]) : 0.f;
                    const uint32_t rl = warp * RW + rr;
                    if (lane == 0 && r0 + rl < p.rows) p.out[(size_t)pair * p.rows + r0 + rl] = GATE_UP ? g0 / (1.0f + expf(-g0)) * u0 : g0;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (aborted && lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
}

// ---------------------------------------------------------------------------
// Plain gather kernels (any shape the format allows): one warp per (pair, row)
// ---------------------------------------------------------------------------
template <typename TBL>
__device__ __forceinline__ float mlx_row_dot(const uint32_t *__restrict__ row, const TBL *__restrict__ sc,
                                             const TBL *__restrict__ bi, const float *__restrict__ x, uint32_t in_dim,
                                             uint32_t group, uint32_t lane) {
    float acc = 0.f;
    const uint32_t words = in_dim / 8;
    for (uint32_t wi = lane; wi < words; wi += 32) {
        uint32_t q = row[wi];
        uint32_t g = (wi * 8) / group;
        float s = tbl_load<TBL>(sc + g), b = tbl_load<TBL>(bi + g);
        const float4 xa = *(const float4 *)(x + wi * 8), xb = *(const float4 *)(x + wi * 8 + 4);
        float dot = (float)(q & 15) * xa.x + (float)((q >> 4) & 15) * xa.y + (float)((q >> 8) & 15) * xa.z +
                    (float)((q >> 12) & 15) * xa.w + (float)((q >> 16) & 15) * xb.x + (float)((q >> 20) & 15) * xb.y +
                    (float)((q >> 24) & 15) * xb.z + (float)(q >> 28) * xb.w;
        acc += s * dot + b * (xa.x + xa.y + xa.z + xa.w + xb.x + xb.y + xb.z + xb.w);
    }
    return warp_sum(acc);
}

template <bool GATE_UP, typename TBL>
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint32_t *__restrict__ w0, const TBL *__restrict__ s0,
                                                        const TBL *__restrict__ b0, const uint32_t *__restrict__ w1,
                                                        const TBL *__restrict__ s1, const TBL *__restrict__ b1,
                                                        const float *__restrict__ act, float *__restrict__ out,
                                                        const uint32_t *__restrict__ idx, uint32_t k, uint32_t rows,
                                                        uint32_t in_dim, uint32_t group) {
    const uint32_t lane = threadIdx.x & 31, pair = blockIdx.y;
    const uint32_t o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= rows) return;
    const uint32_t e = idx[pair];
    const size_t grow = (size_t)e * rows + o, words = in_dim / 8, groups = in_dim / group;
    const float *x = act + (size_t)(GATE_UP ? pair / k : pair) * in_dim;
    float a = mlx_row_dot<TBL>(w0 + grow * words, s0 + grow * groups, b0 + grow * groups, x, in_dim, group, lane);
    if (GATE_UP) {
        float u = mlx_row_dot<TBL>(w1 + grow * words, s1 + grow * groups, b1 + grow * groups, x, in_dim, group, lane);
        a = a / (1.0f + expf(-a)) * u;
    }
    if (lane == 0) out[(size_t)pair * rows + o] = a;
}

// 4. y[t][o] = sum_slot wts[t][slot] * down[t*k+slot][o]   (lib.rs:1484-1487)
__global__ void moe_combine_kernel(const float *__restrict__ down, const float *__restrict__ wts, float *__restrict__ y,
                                   uint32_t n_tok, uint32_t k, uint32_t hidden, const float *__restrict__ res) {
    pdl_wait_prior();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tok * hidden) return;
    const uint32_t t = i / hidden, o = i % hidden;
    float acc = 0.f;
    for (uint32_t s = 0; s < k; ++s) acc += wts[t * k + s] * down[((size_t)t * k + s) * hidden + o];
    y[i] = res ? res[i] + acc : acc; // the residual stream's `x += down` (lib.rs:959-961) when asked for
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
static inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

struct MoePlanInt {
    bool ok = false;
    MoeStreamParams p{};
    int g = 1, grid = 0, threads = 0;
    uint32_t smem = 0;
};

static MoePlanInt plan_moe(const DeviceInfo &dev, bool gate_up, uint32_t rows, uint32_t in_dim, uint32_t group,
                           int tbl_bytes, uint32_t n_vec, uint32_t n_exp) {
    MoePlanInt best;
    if (in_dim % 32 || group % 32 || in_dim % group) return best;
    const uint32_t NM = gate_up ? 2 : 1;
    const uint32_t row_bytes = in_dim / 2, tbl_row_bytes = (in_dim / group) * tbl_bytes;
    const uint32_t ncg = (in_dim + 1023) / 1024;
    if (ncg > 4) return best;
    const uint32_t G = ncg <= 1 ? 1 : (ncg <= 2 ? 2 : 4);
    const uint32_t NW = 16;
    const int budget = dev.max_smem_optin - 1024;
    const uint32_t off_route = 128; // routing table + the CTA's two unit bounds
    const uint32_t off_q = align_up(off_route + ((uint32_t)route_off_pairs((int)n_exp) + MOE_MAX_TOK * MOE_MAX_K + 2 + 32) * 4, 128); // + per-warp sums of squares
    const uint32_t off_ring = align_up(off_q + n_vec * ncg * XREGS_MLX * 32 * 4, 128);
    for (uint32_t RW = 1; RW <= 4; RW *= 2) {
        const uint32_t R = NW * RW;
        if ((R * row_bytes) % 16 || (R * tbl_row_bytes) % 16) continue;
        if (rows % R && ((row_bytes % 16) || (tbl_row_bytes % 16))) continue;
        const uint32_t wst = align_up(R * row_bytes, 128), tst = align_up(R * tbl_row_bytes, 128);
        const uint32_t stage = NM * (wst + 2 * tst);
        if (stage > 100 * 1024 && best.ok) continue;
        if ((int)(off_ring + 2 * stage) > budget) continue;
        const uint32_t S = std::min<uint32_t>(8, (budget - off_ring) / stage);
        // prefer ~16-36 KB stages
        if (best.ok && stage > 100 * 1024) continue;
        best.ok = true;
        best.g = (int)G;
        best.threads = (int)(NW + 1) * 32;
        best.grid = dev.sm_count;
        best.smem = off_ring + S * stage;
        MoeStreamParams &p = best.p;
        p.rows = rows, p.in_dim = in_dim, p.group = group, p.row_bytes = row_bytes, p.tbl_row_bytes = tbl_row_bytes;
        p.R = R, p.NW = NW, p.S = S, p.tiles_per_expert = (rows + R - 1) / R, p.ncg = ncg;
        p.w_stage_bytes = wst, p.tbl_stage_bytes = tst, p.stage_bytes = stage;
        p.off_route = off_route, p.off_q = off_q, p.off_ring = off_ring;
    }
    return best;
}

template <bool GATE_UP, int G, typename TBL, int RW> static cudaError_t launch_moe_t(const MoePlanInt &pl, cudaStream_t st, bool pdl) {
    auto kfn = moe_stream_kernel<GATE_UP, G, TBL, RW>;
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
template <bool GATE_UP, int G, typename TBL> static cudaError_t launch_moe_r(const MoePlanInt &pl, cudaStream_t st, bool pdl) {
    const uint32_t rw = pl.p.R / pl.p.NW;
    if (rw == 1) return launch_moe_t<GATE_UP, G, TBL, 1>(pl, st, pdl);
    if (rw == 2) return launch_moe_t<GATE_UP, G, TBL, 2>(pl, st, pdl);
    return launch_moe_t<GATE_UP, G, TBL, 4>(pl, st, pdl);
}
template <bool GATE_UP, typename TBL> static cudaError_t launch_moe_g(const MoePlanInt &pl, cudaStream_t st, bool pdl) {
    if (pl.g == 1) return launch_moe_r<GATE_UP, 1, TBL>(pl, st, pdl);
    if (pl.g == 2) return launch_moe_r<GATE_UP, 2, TBL>(pl, st, pdl);
    return launch_moe_r<GATE_UP, 4, TBL>(pl, st, pdl);
}

size_t moe_scratch_bytes(const MoeExperts &e) {
    const size_t pairs = (size_t)MOE_MAX_TOK * MOE_MAX_K;
    size_t route = (size_t)(route_off_pairs((int)e.n_experts) + pairs) * 4;
    route = (route + 255) / 256 * 256;
    return route + pairs * e.inter * 4 + pairs * e.hidden * 4 + pairs * 8 + 1024;
}

const char *moe_shape_error(const MoeExperts &e, size_t n_tok, size_t k) {
    if (e.n_experts == 0 || e.n_experts > MOE_MAX_EXPERTS) return "number of experts must be 1..1024";
    if (k == 0 || k > MOE_MAX_K || k > e.n_experts) return "experts per token must be 1..16 and <= n_experts";
    if (n_tok == 0) return "no tokens";
    if (e.hidden % 8 || e.inter % 8 || e.group == 0 || e.group % 8 || e.hidden % e.group || e.inter % e.group)
        return "hidden / inter must be multiples of the group size, group a multiple of 8";
    return nullptr;
}

cudaError_t launch_moe_ffn(const DeviceInfo &dev, const MoeExperts &e, const float *d_x, const float *d_logits,
                           size_t n_tok, size_t k, float *d_y, uint32_t *d_idx, float *d_wts, void *d_scratch,
                           int *d_status, cudaStream_t st, bool force_generic, bool pdl, int *streamed_out, const float *d_res,
                           const float *d_norm_w, float eps) {
    // scratch carve-up
    const size_t pairs_cap = (size_t)MOE_MAX_TOK * MOE_MAX_K;
    uint8_t *sp = (uint8_t *)d_scratch;
    int *route = (int *)sp;
    size_t route_b = ((size_t)(route_off_pairs((int)e.n_experts) + pairs_cap) * 4 + 255) / 256 * 256;
    float *hidden = (float *)(sp + route_b);
    float *down = hidden + pairs_cap * e.inter;
    uint32_t *idx_s = (uint32_t *)(down + pairs_cap * e.hidden);
    float *wts_s = (float *)(idx_s + pairs_cap);
    const uint32_t tb = (uint32_t)e.table_bytes;
    // both the streamed and the plain kernels read x with 128-bit loads: callers check this before launching
    if ((uintptr_t)d_x % 16 || (uintptr_t)d_y % 4 || (uintptr_t)d_logits % 4) return cudaErrorMisalignedAddress;
    if (streamed_out) *streamed_out = 0;

    for (size_t t0 = 0; t0 < n_tok; t0 += MOE_MAX_TOK) {
        const uint32_t nt = (uint32_t)std::min<size_t>(MOE_MAX_TOK, n_tok - t0), npairs = nt * (uint32_t)k;
        const float *x = d_x + t0 * e.hidden;
        uint32_t *idx = d_idx ? d_idx + t0 * k : idx_s;
        float *wts = d_wts ? d_wts + t0 * k : wts_s;
        // the small kernels take part in the programmatic-dependent chain as well (both wait for their
        // predecessor with griddepcontrol.wait before they read anything it wrote)
        cudaLaunchAttribute pat[1];
        pat[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pat[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t rc_cfg = {};
        rc_cfg.gridDim = dim3(1), rc_cfg.blockDim = dim3(256), rc_cfg.stream = st, rc_cfg.attrs = pat, rc_cfg.numAttrs = pdl ? 1 : 0;
        cudaError_t err = cudaLaunchKernelEx(&rc_cfg, moe_route_kernel, d_logits + t0 * e.n_experts, (int)nt, (int)e.n_experts, (int)k, idx,
                                             wts, route);
        if (err != cudaSuccess) return err;

        MoePlanInt pg, pd;
        if (!force_generic) {
            pg = plan_moe(dev, true, (uint32_t)e.inter, (uint32_t)e.hidden, (uint32_t)e.group, (int)tb, nt, (uint32_t)e.n_experts);
            pd = plan_moe(dev, false, (uint32_t)e.hidden, (uint32_t)e.inter, (uint32_t)e.group, (int)tb, nt, (uint32_t)e.n_experts);
        }
        if (pg.ok && pd.ok) {
            if (streamed_out) *streamed_out = 1;
            MoeStreamParams &a = pg.p;
            a.w[0] = (const uint8_t *)e.gate_w, a.sc[0] = (const uint8_t *)e.gate_s, a.bi[0] = (const uint8_t *)e.gate_b;
            a.w[1] = (const uint8_t *)e.up_w, a.sc[1] = (const uint8_t *)e.up_s, a.bi[1] = (const uint8_t *)e.up_b;
            a.act = x, a.norm_w = d_norm_w, a.eps = eps, a.out = hidden, a.route = route, a.status = d_status;
            a.n_exp = (uint32_t)e.n_experts, a.k = (uint32_t)k, a.n_tok = nt;
            err = tb == 2 ? launch_moe_g<true, uint16_t>(pg, st, pdl) : launch_moe_g<true, float>(pg, st, pdl);
            if (err != cudaSuccess) return err;
            MoeStreamParams &b = pd.p;
            b.w[0] = (const uint8_t *)e.down_w, b.sc[0] = (const uint8_t *)e.down_s, b.bi[0] = (const uint8_t *)e.down_b;
            b.w[1] = nullptr, b.sc[1] = nullptr, b.bi[1] = nullptr;
            b.act = hidden, b.norm_w = nullptr, b.eps = 0.f, b.out = down, b.route = route, b.status = d_status;
            b.n_exp = (uint32_t)e.n_experts, b.k = (uint32_t)k, b.n_tok = nt;
            err = tb == 2 ? launch_moe_g<false, uint16_t>(pd, st, pdl) : launch_moe_g<false, float>(pd, st, pdl);
            if (err != cudaSuccess) return err;
        } else {
            if (d_norm_w) return cudaErrorNotSupported; // the plain kernels take the vector as it is
            dim3 g1((unsigned)((e.inter + 7) / 8), npairs), g2((unsigned)((e.hidden + 7) / 8), npairs);
            if (tb == 2) {
                moe_gather_kernel<true, uint16_t><<<g1, 256, 0, st>>>(
                    (const uint32_t *)e.gate_w, (const uint16_t *)e.gate_s, (const uint16_t *)e.gate_b,
                    (const uint32_t *)e.up_w, (const uint16_t *)e.up_s, (const uint16_t *)e.up_b, x, hidden, idx,
                    (uint32_t)k, (uint32_t)e.inter, (uint32_t)e.hidden, (uint32_t)e.group);
                moe_gather_kernel<false, uint16_t><<<g2, 256, 0, st>>>(
                    (const uint32_t *)e.down_w, (const uint16_t *)e.down_s, (const uint16_t *)e.down_b, nullptr, nullptr,
                    nullptr, hidden, down, idx, (uint32_t)k, (uint32_t)e.hidden, (uint32_t)e.inter, (uint32_t)e.group);
            } else {
                moe_gather_kernel<true, float><<<g1, 256, 0, st>>>(
                    (const uint32_t *)e.gate_w, (const float *)e.gate_s, (const float *)e.gate_b,
                    (const uint32_t *)e.up_w, (const float *)e.up_s, (const float *)e.up_b, x, hidden, idx, (uint32_t)k,
                    (uint32_t)e.inter, (uint32_t)e.hidden, (uint32_t)e.group);
                moe_gather_kernel<false, float><<<g2, 256, 0, st>>>(
                    (const uint32_t *)e.down_w, (const float *)e.down_s, (const float *)e.down_b, nullptr, nullptr, nullptr,
                    hidden, down, idx, (uint32_t)k, (uint32_t)e.hidden, (uint32_t)e.inter, (uint32_t)e.group);
            }
            if ((err = cudaGetLastError()) != cudaSuccess) return err;
        }
        const uint32_t n = nt * (uint32_t)e.hidden;
        rc_cfg.gridDim = dim3((n + 255) / 256);
        err = cudaLaunchKernelEx(&rc_cfg, moe_combine_kernel, (const float *)down, (const float *)wts, d_y + t0 * e.hidden, nt, (uint32_t)k,
                                 (uint32_t)e.hidden, (const float *)(d_res ? d_res + t0 * e.hidden : nullptr));
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

} // namespace ullm
