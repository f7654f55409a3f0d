// A list of matvecs in ONE persistent launch (Q4_K and prepared Q6_K weights).
//
// A decode step is a chain of small dependent matvecs: W_o, gate|up, down, the next layer's
// q|k and v ... (crates/ullm-model/src/lib.rs:807-969).  Launched one kernel each, every
// link pays the fixed cost of a launch: the grid drains, the next grid starts, its first
// weight tiles take a DRAM round trip, and only then does the stream run — 4-5 us against
// 0.5-3 us of streaming for matrices of 2-19 MB.  Here the grid stays resident (one CTA per
// SM) and walks the whole list:
//   * the producer warp of every CTA streams the tiles of op 0, op 1, ... back to back
//     through one shared-memory ring — weights do not depend on activations, so the stream
//     never stops at an op boundary;
//   * ops that do not depend on each other are not walked by every CTA: the CTAs are dealt out to
//     the ops in proportion to their bytes, so a CTA prepares the image of one activation vector
//     and streams one matrix' rows for the whole launch (an op's input vector has to be read and
//     converted by every CTA that touches the op, whatever its share of the rows, which is what a
//     launch over many small row slices otherwise spends its time on);
//   * the consumer warps do, per op, what matvec_stream_kernel does (matvec.cu): fixed-point
//     image of x in registers, dp4a row sums, optional RMSNorm prologue and residual / SwiGLU
//     epilogue — and wait at a grid-wide barrier only where an op reads what an earlier op
//     of the same launch wrote;
//   * that barrier is an atomic counter in global memory with a bounded, sleeping spin; a list
//     that uses it is launched cooperatively, so the driver guarantees that all CTAs (one per SM)
//     are resident together (if the wait still expires the kernel records DEV_TIMEOUT, stops
//     computing and walks out through its barriers).
#include "kernels.h"
#include "matvec_core.cuh"
#include "shard_dev.cuh"

#include <algorithm>

namespace ullm {

constexpr int CHAIN_MAX_OPS = 12;
constexpr int CHAIN_MAX_STAGES = 8;
// L2 prefetch distance in tiles.  Off: measured on B200 it slows the c4 step (121 us without, 136 / 149 / 155 us at
// 2 / 4 / 8 tiles ahead): the prefetches compete with the ring's own copies for DRAM and do not come back as hits.
static int g_pf_tiles = 0;
void matvec_chain_set_prefetch(int v) { g_pf_tiles = v < 0 ? 0 : v; }
// Bytes per bulk copy of the producer warp (a tile is copied as pieces of this size, one per lane and round).
// 16 KB: the 70B block measured 127.5 / 111.4 / 107.5 / 107.0 / 106.9 / 106.8 us per step at 2 / 4 / 8 / 16 / 32 / 128 KB.
static int g_overlap_image = 1;
void matvec_chain_set_overlap(int v) { g_overlap_image = v; }
static int g_chain_chunk = 16384;
void matvec_chain_set_chunk(int bytes) { g_chain_chunk = bytes >= 1024 ? bytes / 16 * 16 : 16384; }
static double g_q6k_cost = 1.05; // relative cost per byte of prepared Q6_K rows when CTAs are dealt out to ops
void matvec_chain_set_q6k_cost(double v) { g_q6k_cost = v; }

struct ChainOpDev {
    const uint8_t *w;
    const float *x;      // [in_dim]
    float *y;            // [out_dim] (EPI_SWIGLU: [out_dim / 2])
    const float *norm_w; // prologue: x <- rmsnorm(x, norm_w, eps) when set
    const float *res;    // EPI_RESIDUAL
    float eps;
    int epi, fmt;
    int dep;             // x / res come from an earlier op of this launch: grid barrier first
    uint32_t out_dim, in_dim, row_bytes, gran, ncg;
    uint32_t R, WC, WR, rw, g; // tile rows, column-group warps, row-slice warps, rows per warp, groups per warp
    uint32_t cta0, ncta;       // the CTAs [cta0, cta0 + ncta) share this op's rows; the others skip it
    // shared-memory layout while this op runs: the same for every op when all CTAs walk the whole list (the ring
    // then runs on across ops), the op's own when the CTAs are dealt out (a CTA then sees one op only)
    uint32_t S, stage_bytes, off_part, off_prep, off_ring;
    // Dealt CTAs only: ring stages from this one on lie over the activation image (which is dead once the consumers
    // hold it in registers); the producer fills them for the first time after the consumers have said so.  S: none.
    uint32_t late_stage;
    uint32_t gather_off, gather_len; // sharded launch: the op's whole vector in the gather buffer (floats)
};
struct ChainParams {
    ChainOpDev op[CHAIN_MAX_OPS];
    int n_ops;
    unsigned *sync; // {arrival count, generation}: zero once, self-restoring
    int *status;
    uint32_t NW, chunk;
    uint32_t pf_tiles; // tiles the producer keeps requested in the L2 ahead of the ring's own copies
    ShardDev sh; // sh.world > 0: rows go to every rank's gather buffer and the launch publishes the exchange
};

__device__ __forceinline__ void chain_row_range(const ChainOpDev &o, uint32_t &rbeg, uint32_t &rend) {
    const uint32_t b = blockIdx.x - o.cta0; // wraps to a large value for CTAs in front of the op's group
    if (b >= o.ncta) {
        rbeg = rend = 0;
        return;
    }
    const uint32_t units = o.out_dim / o.gran;
    rbeg = (uint32_t)(((uint64_t)units * b) / o.ncta) * o.gran;
    rend = b + 1 == o.ncta ? o.out_dim : (uint32_t)(((uint64_t)units * (b + 1)) / o.ncta) * o.gran;
}

// Grid-wide barrier of the consumer threads.  sync[0] counts arrivals, sync[1] is the generation:
// the last CTA to arrive clears the count and then bumps the generation, the others wait for the
// bump.  The words return to (0, g+1), so launches need no reset between them (after a timeout
// the host clears them).  Bounded: about a second of sleeping polls.
__device__ __forceinline__ bool chain_grid_sync(unsigned *sync, uint32_t nthr_c, uint32_t tid, int *ok_s) {
    asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory"); // this CTA's stores of the earlier ops are issued
    if (tid == 0) {
        unsigned g;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(sync + 1) : "memory");
        __threadfence();
        int ok = 1;
        if (atomicAdd(sync, 1u) == gridDim.x - 1) {
            atomicExch(sync, 0u);
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sync + 1), "r"(g + 1) : "memory");
        } else {
            const long long t0 = clock64();
            for (;;) {
                unsigned v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sync + 1) : "memory");
                if (v != g) break;
                asm volatile("nanosleep.u32 40;" ::: "memory");
                if (clock64() - t0 > (1ll << 31)) {
                    ok = 0;
                    break;
                }
            }
        }
        *ok_s = ok;
        __threadfence();
    }
    asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
    return *ok_s != 0;
}

// One op, consumer side.  kbase = number of tiles this CTA has streamed before this op.
template <int FMT, int RW, int G>
__device__ __forceinline__ void chain_consume(const ChainOpDev &o, const ChainParams &p, uint8_t *smem, uint32_t kbase,
                                              uint32_t tid, bool &aborted) {
    constexpr int XR = FmtTraits<FMT>::XREGS;
    uint64_t *full = (uint64_t *)smem, *empty = full + CHAIN_MAX_STAGES;
    float *part = (float *)(smem + o.off_part);
    uint32_t *prep = (uint32_t *)(smem + o.off_prep);
    uint8_t *ring = smem + o.off_ring;
    const uint32_t warp = tid >> 5, lane = tid & 31, nthr_c = p.NW * 32;
    uint32_t rbeg, rend;
    chain_row_range(o, rbeg, rend);
    const uint32_t ntiles = (rend - rbeg + o.R - 1) / o.R;

    // ---- x: optional RMSNorm (math.rs:82-86), then the fixed-point register image ----
    ActSrc src{o.x, o.norm_w, 0.f};
    if (o.norm_w) {
        float ss = 0.f;
        for (uint32_t t = tid; t < (o.in_dim >> 3); t += nthr_c) {
            const float4 a = __ldcg((const float4 *)(o.x + 8 * t)), b = __ldcg((const float4 *)(o.x + 8 * t + 4));
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) part[warp] = ss;
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
        float tot = 0.f;
        for (uint32_t w = 0; w < p.NW; ++w) tot += part[w];
        src.inv = 1.0f / sqrtf(tot / (float)o.in_dim + o.eps);
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory"); // part is reused below
    }
    prep_image<FMT>(src, o.in_dim, prep, tid, nthr_c);
    asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");

    const bool active = warp < o.WC * o.WR; // the op may use fewer warps than the launch has
    const uint32_t rs = warp / o.WC, cgw = warp % o.WC;
    uint32_t X[G][XR];
    bool live[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint32_t cg = cgw + g * o.WC;
        live[g] = active && cg < o.ncg && (cg * 8u + (lane >> 2)) * QK_K < o.in_dim;
#pragma unroll
        for (int k = 0; k < XR; ++k) X[g][k] = live[g] ? prep[((size_t)cg * XR + k) * 32 + lane] : 0u;
    }
    const uint32_t nb = o.in_dim / QK_K;
    if (o.late_stage < o.S) { // the image may be overwritten by weight tiles from here on
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic accesses to the image before the bulk copies over it
        __syncwarp();
        if (lane == 0) mbar_arrive((uint64_t *)(smem + 136));
    }

    // sums the column-group partials of tile kt (see matvec.cu); slot = kt mod 2S names its partial area
    auto flush = [&](uint32_t kt, uint32_t slot) {
        if (!active || cgw != 0 || lane >= RW) return;
        const float *pt = part + ((size_t)slot * o.R) * o.WC;
        const uint32_t row = rs * RW + lane, gr = rbeg + kt * o.R + row;
        if (gr >= rend || aborted) return;
        float acc = 0.f;
        for (uint32_t c = 0; c < o.WC; ++c) acc += pt[row * o.WC + c];
        if (o.epi == EPI_STORE) o.y[gr] = acc;
        else if (o.epi == EPI_RESIDUAL) o.y[gr] = __ldcg(o.res + gr) + acc;
        else if ((lane & 1) == 0) {
            float up = 0.f;
            for (uint32_t c = 0; c < o.WC; ++c) up += pt[(row + 1) * o.WC + c];
            o.y[gr >> 1] = acc / (1.0f + expf(-acc)) * up;
        }
    };
    // ring stage and mbarrier phase of the op's first tile (the ring runs on across ops), then carried along;
    // slot = k mod 2S for the partial areas, which are the op's own
    uint32_t s = kbase % o.S, ph = (kbase / o.S) & 1u, slot = 0;
    for (uint32_t k = 0; k < ntiles; ++k, slot = slot + 1 == 2 * o.S ? 0 : slot + 1) {
        if (k) {
            if (++s == o.S) s = 0, ph ^= 1u;
        }
        if (!aborted && !wait_or_timeout(&full[s], ph)) aborted = true;
        if (o.WC > 1 && k >= o.S) flush(k - o.S, slot >= o.S ? slot - o.S : slot + o.S);
        const uint32_t stage = smem_u32(ring + (size_t)s * o.stage_bytes);
        const uint32_t r0 = rbeg + k * o.R;
        if (active) {
            float v[RW];
#pragma unroll
            for (int rr = 0; rr < RW; ++rr) {
                v[rr] = 0.f;
                const uint32_t rl = rs * RW + rr;
                if (!aborted && r0 + rl < rend) {
                    const uint32_t row_addr = stage + rl * o.row_bytes;
                    const uint32_t ts = row_addr + 192u * nb, tb2 = row_addr + 208u * nb; // prepared Q6_K planes
#pragma unroll
                    for (int g = 0; g < G; ++g)
                        if (live[g]) v[rr] += row_partial<FMT, float>(row_addr, X[g], cgw + g * o.WC, lane, ts, tb2, 0u);
                }
            }
            uint32_t myrow;
            const float r = warp_reduce_rows<RW>(v, lane, myrow);
            const uint32_t rl = rs * RW + myrow;
            if (o.WC == 1) {
                float other = 0.f;
                if (RW >= 2) other = __shfl_xor_sync(0xffffffffu, r, RW == 2 ? 16 : 8);
                const bool writer = (lane & 7) == 0 && (RW == 4 || (lane & 8) == 0) && (RW > 1 || lane == 0);
                if (writer && r0 + rl < rend && !aborted) {
                    if (o.epi == EPI_STORE) o.y[r0 + rl] = r;
                    else if (o.epi == EPI_RESIDUAL) o.y[r0 + rl] = __ldcg(o.res + r0 + rl) + r;
                    else if ((myrow & 1) == 0) o.y[(r0 + rl) >> 1] = r / (1.0f + expf(-r)) * other;
                }
            } else {
                float *pt = part + ((size_t)slot * o.R) * o.WC;
                if ((lane & 7) == 0 && (RW == 4 || (lane & 8) == 0)) pt[rl * o.WC + cgw] = r;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]); // partials written, stage may be refilled
    }
    if (o.WC > 1) {
        asm volatile("bar.sync 1, %0;" ::"r"(nthr_c) : "memory"); // all partials of the last tiles are in
        for (uint32_t kt = ntiles > o.S ? ntiles - o.S : 0; kt < ntiles; ++kt) flush(kt, kt % (2 * o.S));
    }
}

// Sharded launch, after an op: this CTA's rows [rbeg, rend) of the op, just written to this rank's result vector,
// go to every other rank (the CTA barrier before the call made them visible to all its threads; they are read back
// past the L1 and sent as plain stores through the peer mappings, a warp's worth contiguous): as {value, step}
// pairs into the receivers' pair areas, or as plain floats into the same place of their vectors.
// Kept out of line, like chain_shard_finish: the sharded tail must not weigh on the registers of the row loop.
__device__ __noinline__ void chain_shard_send(const ChainOpDev &o, const ShardDev &sh, uint32_t rbeg, uint32_t rend, uint32_t tid,
                                              uint32_t nthr_c) {
    if (sh.tagged) {
        const unsigned step = shard_this_step(sh);
        uint2 *mine = sh.pairs + (size_t)(step & 1u) * sh.pair_floats + (o.y - sh.ybase);
        for (uint32_t e = rbeg + tid; e < rend; e += nthr_c) {
            const float v = __ldcg(o.y + e);
            for (int r = 0; r < sh.world; ++r)
                if (r != sh.rank) shard_st_pair((uint2 *)((char *)(mine + e) + sh.delta[r]), v, step);
        }
    } else {
        for (uint32_t e = rbeg + tid; e < rend; e += nthr_c) {
            const float v = __ldcg(o.y + e);
            for (int r = 0; r < sh.world; ++r)
                if (r != sh.rank) *(float *)((char *)(o.y + e) + sh.delta[r]) = v;
        }
    }
}

// Sharded launch, after the last op (all consumer threads).
__device__ __noinline__ void chain_shard_finish(const ChainParams &p, uint8_t *smem, uint32_t tid, uint32_t nthr_c, bool aborted) {
    if (p.sh.tagged) {
        // Tagged exchange: the rows the other ranks owe this one arrive as pairs; all CTAs share the polling (a
        // few elements per thread), whichever op they worked on, and write the values into this rank's vector.
        const unsigned step = shard_this_step(p.sh);
        int &failed = *(int *)(smem + 132);
        if (tid == 0) failed = aborted ? 1 : 0;
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
        if (!aborted && p.sh.world > 1) {
            const unsigned long long t0 = shard_now_ns();
            bool ok = true;
            for (int i = 0; i < p.n_ops && ok; ++i) {
                const ChainOpDev &o = p.op[i];
                const uint32_t own = (uint32_t)(o.y - p.sh.ybase) - o.gather_off, remote = o.gather_len - o.out_dim;
                for (uint32_t j = blockIdx.x * nthr_c + tid; j < remote && ok; j += gridDim.x * nthr_c)
                    ok = shard_take_pair(p.sh, step, (size_t)o.gather_off + (j < own ? j : j + o.out_dim), t0);
            }
            if (!ok) {
                failed = 1;
                *(volatile int *)p.status = DEV_TIMEOUT;
            }
        }
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
        if (tid == 0) shard_cta_done_tagged(p.sh, step, failed != 0);
    } else {
        // Plain stores: once every consumer thread has issued its stores to the peers, one thread orders them and
        // counts the CTA in; the last CTA publishes the exchange to every rank and waits, bounded, for theirs.
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory");
        if (tid == 0 && !shard_cta_done(p.sh, aborted)) *(volatile int *)p.status = DEV_TIMEOUT;
    }
}

constexpr int CHAIN_MAX_THREADS = 21 * 32; // 20 consumer warps + the producer warp

// 20 consumer warps at 80 registers.  Measured against it on the 70B block (B200, us per step): 28 warps at 64
// registers, which would keep every warp busy on rows of 14 column groups (28,672 columns; 14 of 20 warps work
// there), 135-156 instead of 107: a row slice then has to drop to one or two rows per warp, and that costs more
// than the idle warps; tiles capped at 56 KB (two rows per warp, four stages) 139.
__global__ void __launch_bounds__(CHAIN_MAX_THREADS, 1) matvec_chain_kernel(const __grid_constant__ ChainParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem, *empty = full + CHAIN_MAX_STAGES;
    int &sync_ok = *(int *)(smem + 128); // after the 2 x 8 mbarriers; static shared memory would eat into the opt-in maximum
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == p.NW;
    pdl_launch_dependents();
    if (tid == 0) {
        for (uint32_t s = 0; s < CHAIN_MAX_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.NW);
        }
        mbar_init((uint64_t *)(smem + 136), p.NW); // "activation image is in registers" (see ChainOpDev::late_stage)
        sync_ok = 1;
        mbar_fence_init();
    }
    __syncthreads();

    if (producer) {
        // the weight tiles of every op, back to back: one tile = one contiguous byte range
        uint32_t kg = 0, s = 0, ph = 0; // tile count, ring stage and phase of the stage's current use, carried along
        for (int i = 0; i < p.n_ops; ++i) {
            const ChainOpDev &o = p.op[i];
            uint8_t *ring = smem + o.off_ring;
            uint32_t rbeg, rend;
            chain_row_range(o, rbeg, rend);
            const uint32_t ntiles = (rend - rbeg + o.R - 1) / o.R;
            // this CTA's rows of the op are one contiguous byte range; the L2 prefetch runs pf_tiles tiles ahead of the ring
            const uint8_t *range0 = o.w + (size_t)rbeg * o.row_bytes;
            const size_t range_bytes = (size_t)(rend - rbeg) * o.row_bytes, tile_bytes = (size_t)o.R * o.row_bytes;
            auto prefetch_tile = [&](uint32_t kt) {
                const size_t b0 = (size_t)kt * tile_bytes;
                if (b0 >= range_bytes) return;
                const uint32_t nb = (uint32_t)min(tile_bytes, range_bytes - b0);
                for (uint32_t off = lane * p.chunk; off < nb; off += 32 * p.chunk) bulk_prefetch_l2(range0 + b0 + off, min(p.chunk, nb - off));
            };
            for (uint32_t kt = o.S; kt < o.S + p.pf_tiles && p.pf_tiles; ++kt) prefetch_tile(kt); // tiles 0 .. S-1 are requested by the ring at once
            for (uint32_t k = 0; k < ntiles; ++k, ++kg, s = s + 1 == o.S ? 0 : s + 1, ph ^= (s == 0)) {
                if (p.pf_tiles) prefetch_tile(k + o.S + p.pf_tiles);
                bool ok = true;
                if (lane == 0 && kg >= o.S) ok = wait_or_timeout(&empty[s], ph ^ 1u);
                else if (lane == 0 && s >= o.late_stage) ok = wait_or_timeout((uint64_t *)(smem + 136), 0);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
                    return;
                }
                const uint32_t r0 = rbeg + k * o.R, rows = min(o.R, rend - r0), wb = rows * o.row_bytes;
                uint8_t *dst = ring + (size_t)s * o.stage_bytes;
                if (lane == 0) mbar_arrive_expect_tx(&full[s], wb);
                __syncwarp();
                const uint8_t *src = o.w + (size_t)r0 * o.row_bytes;
                for (uint32_t off = lane * p.chunk; off < wb; off += 32 * p.chunk)
                    bulk_g2s(dst + off, src + off, min(p.chunk, wb - off), &full[s]);
            }
        }
        return;
    }

    // ---- consumer warps ----
    pdl_wait_prior(); // activations may come from the previous kernel in the stream
    const uint32_t nthr_c = p.NW * 32;
    bool aborted = false;
    uint32_t kbase = 0;
    for (int i = 0; i < p.n_ops; ++i) {
        const ChainOpDev &o = p.op[i];
        if (o.dep && !chain_grid_sync(p.sync, nthr_c, tid, &sync_ok)) aborted = true;
        uint32_t rbeg, rend;
        chain_row_range(o, rbeg, rend);
        if (rbeg == rend) continue; // no rows of this op here (another group of CTAs has them): no image of its x either
#define ULLM_CHAIN_CASE(F, RWv, Gv) \
    if (o.fmt == F && o.rw == RWv && o.g == Gv) chain_consume<F, RWv, Gv>(o, p, smem, kbase, tid, aborted);
        ULLM_CHAIN_CASE(FMT_Q4K, 1, 1) ULLM_CHAIN_CASE(FMT_Q4K, 2, 1) ULLM_CHAIN_CASE(FMT_Q4K, 4, 1)
        ULLM_CHAIN_CASE(FMT_Q6KR, 1, 1) ULLM_CHAIN_CASE(FMT_Q6KR, 2, 1) ULLM_CHAIN_CASE(FMT_Q6KR, 4, 1)
#undef ULLM_CHAIN_CASE
        kbase += (rend - rbeg + o.R - 1) / o.R;
        asm volatile("bar.sync 2, %0;" ::"r"(nthr_c) : "memory"); // prep / part areas are free for the next op
        if (p.sh.world > 1 && !aborted) chain_shard_send(o, p.sh, rbeg, rend, tid, nthr_c);
    }
    if (aborted && lane == 0) *(volatile int *)p.status = DEV_TIMEOUT;
    if (p.sh.world) chain_shard_finish(p, smem, tid, nthr_c, aborted);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static inline uint32_t align_up_u32(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
static inline uint32_t gcd_u(uint32_t a, uint32_t b) {
    while (b) {
        const uint32_t t = a % b;
        a = b, b = t;
    }
    return a;
}

bool matvec_chain_supported(int fmt, size_t out_dim, size_t in_dim, int epi) {
    if (fmt != FMT_Q4K && fmt != FMT_Q6KR) return false;
    if (in_dim % QK_K || in_dim == 0 || out_dim == 0 || out_dim > 0x7fffffffull) return false;
    if (fmt == FMT_Q6KR && in_dim % 2048) return false;
    if (epi == EPI_SWIGLU && (out_dim & 1)) return false;
    return (in_dim + 2047) / 2048 <= 16; // one column group (2048 columns) per warp; up to 16 of the 20 consumer warps form a row slice
}

// How `grid` CTAs are dealt out to `n` independent ops (n <= grid): ncta[i] CTAs share op i's rows.
// Model of an op's time with m CTAs: fixed_i + work_i / m, where work_i is its weight bytes at the rate a CTA
// streams them (prepared Q6_K rows weigh g_q6k_cost, fitted on the 70B block: 111.7 / 107.0 / 108.7 us per step at
// 1.3 / 1.4 / 1.5 before, 100.9 / 98.6 / 95.7 / 98.0 / 100.5 at 1.2 / 1.1 / 1.05 / 1.0 / 0.95 after four rows per
// warp came to its widest matrix) and fixed_i is what every CTA of the op spends before its first tile: reading
// and converting the op's whole input vector.  The launch ends when the slowest group does, so the CTAs are dealt
// out to minimise the largest group time: one CTA each, then every further CTA to the group that is slowest at
// that moment (optimal for this model; rounding byte shares to the nearest count instead left the 1024-row
// matrices of the 70B block with one CTA each, and those two CTAs then set the time of the whole step).
void matvec_chain_deal(int n, const MatvecChainOp *ops, uint32_t grid, uint32_t *ncta) {
    double work[CHAIN_MAX_OPS], fixed[CHAIN_MAX_OPS];
    for (int i = 0; i < n; ++i) {
        const double rb = (double)(ops[i].in_dim / QK_K) * (ops[i].fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
        work[i] = (double)ops[i].out_dim * rb * (ops[i].fmt == FMT_Q4K ? 1.0 : g_q6k_cost) / 33000.0; // us of one CTA
        fixed[i] = 0.5 + (double)ops[i].in_dim * 7.0e-5;                                             // us
        ncta[i] = 1;
    }
    for (uint32_t used = (uint32_t)n; used < grid; ++used) {
        int slow = 0;
        double worst = -1.0;
        for (int i = 0; i < n; ++i) {
            const uint32_t units = std::max<uint32_t>(1, (uint32_t)(ops[i].out_dim / 2)); // no more CTAs than pairs of rows
            const double t = ncta[i] >= units ? -1.0 : fixed[i] + work[i] / ncta[i];
            if (t > worst) worst = t, slow = i;
        }
        ++ncta[slow];
    }
}

cudaError_t launch_matvec_chain(const DeviceInfo &dev, int n, const MatvecChainOp *ops, unsigned *d_sync, int *d_status,
                                cudaStream_t st, bool pdl, const ShardDev *shard) {
    if (n <= 0 || n > CHAIN_MAX_OPS) return cudaErrorInvalidValue;
    ChainParams p{};
    if (shard) {
        if (shard->world < 1 || shard->world > SHARD_MAX_RANKS) return cudaErrorInvalidValue;
        for (int i = 0; i < n; ++i)
            if (ops[i].epi != EPI_STORE) return cudaErrorNotSupported; // fused epilogues stay on one GPU
        p.sh = *shard;
    }
    p.n_ops = n, p.sync = d_sync, p.status = d_status, p.NW = 20, p.chunk = (uint32_t)g_chain_chunk, p.pf_tiles = (uint32_t)g_pf_tiles;
    const int budget = dev.max_smem_optin - 1024;
    const uint32_t grid = (uint32_t)dev.sm_count;
    // Independent ops: the CTAs are dealt out to the ops (at least one CTA each, never more CTAs than the op has
    // pairs of rows), so that every group of CTAs is expected to finish at the same time.
    uint32_t cta0[CHAIN_MAX_OPS], ncta[CHAIN_MAX_OPS];
    bool dealt = n > 1 && (uint32_t)n <= grid;
    for (int i = 0; i < n; ++i) dealt = dealt && !ops[i].dep;
    if (dealt) {
        matvec_chain_deal(n, ops, grid, ncta);
        uint32_t at = 0;
        for (int i = 0; i < n; ++i) cta0[i] = at, at += ncta[i];
    } else {
        for (int i = 0; i < n; ++i) cta0[i] = 0, ncta[i] = grid;
    }
    for (int i = 0; i < n; ++i) {
        const MatvecChainOp &h = ops[i];
        if (!matvec_chain_supported(h.fmt, h.out_dim, h.in_dim, h.epi)) return cudaErrorNotSupported;
        if (((uintptr_t)h.w | (uintptr_t)h.x) & 15 || (h.norm_w && ((uintptr_t)h.norm_w & 15))) return cudaErrorNotSupported;
        ChainOpDev &o = p.op[i];
        o.w = (const uint8_t *)h.w, o.x = h.x, o.y = h.y, o.norm_w = h.norm_w, o.res = h.res, o.eps = h.eps, o.epi = h.epi;
        o.fmt = h.fmt, o.dep = h.dep ? 1 : 0, o.out_dim = (uint32_t)h.out_dim, o.in_dim = (uint32_t)h.in_dim;
        o.gather_off = (uint32_t)h.gather_off, o.gather_len = (uint32_t)h.gather_len;
        if (shard && shard->tagged && (h.gather_len < h.out_dim || h.gather_off + h.gather_len > 0xffffffffull)) return cudaErrorInvalidValue;
        o.row_bytes = (uint32_t)(h.in_dim / QK_K) * (h.fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
        o.gran = 16 / gcd_u(o.row_bytes, 16);
        if (h.epi == EPI_SWIGLU) o.gran = std::max(o.gran, 2u);
        if (o.out_dim % o.gran) return cudaErrorNotSupported;
        o.ncg = (uint32_t)((h.in_dim + 2047) / 2048);
        o.g = (o.ncg + 15) / 16;
        o.WC = (o.ncg + o.g - 1) / o.g;
        o.WR = p.NW / o.WC;
        o.cta0 = cta0[i], o.ncta = std::min<uint32_t>(ncta[i], std::max<uint32_t>(1, o.out_dim / o.gran));
    }
    // Rows per warp of op i: the largest of 4, 2, 1 whose tile stays within `tile_cap`, unless a tile of half the
    // rows already covers a CTA's whole share of the op (then the rest would be padding).
    auto pick_rows = [&](ChainOpDev &o, uint32_t tile_cap) -> bool {
        const uint32_t rows_cta = (o.out_dim / o.gran + o.ncta - 1) / o.ncta * o.gran;
        const uint32_t rw_min = o.epi == EPI_SWIGLU ? 2u : 1u;
        o.rw = 0;
        for (uint32_t rw = 4; rw >= rw_min; rw /= 2) {
            const uint32_t R = o.WR * rw;
            if (R % o.gran || (uint64_t)R * o.row_bytes > tile_cap) continue;
            if (rw > rw_min && o.WR * (rw / 2) >= rows_cta && (o.WR * (rw / 2)) % o.gran == 0) continue;
            o.rw = rw;
            break;
        }
        o.R = o.WR * o.rw;
        return o.rw != 0;
    };
    auto part_bytes = [](const ChainOpDev &o) { return std::max(128u, 2u * 8u * o.R * o.WC * 4u); };
    auto prep_bytes = [](const ChainOpDev &o) { return o.ncg * (uint32_t)(o.fmt == FMT_Q4K ? XREGS_Q4K : XREGS_Q6KR) * 32u * 4u; };
    // Tiles of up to 100 KB (four rows per warp on wide matrices) when the ring of at least two of them still fits
    // beside the partial sums and the activation image; else tiles of up to 56 KB.
    uint32_t smem = 0;
    if (dealt) { // a CTA meets one op: every op has the layout that suits it
        for (int i = 0; i < n; ++i) {
            ChainOpDev &o = p.op[i];
            bool fits = false;
            // 1: large tiles beside the image; 2: large tiles, the last stages laid over the image (the consumers hold
            // it in registers by the time the ring needs them: the 66 KB image of a 28,672-column vector otherwise
            // forces tiles of two rows); 3: small tiles beside the image
            for (int form = 1; form <= 3 && !fits; ++form) {
                if (form == 2 && !g_overlap_image) continue;
                if (!pick_rows(o, form == 3 ? 56u * 1024u : 100u * 1024u)) continue;
                o.stage_bytes = align_up_u32(o.R * o.row_bytes, 128);
                o.off_part = 256;
                const uint32_t after_part = align_up_u32(o.off_part + part_bytes(o), 128), pb = align_up_u32(prep_bytes(o), 128);
                if (form != 2) {
                    o.off_prep = after_part;
                    o.off_ring = o.off_prep + pb;
                    if ((int)o.off_ring + 2 * (int)o.stage_bytes > budget) continue;
                    o.S = std::min<uint32_t>(CHAIN_MAX_STAGES, (uint32_t)(budget - (int)o.off_ring) / o.stage_bytes);
                    o.late_stage = o.S;
                } else {
                    o.off_ring = after_part;
                    if ((int)o.off_ring + 2 * (int)o.stage_bytes > budget || pb > o.stage_bytes) continue;
                    o.S = std::min<uint32_t>(CHAIN_MAX_STAGES, (uint32_t)(budget - (int)o.off_ring) / o.stage_bytes);
                    o.off_prep = o.off_ring + o.S * o.stage_bytes - pb; // inside the last stage
                    o.late_stage = o.S - 1;
                }
                fits = true;
            }
            if (!fits) return cudaErrorNotSupported;
            smem = std::max(smem, o.off_ring + o.S * o.stage_bytes);
        }
    } else { // all CTAs walk the list: one layout, sized for the largest op, so that the ring runs on across ops
        bool fits = false;
        uint32_t max_stage = 0, max_part = 128, max_prep = 0;
        for (uint32_t tile_cap : {100u * 1024u, 56u * 1024u}) {
            max_stage = 0, max_part = 128, max_prep = 0;
            bool ok = true;
            for (int i = 0; i < n && ok; ++i) {
                ChainOpDev &o = p.op[i];
                ok = pick_rows(o, tile_cap);
                max_stage = std::max(max_stage, align_up_u32(o.R * o.row_bytes, 128));
                max_part = std::max(max_part, part_bytes(o));
                max_prep = std::max(max_prep, prep_bytes(o));
            }
            if (ok && 256 + (int)align_up_u32(max_part, 128) + (int)align_up_u32(max_prep, 128) + 2 * (int)max_stage <= budget) {
                fits = true;
                break;
            }
        }
        if (!fits) return cudaErrorNotSupported;
        const uint32_t off_part = 256, off_prep = align_up_u32(off_part + max_part, 128), off_ring = align_up_u32(off_prep + max_prep, 128);
        const uint32_t S = std::min<uint32_t>(CHAIN_MAX_STAGES, (uint32_t)(budget - (int)off_ring) / max_stage);
        for (int i = 0; i < n; ++i) {
            ChainOpDev &o = p.op[i];
            o.S = S, o.stage_bytes = max_stage, o.off_part = off_part, o.off_prep = off_prep, o.off_ring = off_ring, o.late_stage = S;
        }
        smem = off_ring + S * max_stage;
    }
    static bool attr_set[64] = {};
    int devid = 0;
    cudaGetDevice(&devid);
    if (devid < 64 && !attr_set[devid]) {
        cudaError_t e = cudaFuncSetAttribute(matvec_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[devid] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3((p.NW + 1) * 32), cfg.dynamicSmemBytes = smem, cfg.stream = st;
    // A list with a dependent op meets at the grid-wide barrier, which needs every CTA resident at once: such a
    // list is a cooperative launch (the driver refuses it when the grid does not fit beside what else is running,
    // and the caller then runs the ops one by one).  Independent ops never wait for another CTA and may instead
    // be launched programmatically dependent on the previous kernel.
    bool any_dep = false;
    for (int i = 0; i < n; ++i) any_dep = any_dep || ops[i].dep;
    cudaLaunchAttribute at[1];
    if (any_dep) {
        at[0].id = cudaLaunchAttributeCooperative;
        at[0].val.cooperative = 1;
    } else {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
    }
    cfg.attrs = at, cfg.numAttrs = (any_dep || pdl) ? 1 : 0;
    if (any_dep) {
        const cudaError_t e = cudaLaunchKernelEx(&cfg, matvec_chain_kernel, p);
        if (e == cudaErrorCooperativeLaunchTooLarge) {
            cudaGetLastError();
            return cudaErrorNotSupported;
        }
        return e;
    }
    return cudaLaunchKernelEx(&cfg, matvec_chain_kernel, p);
}

} // namespace ullm
