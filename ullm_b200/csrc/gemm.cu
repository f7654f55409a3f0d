// Prefill GEMM on quantized weights:  Y[s, o] = sum_i W[o, i] * X[s, i]  for many
// tokens at once (CPU form: matmul_q, crates/ullm-model/src/math.rs:38-63; Metal form:
// matmul_q4k / matmul_q6k, crates/ullm-metal/src/shader.metal:620-740).
//
// A dense contraction, so it runs on the 5th-generation tensor cores.  A pair of CTAs
// (cta_group::2) owns a [256 weight rows x 256 tokens] tile; each CTA keeps its 128 rows of
// the fp32 accumulator in its tensor memory (TMEM).  The packed weight bytes arrive in shared
// memory by tiled TMA, dequantization threads turn them into bf16 (values rounded once, from
// the exact f32 dequantization) and write them with tcgen05.st straight into tensor memory,
// where tcgen05.mma reads its A operand — the weights never pass through shared memory in
// bf16 form, which keeps its bandwidth for the B operand: the bf16 activation tile, loaded
// by tiled TMA with the 128-byte swizzle, half of the tokens into each CTA.  One elected
// thread of the pair issues the MMAs (kind::f16, M=256, N=256, K=16) and commits them onto
// the mbarriers that recycle the operand stages in both CTAs.  The epilogue reads the
// accumulator back with tcgen05.ld and stores token-major f32.
//
// Roles in a CTA of 20 warps (a pair of CTAs on neighbouring SMs works on one tile):
//   warp 0      TMA: this CTA's half of the activation tile of every k-chunk, 8 stages
//   warp 1      tensor-memory allocation
//   warps 2-17  dequantization from the staged bytes into tensor memory (thread = one row = one TMEM
//               lane; a warp reaches only lanes 32 * (warp % 4) .., so each row quarter has four warps:
//               two column parts x two phases, a phase taking every other 64-k chunk), then the epilogue
//   warp 18     TMA: the packed weight bytes of [128 rows x 256 k] per block, 3-4 stages
//   warp 19     MMA issue and commits (leader CTA of the pair only)
// Every mbarrier wait is bounded; on expiry the CTA records a status, stops issuing
// work, still frees its tensor memory and leaves.
//
// Why two phases: a dequantization warp's chain wait -> unpack -> tcgen05.st -> wait::st -> arrive is long
// against the chunk period; with two phases every warp has two chunk periods for it.  The service warps
// (TMA, allocation, MMA issue) sit on four different warp schedulers.
#include "kernels.h"
#include "matvec_core.cuh"
#include "shard_dev.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

namespace ullm {

constexpr int GM = 128;   // weight rows per CTA; a CTA pair covers 256 (MMA M)
constexpr int GN = 256;   // tokens per CTA pair (MMA N, TMEM columns); each CTA stages 128 of them
constexpr int GNH = GN / 2;
constexpr int GKC = 64;   // k per chunk: 64 bf16 = one 128-byte swizzle row
constexpr int G_STAGES = 8;  // operand stages in flight: one dequantized weight chunk (tensor memory) + one activation chunk (shared memory) each
constexpr int G_A_COLS = GKC / 2;         // a weight chunk in tensor memory: 64 bf16 per row = 32 columns of 32 bit
constexpr int G_TMEM_COLS = 512;          // accumulator (256) + 8 weight chunks (8 x 32)
constexpr int G_B_BYTES = GNH * GKC * 2;  // 16 KB
// Warps: 0 activation TMA, 1 tensor-memory allocation, 2 .. 1 + 8 * PHASES dequantization, then weight-byte TMA, then MMA issue.
// A warp reaches only the tensor-memory lanes 32 * (warp % 4) .., so every row quarter has four dequantization
// warps: two column parts x PHASES phases.  A phase takes every PHASES-th 64-k chunk, which gives a warp that many chunk
// periods for its wait -> unpack -> tcgen05.st -> arrive chain instead of one (the format's register need caps it).
constexpr int g_deq_warps(int phases) { return 8 * phases; }
constexpr int g_raw_warp(int phases) { return 2 + 8 * phases; }
constexpr int g_mma_warp(int phases) { return 3 + 8 * phases; }
constexpr int g_threads(int phases) { return (4 + 8 * phases) * 32; }

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)0 << 16;                        // leading byte offset (unused: K extent inside the swizzle row)
    d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset
    d |= (uint64_t)1 << 46;                        // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// instruction descriptor: D f32, A/B bf16, both K-major, M = 256 (two CTAs x 128), N = 256
__host__ __device__ constexpr uint32_t umma_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GN >> 3) << 17) | ((uint32_t)((2 * GM) >> 4) << 24);
}

// shared::cluster address of `local` (an address in this CTA's shared window) inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier of any CTA of the cluster (address from mapa_u32)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled TMA load into this CTA's own shared memory, completion counted on an mbarrier
// given by its shared::cluster address (this CTA's or the pair leader's).
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
                 : "memory");
}
// One MMA over the CTA pair: D[256 x 256] (+)= A[256 x 16] * B[256 x 16]^T.  Each CTA supplies its
// 128 rows of A from its own tensor memory (lane = row, one 32-bit column = two consecutive k),
// its 128 of B's tokens from shared memory (same offsets in both CTAs), and holds its 128 rows
// of D in its own tensor memory.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// the same with D always accumulated (no predicate to set up)
__device__ __forceinline__ void umma_bf16_acc(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n.reg .pred p;\nsetp.eq.b32 p, 0, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d), "r"(tmem_a),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
}
// Arrives (once the MMAs issued so far are complete) on the mbarrier at the same offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Eight consecutive 32-bit columns of this thread's tensor-memory lane (the warp's lane quarter is in taddr)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

struct GemmParams {
    float *y;  // [s, out]
    int *status;
    uint32_t out_dim, in_dim, s;
    uint32_t blocks_per_split; // 256-k blocks handled by one grid.z slice (split-K for matrices with few row tiles)
    int epi;                   // EPI_STORE / EPI_RESIDUAL / EPI_SWIGLU, applied here only when there is one k slice
    const float *res;          // EPI_RESIDUAL: y = res + W x (may alias y)
    uint32_t ldy;              // elements between two tokens in y / res (the full matrix' rows when this launch covers a row range)
    uint32_t tbl_bytes;        // MLX 4-bit: bytes per table entry (4 = f32, 2 = bf16 bits); group size is 64
    int sh_world;              // > 0: every output element goes to the same place in all ranks' gather buffers (EPI_STORE)
    long long sh_delta[SHARD_MAX_RANKS];
#ifdef ULLM_TUNING
    long long *trace; // measurement only: cycle stamps of CTA (0, 0)
    uint32_t mode; // measurement only: bit 0 skips the dequantization, bit 1 the activation loads, bit 2 the MMAs
#endif
};
// x: bf16 activations [s, in], 128-byte swizzle.  w0..w2: the packed weight bytes as plain
// 2-D byte tensors [out rows, row bytes] — Q4_K: w0 = whole 144-byte blocks; prepared
// Q6_K: w0 = 48-byte records, w1 = the 16 scale bytes of a block, w2 = eight blocks' f16 d;
// MLX 4-bit (group 64): w0 = the 128 bytes of packed words of a 256-k block, w1 / w2 = 16 bytes of the row's
// scale / bias table around the block's four entries.
struct GemmMaps {
    CUtensorMap x, w0, w1, w2;
};

#ifndef PHASES_Q4K
#define PHASES_Q4K 2
#endif
template <int FMT> struct GemmCfg;
template <> struct GemmCfg<FMT_Q4K> {
    static constexpr int RAW_BYTES = GM * Q4K_BYTES; // [128 rows][144 B]: 16-byte reads one row apart hit distinct banks
    static constexpr int PHASES = PHASES_Q4K;
    static constexpr int RAW_STAGES = 4;
};
template <> struct GemmCfg<FMT_MLX4> {
    static constexpr int RAW_BYTES = GM * 128 + 2 * GM * 16; // [128 rows][128 B of words], [128][16 B] scales, [128][16 B] biases
    static constexpr int PHASES = 2;
    static constexpr int RAW_STAGES = 4;
};
template <> struct GemmCfg<FMT_Q6KR> {
    static constexpr int REC_BYTES = GM * 48;                  // one record of every row: [128][48 B], conflict-free as well
    static constexpr int RAW_BYTES = 4 * REC_BYTES + 2 * GM * 16; // 4 records, [128][16 B] scales, [128][16 B] d
    static constexpr int PHASES = 2;
    static constexpr int RAW_STAGES = 3;
};

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// Integer -> float without the conversion unit: a 16-bit lane holding 0x6400 | v is the
// half-precision number 1024 + v exactly (v < 1024), so one logic op places two packed
// integers into a half2 and one half2 subtract (exact) turns them into the values; the
// half -> float widening is exact as well.
__device__ __forceinline__ __half2 h2_bits(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ __half2 h2_const(float v) { return __float2half2_rn(v); }

// ---- what one dequantization thread keeps of a 256-k block of its row -----------------
// Q4_K: thread (row, q) owns qs bytes [16q, 16q+16) of each of the four 64-k chunks.
struct BlkQ4K {
    uint4 hdr;   // d, dmin, 12 packed scale bytes
    uint4 qs[4];
};
__device__ __forceinline__ void blk_load(BlkQ4K &b, uint32_t raw, uint32_t row, uint32_t q, uint32_t) {
    const uint32_t a = raw + row * Q4K_BYTES;
    b.hdr = lds128(a);
#pragma unroll
    for (int c = 0; c < 4; ++c) b.qs[c] = lds128(a + 16 + 32 * c + 16 * q);
}
// Writes the thread's 32 values of chunk c (low nibbles -> k 16q.., high -> k 32+16q..):
// d*sc and dmin*m as crates/ullm-core/src/dequant.rs:203-210 forms them, then
// (d*sc)*q - dmin*m — the product is exact in f32 (q < 16), so the fused multiply-subtract
// rounds exactly where the reference's subtraction does — and one more rounding to bf16.
__device__ __forceinline__ void chunk_store(const BlkQ4K &b, int c, uint32_t q, uint32_t ta) {
    const float d = f16_bits_to_f32((uint16_t)(b.hdr.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(b.hdr.x >> 16));
    const __half2 k1024 = h2_const(1024.f), k16th = h2_const(0.0625f), km64 = h2_const(-64.f);
    int sA, mA, sB, mB;
    q4k_pair(b.hdr.y, b.hdr.z, b.hdr.w, c, sA, mA, sB, mB);
    const float d1 = __fmul_rn(d, (float)sA), nm1 = -__fmul_rn(dmin, (float)mA);
    const float d2 = __fmul_rn(d, (float)sB), nm2 = -__fmul_rn(dmin, (float)mB);
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = word_of(b.qs[c], i), w8 = w >> 8;
        // bytes (0, 2) and (1, 3) of the word: low nibbles, then high nibbles (held as 16 * q)
        const __half2 l02 = __hsub2(h2_bits((w & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 l13 = __hsub2(h2_bits((w8 & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 h02 = __hfma2(h2_bits((w & 0x00f000f0u) | 0x64006400u), k16th, km64);
        const __half2 h13 = __hfma2(h2_bits((w8 & 0x00f000f0u) | 0x64006400u), k16th, km64);
        lo[2 * i] = pack_bf16x2(__fmaf_rn(d1, __low2float(l02), nm1), __fmaf_rn(d1, __low2float(l13), nm1));
        lo[2 * i + 1] = pack_bf16x2(__fmaf_rn(d1, __high2float(l02), nm1), __fmaf_rn(d1, __high2float(l13), nm1));
        hi[2 * i] = pack_bf16x2(__fmaf_rn(d2, __low2float(h02), nm2), __fmaf_rn(d2, __low2float(h13), nm2));
        hi[2 * i + 1] = pack_bf16x2(__fmaf_rn(d2, __high2float(h02), nm2), __fmaf_rn(d2, __high2float(h13), nm2));
    }
    tmem_st8(ta + 8 * q, lo);       // k 16q .. 16q+15
    tmem_st8(ta + 16 + 8 * q, hi);  // k 32+16q .. 32+16q+15
}

// Prepared Q6_K (prepare.cu): thread (row, tp) owns records (h, tp), h = 0, 1: positions
// l = 16tp..16tp+15 of all four groups of half h.  Chunk c = 2h + gp holds groups 2gp, 2gp+1.
struct BlkQ6KR {
    uint4 rec[2][3]; // W1, W2, W3
    uint32_t sc[2];  // the record's four int8 scales
    uint32_t d;      // f16 bits
};
__device__ __forceinline__ void blk_load(BlkQ6KR &b, uint32_t raw, uint32_t row, uint32_t tp, uint32_t kb) {
    constexpr uint32_t REC = GemmCfg<FMT_Q6KR>::REC_BYTES;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t a = raw + (2 * h + tp) * REC + row * 48;
#pragma unroll
        for (int k = 0; k < 3; ++k) b.rec[h][k] = lds128(a + 16 * k);
        b.sc[h] = lds32(raw + 4 * REC + row * 16 + (2 * h + tp) * 4);
    }
    b.d = lds_u16(raw + 4 * REC + GM * 16 + row * 16 + (kb & 7u) * 2);
}
// value = (d * sc) * (q - 32), left to right as dequant.rs:275-278, then rounded to bf16
__device__ __forceinline__ void chunk_store(const BlkQ6KR &b, int c, uint32_t tp, uint32_t ta) {
    const int h = c >> 1, gp = c & 1;
    const float d = f16_bits_to_f32((uint16_t)b.d);
    const __half2 k1056 = h2_const(1056.f); // 1024 + the format's offset of 32
    const uint32_t scw = b.sc[h];
    const float dsA = __fmul_rn(d, (float)((int)(scw << (24 - 16 * gp)) >> 24));
    const float dsB = __fmul_rn(d, (float)((int)(scw << (16 - 16 * gp)) >> 24));
    uint32_t oA[8], oB[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w1 = word_of(b.rec[h][0], i), w2 = word_of(b.rec[h][1], i), w3 = word_of(b.rec[h][2], i);
        // four 6-bit values per word, one per byte, for the chunk's two groups
        const uint32_t qa = gp ? (((w2 >> 4) & 0x0f0f0f0fu) | ((w3 >> 2) & 0x30303030u)) : (w1 & 0x3f3f3f3fu);
        const uint32_t qb = gp ? (w3 & 0x3f3f3f3fu) : ((w2 & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u));
        const __half2 a02 = __hsub2(h2_bits((qa & 0x00ff00ffu) | 0x64006400u), k1056);
        const __half2 a13 = __hsub2(h2_bits(((qa >> 8) & 0x00ff00ffu) | 0x64006400u), k1056);
        const __half2 b02 = __hsub2(h2_bits((qb & 0x00ff00ffu) | 0x64006400u), k1056);
        const __half2 b13 = __hsub2(h2_bits(((qb >> 8) & 0x00ff00ffu) | 0x64006400u), k1056);
        oA[2 * i] = pack_bf16x2(__fmul_rn(dsA, __low2float(a02)), __fmul_rn(dsA, __low2float(a13)));
        oA[2 * i + 1] = pack_bf16x2(__fmul_rn(dsA, __high2float(a02)), __fmul_rn(dsA, __high2float(a13)));
        oB[2 * i] = pack_bf16x2(__fmul_rn(dsB, __low2float(b02)), __fmul_rn(dsB, __low2float(b13)));
        oB[2 * i + 1] = pack_bf16x2(__fmul_rn(dsB, __high2float(b02)), __fmul_rn(dsB, __high2float(b13)));
    }
    tmem_st8(ta + 8 * tp, oA);       // first group of the chunk, positions 16tp .. 16tp+15
    tmem_st8(ta + 16 + 8 * tp, oB);  // second group
}

// MLX 4-bit, group 64 (crates/ullm-core/src/dequant.rs:297-317): a 64-k chunk is one group; thread (row, q) owns the
// chunk's words 4q .. 4q+3 = k 32q .. 32q+31, nibble n of word j being element 8j + n.
struct BlkMLX {
    uint4 qs[4];      // per chunk: the thread's four words
    float sc[4], bi[4]; // per chunk: the group's scale and bias
};
__device__ __forceinline__ void blk_load_mlx(BlkMLX &b, uint32_t raw, uint32_t row, uint32_t q, uint32_t kb, uint32_t tbl_bytes) {
#pragma unroll
    for (int c = 0; c < 4; ++c) b.qs[c] = lds128(raw + row * 128 + 32 * c + 16 * q);
    const uint32_t ts = raw + GM * 128 + row * 16, tb = ts + GM * 16;
    if (tbl_bytes == 4) {
        const uint4 s4 = lds128(ts), b4 = lds128(tb);
        b.sc[0] = __uint_as_float(s4.x), b.sc[1] = __uint_as_float(s4.y), b.sc[2] = __uint_as_float(s4.z), b.sc[3] = __uint_as_float(s4.w);
        b.bi[0] = __uint_as_float(b4.x), b.bi[1] = __uint_as_float(b4.y), b.bi[2] = __uint_as_float(b4.z), b.bi[3] = __uint_as_float(b4.w);
    } else { // bf16 bits: the 16 staged bytes hold two blocks' entries, this block's four at (kb & 1) * 8
        const uint32_t o = (kb & 1u) * 8u;
        const uint32_t s01 = lds32(ts + o), s23 = lds32(ts + o + 4), b01 = lds32(tb + o), b23 = lds32(tb + o + 4);
        b.sc[0] = __uint_as_float(s01 << 16), b.sc[1] = __uint_as_float(s01 & 0xffff0000u);
        b.sc[2] = __uint_as_float(s23 << 16), b.sc[3] = __uint_as_float(s23 & 0xffff0000u);
        b.bi[0] = __uint_as_float(b01 << 16), b.bi[1] = __uint_as_float(b01 & 0xffff0000u);
        b.bi[2] = __uint_as_float(b23 << 16), b.bi[3] = __uint_as_float(b23 & 0xffff0000u);
    }
}
__device__ __forceinline__ void blk_load(BlkMLX &, uint32_t, uint32_t, uint32_t, uint32_t) {} // (the MLX path loads with its table width)
// value = q * scale + bias (dequant.rs:311-314; the product is exact for bf16-derived scales, so the fused
// multiply-add rounds where the reference's addition does), then rounded to bf16
__device__ __forceinline__ void chunk_store(const BlkMLX &b, int c, uint32_t q, uint32_t ta) {
    const __half2 k1024 = h2_const(1024.f);
    const float s = b.sc[c], bias = b.bi[c];
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = word_of(b.qs[c], i);
        // nibbles (0, 4), (1, 5), (2, 6), (3, 7) of the word as exact halves
        const __half2 a0 = __hsub2(h2_bits((w & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 a1 = __hsub2(h2_bits(((w >> 4) & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 a2 = __hsub2(h2_bits(((w >> 8) & 0x000f000fu) | 0x64006400u), k1024);
        const __half2 a3 = __hsub2(h2_bits(((w >> 12) & 0x000f000fu) | 0x64006400u), k1024);
        o[4 * i + 0] = pack_bf16x2(__fmaf_rn(s, __low2float(a0), bias), __fmaf_rn(s, __low2float(a1), bias));   // elements 0, 1
        o[4 * i + 1] = pack_bf16x2(__fmaf_rn(s, __low2float(a2), bias), __fmaf_rn(s, __low2float(a3), bias));   // 2, 3
        o[4 * i + 2] = pack_bf16x2(__fmaf_rn(s, __high2float(a0), bias), __fmaf_rn(s, __high2float(a1), bias)); // 4, 5
        o[4 * i + 3] = pack_bf16x2(__fmaf_rn(s, __high2float(a2), bias), __fmaf_rn(s, __high2float(a3), bias)); // 6, 7
    }
    const uint32_t lo[8] = {o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]}, hi[8] = {o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]};
    tmem_st8(ta + 16 * q, lo);     // k 32q .. 32q+15
    tmem_st8(ta + 16 * q + 8, hi); // k 32q+16 .. 32q+31
}

// A waiting thread must stay off the warp scheduler: a thread parked in try_wait (or spinning on
// it) takes issue slots from the dequantization warps of its scheduler, which then finish last and
// make everyone wait longer.  So waits test the barrier once (test_wait never blocks) and sleep
// between tests.  Bounded: about a second.
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool wait_polite_or_timeout(uint64_t *bar, uint32_t parity) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            asm volatile("nanosleep.u32 64;" ::: "memory");
            if (mbar_test_wait(bar, parity)) return true;
        }
        if (clock64() - t0 > (1ll << 31)) return false;
    }
}
// A whole warp waits on an mbarrier with one polling lane: 256 threads spinning on
// try_wait crowd the shared-memory pipe the MMA-issuing thread's own waits go through.
// Every lane then observes the completed phase itself (one try_wait that succeeds at
// once), which orders its following accesses after the barrier.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, uint32_t lane) {
    int ok = 1;
    if (lane == 0) ok = wait_polite_or_timeout(bar, parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) (void)mbar_test_wait(bar, parity);
    return ok != 0;
}

template <int FMT> struct BlkOf;
template <> struct BlkOf<FMT_Q4K> { using type = BlkQ4K; };
template <> struct BlkOf<FMT_Q6KR> { using type = BlkQ6KR; };
template <> struct BlkOf<FMT_MLX4> { using type = BlkMLX; };

// grid (2 * ceil(out / 256), ceil(s / 256)) in clusters of 2 along x, 352 threads
template <int FMT, bool DBG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g_threads(GemmCfg<FMT>::PHASES), 1)
    gemm_q_tc_kernel(const GemmParams p, const __grid_constant__ GemmMaps maps) {
    using Cfg = GemmCfg<FMT>;
    using Blk = typename BlkOf<FMT>::type;
    constexpr int RS = Cfg::RAW_STAGES;
    constexpr uint32_t PH = Cfg::PHASES;
    extern __shared__ __align__(1024) uint8_t gsm[];
    // dynamic smem is only guaranteed 16-byte aligned: round up to the 1024 B the swizzle atoms need
    // (the same amount in both CTAs of the pair, so operand offsets agree)
    uint8_t *base = (uint8_t *)(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
    uint8_t *b_tiles = base;                                 // G_STAGES x 16 KB: this CTA's 128 tokens
    uint8_t *raw = b_tiles + G_STAGES * G_B_BYTES;           // RS x packed bytes of [128 rows x 256 k]
    // full (used in the leader only): 16 dequantization warps of the pair + the leader's expect_tx arrival;
    // freeb / acc_full: one multicast tcgen05.commit each
    __shared__ uint64_t full[G_STAGES], freeb[G_STAGES], raw_full[RS], raw_free[RS], acc_full;
    __shared__ uint32_t tmem_base_s;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t m0 = blockIdx.x * GM, n0 = blockIdx.y * GN;
    // this CTA's share of k: blocks [kb0, kb0 + nb); with split-K, slice z writes its partial sums to y + z * s * out
    const uint32_t kb0 = blockIdx.z * p.blocks_per_split;
    const uint32_t nb = min(p.blocks_per_split, p.in_dim / QK_K - kb0), nchunks = nb * 4;
    float *const yout = p.y + (size_t)blockIdx.z * p.s * p.out_dim;
#ifdef ULLM_TUNING
    const bool traced = DBG && p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    const uint32_t mode = DBG ? p.mode : 0u; // stages switched off for measurement
    long long *const trace = p.trace;
    const bool traced_any = DBG && p.trace;
#else
    constexpr bool traced_any = false;
    constexpr bool traced = false;
    constexpr uint32_t mode = 0u;
    long long *const trace = nullptr;
#endif

    if (tid == 0) {
        for (int i = 0; i < G_STAGES; ++i) {
            mbar_init(&full[i], 16 + 1); // per chunk one phase of both CTAs arrives: 2 x 8 warps, + the expect_tx arrival
            mbar_init(&freeb[i], 1);
        }
        for (int i = 0; i < RS; ++i) {
            mbar_init(&raw_full[i], 1);
            mbar_init(&raw_free[i], g_deq_warps(PH));
        }
        mbar_init(&acc_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) { // all of tensor memory in each CTA of the pair: accumulator columns 0-255, weight chunks 256-511
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)G_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all(); // the peer's barriers exist before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_s;

    if (warp == 0) {
        // ---- TMA producer: this CTA's half of the activation tile of every k-chunk ----
        if (lane == 0) {
            for (uint32_t g = 0; g < nchunks; ++g) {
                const uint32_t c = g % G_STAGES;
                if (g >= G_STAGES && !(mode & 16u) && !wait_polite_or_timeout(&freeb[c], ((g / G_STAGES) - 1) & 1)) {
                    *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                const uint32_t lead_full = mapa_u32(smem_u32(&full[c]), 0);
                if (mode & 2u) {
                    if (rank == 0) mbar_arrive(&full[c]);
                    continue;
                }
                if (rank == 0) mbar_arrive_expect_tx(&full[c], 2 * G_B_BYTES); // both halves land on the leader's barrier
                tma_load_2d(b_tiles + c * G_B_BYTES, &maps.x, (int)((kb0 * 4 + g) * GKC), (int)(n0 + rank * GNH), lead_full);
                if (traced && g < 500) trace[6000 + g] = clock64();
            }
        }
    } else if (warp == (uint32_t)g_raw_warp(PH)) {
        // ---- TMA producer: packed weight bytes of every 256-k block (rows past the matrix read as zero) ----
        if (lane == 0) {
            for (uint32_t kb = 0; kb < nb; ++kb) {
                const uint32_t st = kb % RS;
                if (kb >= RS && !wait_polite_or_timeout(&raw_free[st], ((kb / RS) - 1) & 1)) {
                    *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                uint8_t *dst = raw + st * Cfg::RAW_BYTES;
                const uint32_t bar = smem_u32(&raw_full[st]), kg = kb0 + kb;
                mbar_arrive_expect_tx(&raw_full[st], Cfg::RAW_BYTES);
                if constexpr (FMT == FMT_Q4K) {
                    tma_load_2d(dst, &maps.w0, (int)(kg * Q4K_BYTES), (int)m0, bar);
                } else if constexpr (FMT == FMT_MLX4) {
                    // four table entries per block: 16 bytes of f32, or the aligned 16 bytes around 8 bytes of bf16
                    const int tx = p.tbl_bytes == 4 ? (int)(kg * 16) : (int)((kg >> 1) * 16);
                    tma_load_2d(dst, &maps.w0, (int)(kg * 128), (int)m0, bar);
                    tma_load_2d(dst + GM * 128, &maps.w1, tx, (int)m0, bar);
                    tma_load_2d(dst + GM * 128 + GM * 16, &maps.w2, tx, (int)m0, bar);
                } else {
#pragma unroll
                    for (int r = 0; r < 4; ++r) tma_load_2d(dst + r * Cfg::REC_BYTES, &maps.w0, (int)((kg * 4 + r) * 48), (int)m0, bar);
                    tma_load_2d(dst + 4 * Cfg::REC_BYTES, &maps.w1, (int)(kg * 16), (int)m0, bar);
                    tma_load_2d(dst + 4 * Cfg::REC_BYTES + GM * 16, &maps.w2, (int)((kg >> 3) * 16), (int)m0, bar);
                }
            }
        }
    } else if (warp == 1) {
        // (tensor-memory allocation warp: nothing in the main loop)
    } else if (warp == (uint32_t)g_mma_warp(PH)) {
        // ---- MMA issuer: one thread of the pair's leader CTA ----
        // Issuing four MMAs costs this thread most of the time the tensor pipe needs to run
        // them, so everything else is kept off its path: the test of the NEXT chunk's barrier
        // is started before the current chunk's MMAs are issued and only read afterwards (its
        // shared-memory latency overlaps the issue), the stage index is a compile-time
        // constant (operand descriptors differ by constants), and only the first MMA of the
        // tile carries the "overwrite" predicate.
        // The whole warp runs the loop with uniform control flow and one elected lane issues:
        // operands that are warp-uniform can then live in uniform registers, which is what the
        // MMA and commit instructions read.
        if (rank == 0) {
            const uint32_t idesc = umma_idesc();
            const uint32_t ta0 = tmem_d + GN; // weight chunks follow the accumulator
            const uint64_t bd0 = umma_desc_sw128(smem_u32(b_tiles));
            bool ok = (mode & 8u) ? true : warp_wait(&full[0], 0, lane);
            for (uint32_t g0 = 0, it = 0; g0 < nchunks && ok; g0 += G_STAGES, ++it) {
#pragma unroll
                for (uint32_t c = 0; c < G_STAGES; ++c) {
                    const uint32_t g = g0 + c;
                    if (g >= nchunks || !ok) break;
                    const bool tr = traced && g < 1024 && lane == 0;
                    if (tr) trace[4 * g] = clock64();
                    if (tr && g >= 96 && g < 112) {
                        unsigned long long gt;
                        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
                        trace[7000 + 16 * 32 + (g - 96)] = (long long)gt;
                    }
                    const uint32_t cn = (c + 1) % G_STAGES, parn = (c + 1 == G_STAGES ? it + 1 : it) & 1;
                    const bool has_next = g + 1 < nchunks && !(mode & 8u);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t ad = ta0 + c * G_A_COLS;
                    const uint64_t bd = bd0 + (uint64_t)(c * (G_B_BYTES >> 4));
                    // One instruction sequence: start the test of the next chunk's barrier, issue the four
                    // MMAs (K = 16 each: 32 bytes along the swizzle row) and the commit, and only then read
                    // the test's result, so that nothing issued in between waits for it.
                    uint32_t next_ready;
                    if (DBG && (mode & 28u)) { // measurement variants: pieces of the sequence left out
                        next_ready = (mode & 8u) ? 1u : (uint32_t)mbar_test_wait(&full[cn], parn);
                        if (!(mode & 4u) && lane == 0) {
                            umma_bf16(tmem_d, ad, bd, idesc, g != 0);
                            umma_bf16_acc(tmem_d, ad + 8, bd + 2, idesc);
                            umma_bf16_acc(tmem_d, ad + 16, bd + 4, idesc);
                            umma_bf16_acc(tmem_d, ad + 24, bd + 6, idesc);
                        }
                        if (!(mode & 16u) && lane == 0) umma_commit_pair(&freeb[c]);
                    } else
                    asm volatile(
                        "{\n"
                        ".reg .pred pw, pa, pt, pe;\n"
                        ".reg .b32 a1, a2, a3;\n"
                        ".reg .b64 b1, b2, b3;\n"
                        "setp.ne.b32 pa, %7, 0;\n"
                        "setp.eq.b32 pt, 0, 0;\n"
                        "elect.sync _|pe, 0xffffffff;\n"
                        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 pw, [%1], %2;\n"
                        "add.u32 a1, %4, 8;\n add.u32 a2, %4, 16;\n add.u32 a3, %4, 24;\n"
                        "add.u64 b1, %5, 2;\n add.u64 b2, %5, 4;\n add.u64 b3, %5, 6;\n"
                        "@pe tcgen05.mma.cta_group::2.kind::f16 [%3], [%4], %5, %6, pa;\n"
                        "@pe tcgen05.mma.cta_group::2.kind::f16 [%3], [a1], b1, %6, pt;\n"
                        "@pe tcgen05.mma.cta_group::2.kind::f16 [%3], [a2], b2, %6, pt;\n"
                        "@pe tcgen05.mma.cta_group::2.kind::f16 [%3], [a3], b3, %6, pt;\n"
                        "@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%8], %9;\n"
                        "selp.u32 %0, 1, 0, pw;\n"
                        "}"
                        : "=r"(next_ready)
                        : "r"(smem_u32(&full[cn])), "r"(parn), "r"(tmem_d), "r"(ad), "l"(bd), "r"(idesc), "r"((uint32_t)(g != 0)),
                          "r"(smem_u32(&freeb[c])), "h"((uint16_t)3)
                        : "memory");
                    if (!has_next) next_ready = 1;
                    if (tr) trace[4 * g + 1] = clock64();
                    if (!__all_sync(0xffffffffu, next_ready != 0)) ok = warp_wait(&full[cn], parn, lane);
                    if (tr) trace[4 * g + 3] = clock64();
                }
            }
            if (lane == 0) {
                if (ok) umma_commit_pair(&acc_full);
                else *(volatile int *)p.status = DEV_TIMEOUT;
            }
        }
    } else {
        // ---- dequantization: the 256 threads of a phase work on one 64-k chunk at a time ----
        // a warp reaches only its own quarter of the tensor-memory lanes: row = lane of that quarter
        const uint32_t dt = tid - 64, lq = warp & 3, row = lq * 32 + lane, part = ((warp - 2) >> 2) & 1, phase = (warp - 2) >> 3;
        const uint32_t ta_lane = tmem_d + ((lq * 32u) << 16) + GN;
        bool ok = true;
        for (uint32_t kb = 0; kb < nb && ok; ++kb) {
            const uint32_t st = kb % RS;
            ok = warp_wait(&raw_full[st], (kb / RS) & 1, lane);
            if (!ok) break;
            Blk blk;
            if constexpr (FMT == FMT_MLX4) blk_load_mlx(blk, smem_u32(raw + st * Cfg::RAW_BYTES), row, part, kb0 + kb, p.tbl_bytes);
            else blk_load(blk, smem_u32(raw + st * Cfg::RAW_BYTES), row, part, kb0 + kb);
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_free[st]); // the block's bytes are in registers: its stage can be refilled
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t g = 4 * kb + c, ca = g % G_STAGES;
                if (g % PH != phase) continue; // another phase's chunk
                const bool tr = traced && g < 1024 && dt == 0;
                if (tr) trace[4096 + 4 * g] = clock64();
                if (g >= G_STAGES && !(mode & 16u)) ok = ok && warp_wait(&freeb[ca], ((g / G_STAGES) - 1) & 1, lane);
                if (tr) trace[4096 + 4 * g + 1] = clock64();
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); // the MMAs that read this stage are done
                if (!(mode & 1u)) chunk_store(blk, c, part, ta_lane + ca * G_A_COLS);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); // the chunk is in tensor memory
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&full[ca]), 0));
                if (DBG && traced_any && blockIdx.x < 2 && blockIdx.y == 0 && lane == 0 && g >= 96 && g < 112) {
                    unsigned long long gt;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
                    trace[7000 + (g - 96) * 32 + rank * 16 + (warp - 2)] = (long long)gt;
                }
                if (tr) trace[4096 + 4 * g + 2] = clock64();
            }
        }
        if (!ok) *(volatile int *)p.status = DEV_TIMEOUT;
        // ---- epilogue: TMEM -> registers -> Y[token, row] ----
        if (ok && warp_wait(&acc_full, 0, lane)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t q = warp & 3, colq = (warp - 2) >> 2; // TMEM lane quarter of this warp, column quarter
            const uint32_t orow = m0 + q * 32 + lane;
#pragma unroll 1
            for (uint32_t cb = 0; cb < 2 && colq < 4; ++cb) { // sixteen warps cover the 4 x 4 (lane quarter, column quarter) grid
                const uint32_t col0 = colq * 64 + cb * 32;
                uint32_t v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(tmem_d + ((q * 32u) << 16) + col0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.epi == EPI_SWIGLU) {
                    // rows are interleaved (gate_j, up_j): neighbouring lanes hold the pair (math.rs:103-105)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float a = __uint_as_float(v[j]), o = __shfl_xor_sync(0xffffffffu, a, 1);
                        const uint32_t tok = n0 + col0 + j;
                        if (!(lane & 1) && orow < p.out_dim && tok < p.s)
                            yout[(size_t)tok * (p.ldy >> 1) + (orow >> 1)] = __fdividef(a, 1.0f + __expf(-a)) * o; // operands are bf16 products: fast exp / divide lose nothing that matters
                    }
                } else if (orow < p.out_dim) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t tok = n0 + col0 + j;
                        if (tok < p.s) {
                            const size_t at = (size_t)tok * p.ldy + orow;
                            if (p.sh_world) {
                                for (int r = 0; r < p.sh_world; ++r) *(float *)((char *)(yout + at) + p.sh_delta[r]) = __uint_as_float(v[j]);
                            } else {
                                yout[at] = p.epi == EPI_RESIDUAL ? p.res[at] + __uint_as_float(v[j]) : __uint_as_float(v[j]);
                            }
                        }
                    }
                }
            }
        } else if (ok) {
            *(volatile int *)p.status = DEV_TIMEOUT;
        }
    }
    // Neither CTA leaves, or frees tensor memory, while the other may still read its shared
    // memory (the leader's MMAs), signal its barriers or hold accumulator rows.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)G_TMEM_COLS) : "memory");
    }
}

// X f32 [s, in] -> bf16 (round to nearest even), the tensor cores' input type
__global__ void cast_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ y, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *(const float4 *)(x + i);
        uint2 o;
        o.x = pack_bf16x2(v.x, v.y), o.y = pack_bf16x2(v.z, v.w);
        *(uint2 *)(y + i) = o;
    } else {
        for (size_t j = i; j < n; ++j) y[j] = __float2bfloat16_rn(x[j]);
    }
}

// split-K: the [s, rows] partial sums of the k slices added in slice order (deterministic), then the
// epilogue; y / res have `ldy` elements between tokens
struct ShardDeltas {
    int world;
    long long delta[SHARD_MAX_RANKS];
};
__global__ void splitk_reduce_kernel(const float *__restrict__ part, float *y, size_t s, size_t rows, size_t ldy, int splits, int epi,
                                     const float *res, const ShardDeltas sd) {
    const size_t n = s * rows, i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const int cnt = i + 3 < n ? 4 : (int)(n - i);
    if (cnt == 4 && rows % 4 == 0) {
        for (int z = 0; z < splits; ++z) {
            const float4 b = *(const float4 *)(part + (size_t)z * n + i);
            a[0] += b.x, a[1] += b.y, a[2] += b.z, a[3] += b.w;
        }
    } else {
        for (int z = 0; z < splits; ++z)
            for (int k = 0; k < cnt; ++k) a[k] += part[(size_t)z * n + i + k];
    }
    if (epi == EPI_SWIGLU) { // rows is even and i a multiple of 4: a (gate, up) pair never straddles two threads or tokens
        for (int k = 0; k + 1 < cnt; k += 2) {
            const size_t tok = (i + k) / rows, r = (i + k) % rows;
            y[tok * (ldy >> 1) + (r >> 1)] = __fdividef(a[k], 1.0f + __expf(-a[k])) * a[k + 1];
        }
    } else {
        for (int k = 0; k < cnt; ++k) {
            const size_t tok = (i + k) / rows, r = (i + k) % rows, at = tok * ldy + r;
            if (sd.world) {
                for (int q = 0; q < sd.world; ++q) *(float *)((char *)(y + at) + sd.delta[q]) = a[k];
            } else {
                y[at] = epi == EPI_RESIDUAL ? res[at] + a[k] : a[k];
            }
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D row-major tensor [rows, inner elements], box [box_rows, box_inner]
static bool encode_2d(EncodeTiledFn enc, CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t rows,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle sw) {
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstride[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows}, estr[2] = {1, 1};
    return enc(map, dt, 2, const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef ULLM_TUNING
static uint32_t g_gemm_mode = 0;
static long long *g_gemm_trace = nullptr;
void gemm_set_trace(void *d_buf) { g_gemm_trace = (long long *)d_buf; }
void gemm_set_debug_mode(int mode) { g_gemm_mode = (uint32_t)mode; }
#endif

bool gemm_tc_supported_mlx4(size_t out_dim, size_t in_dim, size_t s, const MlxTables &tb) {
    if (tb.group != 64 || (tb.elem_bytes != 2 && tb.elem_bytes != 4) || !tb.scales || !tb.biases) return false;
    if (in_dim % QK_K || in_dim < QK_K || out_dim == 0 || s == 0) return false;
    if (((in_dim / 64) * tb.elem_bytes) % 16) return false; // table rows are TMA rows: strides in multiples of 16 bytes
    if (((uintptr_t)tb.scales | (uintptr_t)tb.biases) & 15) return false;
    return in_dim <= (1u << 24) && out_dim <= (1u << 30) && s <= (1u << 30);
}

bool gemm_tc_supported(int fmt, size_t out_dim, size_t in_dim, size_t s) {
    if (fmt != FMT_Q4K && fmt != FMT_Q6KR) return false;
    if (in_dim % QK_K || in_dim < QK_K || out_dim == 0 || s == 0) return false;
    if (fmt == FMT_Q6KR && in_dim % 2048) return false;
    return in_dim <= (1u << 24) && out_dim <= (1u << 30) && s <= (1u << 30);
}

// Matrices with few row tiles leave most SMs idle: their k range is split over grid.z slices
// (whole 256-k blocks each), partial sums go to scratch and are added in slice order.
static int gemm_splits(size_t out_dim, size_t in_dim, size_t s, int sm_count) {
    const size_t ctas = 2 * ((out_dim + 2 * GM - 1) / (2 * GM)) * ((s + GN - 1) / GN), nb = in_dim / QK_K;
    if (ctas * 2 > (size_t)sm_count) return 1;
    size_t z = (size_t)sm_count / ctas;
    if (z > nb / 2) z = nb / 2; // at least two blocks per slice
    if (z > 16) z = 16;
    return z < 2 ? 1 : (int)z;
}
static size_t x16_bytes(size_t in_dim, size_t s) { return (s * in_dim * 2 + 255) & ~(size_t)255; }

// How a product is launched.  When the tiles need more than one wave of CTA pairs and the last wave
// would be less than half full, the rows of that last wave are cut off into a second launch with
// split-K (a [256 x 256] tile per pair is 75 % efficiency at 3.03 waves, and k slices of two rows of
// tiles fill the machine instead).
struct GemmPlan {
    size_t rows_main = 0, rows_tail = 0;
    int z_main = 1, z_tail = 1;
};
static GemmPlan gemm_plan(size_t out_dim, size_t in_dim, size_t s, int sm_count) {
    GemmPlan pl;
    const size_t pairs = (size_t)sm_count / 2, row_tiles = (out_dim + 2 * GM - 1) / (2 * GM), tok_tiles = (s + GN - 1) / GN;
    const size_t total = row_tiles * tok_tiles, rem = pairs ? total % pairs : 0;
    pl.rows_main = out_dim;
    if (total <= pairs) {
        pl.z_main = gemm_splits(out_dim, in_dim, s, sm_count);
    } else if (rem != 0 && rem * 2 <= pairs) {
        const size_t tail_tiles = (rem + tok_tiles - 1) / tok_tiles;
        if (tail_tiles < row_tiles) {
            pl.rows_main = (row_tiles - tail_tiles) * 2 * GM;
            pl.rows_tail = out_dim - pl.rows_main;
            pl.z_tail = gemm_splits(pl.rows_tail, in_dim, s, sm_count);
        }
    }
    return pl;
}

size_t gemm_tc_scratch_bytes(size_t out_dim, size_t in_dim, size_t s, int sm_count) {
    const GemmPlan pl = gemm_plan(out_dim, in_dim, s, sm_count);
    const size_t pm = pl.z_main > 1 ? (size_t)pl.z_main * s * pl.rows_main * 4 : 0, pt = pl.z_tail > 1 ? (size_t)pl.z_tail * s * pl.rows_tail * 4 : 0;
    return x16_bytes(in_dim, s) + std::max(pm, pt);
}

template <int FMT, bool DBG> static cudaError_t launch_one(const GemmParams &p, const GemmMaps &maps, dim3 grid, cudaStream_t st) {
    using Cfg = GemmCfg<FMT>;
    const size_t smem = (size_t)G_STAGES * G_B_BYTES + (size_t)Cfg::RAW_STAGES * Cfg::RAW_BYTES + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_q_tc_kernel<FMT, DBG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gemm_q_tc_kernel<FMT, DBG><<<grid, g_threads(Cfg::PHASES), smem, st>>>(p, maps);
    return cudaGetLastError();
}

// One launch (plus the split-K reduction) over `rows` weight rows starting at `w`; y / res point at the
// first of these rows' outputs, `ldy` elements between tokens.
static cudaError_t gemm_part(EncodeTiledFn enc, int fmt, const uint8_t *w, size_t rows, size_t in_dim, size_t s, int z, GemmMaps maps,
                             float *y, const float *res, size_t ldy, int epi, float *part, int *d_status, cudaStream_t st,
                             const ShardDev *shard, const MlxTables *mlx = nullptr, size_t mlx_row0 = 0) {
    const size_t nb = in_dim / QK_K;
    bool ok = true;
    if (fmt == FMT_MLX4) {
        const size_t rb = in_dim / 2, trb = (in_dim / 64) * mlx->elem_bytes;
        const uint8_t *sc = (const uint8_t *)mlx->scales + mlx_row0 * trb, *bi = (const uint8_t *)mlx->biases + mlx_row0 * trb;
        ok = encode_2d(enc, &maps.w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, rb, rows, rb, 128, GM, CU_TENSOR_MAP_SWIZZLE_NONE) &&
             encode_2d(enc, &maps.w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, sc, trb, rows, trb, 16, GM, CU_TENSOR_MAP_SWIZZLE_NONE) &&
             encode_2d(enc, &maps.w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, bi, trb, rows, trb, 16, GM, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else if (fmt == FMT_Q4K) {
        const size_t rb = nb * Q4K_BYTES;
        ok = encode_2d(enc, &maps.w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, rb, rows, rb, Q4K_BYTES, GM, CU_TENSOR_MAP_SWIZZLE_NONE);
        maps.w1 = maps.w0, maps.w2 = maps.w0;
    } else {
        const size_t rb = nb * Q6K_BYTES; // prepared rows: records | scales | d planes
        ok = encode_2d(enc, &maps.w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, nb * 192, rows, rb, 48, GM, CU_TENSOR_MAP_SWIZZLE_NONE) &&
             encode_2d(enc, &maps.w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, w + nb * 192, nb * 16, rows, rb, 16, GM, CU_TENSOR_MAP_SWIZZLE_NONE) &&
             encode_2d(enc, &maps.w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, w + nb * 208, nb * 2, rows, rb, 16, GM, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (!ok) return cudaErrorInvalidValue;
    GemmParams p;
    p.blocks_per_split = (uint32_t)((nb + z - 1) / z);
    const unsigned gz = (unsigned)((nb + p.blocks_per_split - 1) / p.blocks_per_split);
    p.y = gz > 1 ? part : y, p.status = d_status;
    p.epi = gz > 1 ? EPI_STORE : epi, p.res = res, p.ldy = gz > 1 ? (uint32_t)rows : (uint32_t)ldy;
    p.out_dim = (uint32_t)rows, p.in_dim = (uint32_t)in_dim, p.s = (uint32_t)s;
    p.tbl_bytes = mlx ? (uint32_t)mlx->elem_bytes : 0u;
    // sharded: the launch that produces the final values stores them into every rank's buffer
    ShardDeltas sd{};
    if (shard) {
        sd.world = shard->world;
        for (int r = 0; r < shard->world; ++r) sd.delta[r] = shard->delta[r];
    }
    p.sh_world = gz > 1 ? 0 : sd.world;
    for (int r = 0; r < SHARD_MAX_RANKS; ++r) p.sh_delta[r] = sd.delta[r];
    const dim3 grid(2 * (unsigned)((rows + 2 * GM - 1) / (2 * GM)), (unsigned)((s + GN - 1) / GN), gz);
    cudaError_t e;
#ifdef ULLM_TUNING
    p.mode = g_gemm_mode, p.trace = g_gemm_trace;
    if (p.mode || p.trace) e = fmt == FMT_Q4K ? launch_one<FMT_Q4K, true>(p, maps, grid, st) : launch_one<FMT_Q6KR, true>(p, maps, grid, st);
    else
#endif
    e = fmt == FMT_Q4K ? launch_one<FMT_Q4K, false>(p, maps, grid, st)
                       : (fmt == FMT_MLX4 ? launch_one<FMT_MLX4, false>(p, maps, grid, st) : launch_one<FMT_Q6KR, false>(p, maps, grid, st));
    if (e != cudaSuccess || gz == 1) return e;
    const size_t ny = s * rows;
    splitk_reduce_kernel<<<(unsigned)((ny / 4 + 255) / 256 + 1), 256, 0, st>>>(part, y, s, rows, ldy, (int)gz, epi, res, sd);
    return cudaGetLastError();
}

// d_w: FMT_Q4K verbatim rows or FMT_Q6KR prepared rows (16-byte aligned).  d_x f32 [s, in],
// d_y f32 [s, out], d_xb16: scratch of gemm_tc_scratch_bytes (256-byte aligned).
cudaError_t launch_gemm_tc(int fmt, const void *d_w, const float *d_x, float *d_y, void *d_xb16, size_t out_dim, size_t in_dim,
                           size_t s, int sm_count, int *d_status, cudaStream_t st, int epi, const float *d_res, size_t ldy,
                           const ShardDev *shard, const MlxTables *mlx) {
    if (ldy == 0) ldy = out_dim;
    if (shard && (epi != EPI_STORE || shard->world < 1 || shard->world > SHARD_MAX_RANKS)) return cudaErrorInvalidValue;
    if (epi == EPI_SWIGLU && (out_dim & 1)) return cudaErrorInvalidValue;
    if (epi == EPI_RESIDUAL && !d_res) return cudaErrorInvalidValue;
    const bool supported = fmt == FMT_MLX4 ? (mlx && gemm_tc_supported_mlx4(out_dim, in_dim, s, *mlx)) : gemm_tc_supported(fmt, out_dim, in_dim, s);
    if (!supported || ((uintptr_t)d_w & 15)) return cudaErrorNotSupported;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    const size_t n = s * in_dim, row_bytes = fmt == FMT_MLX4 ? in_dim / 2 : in_dim / QK_K * (fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
    cast_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, st>>>(d_x, (__nv_bfloat16 *)d_xb16, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    GemmMaps maps;
    if (!encode_2d(enc, &maps.x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d_xb16, in_dim, s, in_dim * 2, GKC, GNH, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    float *part = (float *)((uint8_t *)d_xb16 + x16_bytes(in_dim, s));
    const GemmPlan pl = gemm_plan(out_dim, in_dim, s, sm_count);
    const uint8_t *w = (const uint8_t *)d_w;
    const size_t ydiv = epi == EPI_SWIGLU ? 2 : 1; // SwiGLU halves the output rows
    e = gemm_part(enc, fmt, w, pl.rows_main, in_dim, s, pl.z_main, maps, d_y, d_res, ldy, epi, part, d_status, st, shard, mlx, 0);
    if (e != cudaSuccess || pl.rows_tail == 0) return e;
    return gemm_part(enc, fmt, w + pl.rows_main * row_bytes, pl.rows_tail, in_dim, s, pl.z_tail, maps, d_y + pl.rows_main / ydiv,
                     d_res ? d_res + pl.rows_main : nullptr, ldy, epi, part, d_status, st, shard, mlx, pl.rows_main);
}

} // namespace ullm
