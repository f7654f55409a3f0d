// Prefill GEMM on quantized weights:  Y[s, o] = sum_i W[o, i] * X[s, i]  for many
// tokens at once (CPU form: matmul_q, crates/ullm-model/src/math.rs:38-63; Metal form:
// matmul_q4k / matmul_q6k, crates/ullm-metal/src/shader.metal:620-740).
//
// A dense contraction, so it runs on the 5th-generation tensor cores: per CTA a
// [128 weight rows x 256 tokens] fp32 accumulator lives in tensor memory (TMEM);
// producer warps dequantize the packed weight blocks to bf16 (values rounded once,
// from the exact f32 dequantization) straight into the 128-byte-swizzled K-major
// shared-memory layout `tcgen05.mma` reads, the bf16 activation tile arrives by
// tiled TMA with the same swizzle, one elected thread issues the MMAs
// (kind::f16, M=128, N=256, K=16, cta_group::1) and commits them onto the mbarriers
// that recycle the operand slots.  The epilogue reads the accumulator back with
// tcgen05.ld and stores token-major f32.
//
// Roles in a CTA of 10 warps:
//   warp 0      TMA: activation tile [256 tokens x 64 k] per k-chunk, 4 slots
//   warp 1      TMEM allocation, MMA issue, commits
//   warps 2-9   dequantization (thread = (row, half of the 256-k block)), then epilogue
// Every mbarrier wait is bounded; on expiry the CTA records a status, stops issuing
// work, still frees its TMEM and leaves.
#include "kernels.h"
#include "matvec_core.cuh"

#include <cuda.h>

namespace ullm {

constexpr int GM = 128;  // weight rows per CTA (MMA M)
constexpr int GN = 256;  // tokens per CTA (MMA N, TMEM columns)
constexpr int GKC = 64;  // k per chunk: 64 bf16 = one 128-byte swizzle row
constexpr int G_SLOTS = 4;
constexpr int G_A_BYTES = GM * GKC * 2;  // 16 KB
constexpr int G_B_BYTES = GN * GKC * 2;  // 32 KB
constexpr int G_THREADS = 320;

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
// instruction descriptor: D f32, A/B bf16, both K-major, M = 128, N = 256
__host__ __device__ constexpr uint32_t umma_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GN >> 3) << 17) | ((uint32_t)(GM >> 4) << 24);
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// 16 bytes of row `row`, 16-byte column `c16` (0..7) of a [rows x 128 B] tile with the
// 128-byte swizzle: the column index is XORed with the row index modulo 8.
__device__ __forceinline__ void st_a_sw128(uint32_t tile, uint32_t row, uint32_t c16, uint4 v) {
    const uint32_t addr = tile + row * 128u + ((c16 ^ (row & 7u)) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

struct GemmParams {
    const uint8_t *w;  // FMT_Q4K verbatim rows or FMT_Q6KR prepared rows
    float *y;          // [s, out]
    int *status;
    uint32_t out_dim, in_dim, s;
};

// ---- raw bytes one dequant thread needs for (row, 256-k block, half h) ----------
struct RawQ4K {
    uint4 hdr;     // d, dmin, 12 packed scale bytes
    uint4 qs[4];   // qs[64h .. 64h+63]: chunks 2h and 2h+1
};
struct RawQ6KR {
    uint4 rec[6];  // records (h, t'=0) and (h, t'=1): W1, W2, W3 each
    uint2 sc;      // their 2 x 4 int8 scales
    uint32_t d;    // f16 bits
};

__device__ __forceinline__ void raw_load(RawQ4K &r, const uint8_t *w, uint32_t row, uint32_t nb, uint32_t kb, uint32_t h) {
    const uint4 *blk = (const uint4 *)(w + ((size_t)row * nb + kb) * Q4K_BYTES);
    r.hdr = __ldg(blk);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.qs[i] = __ldg(blk + 1 + 4 * h + i);
}
__device__ __forceinline__ void raw_load(RawQ6KR &r, const uint8_t *w, uint32_t row, uint32_t nb, uint32_t kb, uint32_t h) {
    const uint8_t *rw = w + (size_t)row * nb * Q6K_BYTES;
    const uint32_t ri = kb * 4 + h * 2;
    const uint4 *rec = (const uint4 *)(rw + (size_t)ri * 48);
#pragma unroll
    for (int i = 0; i < 6; ++i) r.rec[i] = __ldg(rec + i);
    r.sc = __ldg((const uint2 *)(rw + (size_t)nb * 192 + (size_t)ri * 4));
    r.d = __ldg((const uint16_t *)(rw + (size_t)nb * 208 + (size_t)kb * 2));
}
__device__ __forceinline__ void raw_zero(RawQ4K &r) {
    r.hdr = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.qs[i] = make_uint4(0, 0, 0, 0);
}
__device__ __forceinline__ void raw_zero(RawQ6KR &r) {
#pragma unroll
    for (int i = 0; i < 6; ++i) r.rec[i] = make_uint4(0, 0, 0, 0);
    r.sc = make_uint2(0, 0), r.d = 0;
}

__device__ __forceinline__ uint32_t byte_of(const uint4 &v, int i) {
    const uint32_t w = i < 4 ? v.x : (i < 8 ? v.y : (i < 12 ? v.z : v.w));
    return (w >> (8 * (i & 3))) & 0xffu;
}

// Writes the two k-chunks (2h, 2h+1) of one row into their A tiles, values computed as
// crates/ullm-core/src/dequant.rs:203-210 does (d*sc exact, (d*sc)*q exact, one rounding
// at the subtraction) and then rounded once more to bf16.
__device__ __forceinline__ void dequant_store(const RawQ4K &r, uint32_t h, uint32_t row, uint32_t tile_c0, uint32_t tile_c1) {
    const float d = f16_bits_to_f32((uint16_t)(r.hdr.x & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(r.hdr.x >> 16));
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        int sA, mA, sB, mB;
        q4k_pair(r.hdr.y, r.hdr.z, r.hdr.w, (int)(2 * h + cc), sA, mA, sB, mB);
        const float d1 = __fmul_rn(d, (float)sA), m1 = __fmul_rn(dmin, (float)mA);
        const float d2 = __fmul_rn(d, (float)sB), m2 = __fmul_rn(dmin, (float)mB);
        const uint32_t tile = cc ? tile_c1 : tile_c0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { // 8 qs bytes -> 8 low-nibble and 8 high-nibble values
            const uint4 &q = r.qs[2 * cc + (j >> 1)];
            const uint32_t w0 = (j & 1) ? q.z : q.x, w1 = (j & 1) ? q.w : q.y;
            float lo[8], hi[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint32_t byte = ((b < 4 ? w0 : w1) >> (8 * (b & 3))) & 0xffu;
                lo[b] = __fsub_rn(__fmul_rn(d1, (float)(byte & 15u)), m1);
                hi[b] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
            }
            st_a_sw128(tile, row, j, make_uint4(pack_bf16x2(lo[0], lo[1]), pack_bf16x2(lo[2], lo[3]), pack_bf16x2(lo[4], lo[5]), pack_bf16x2(lo[6], lo[7])));
            st_a_sw128(tile, row, 4 + j, make_uint4(pack_bf16x2(hi[0], hi[1]), pack_bf16x2(hi[2], hi[3]), pack_bf16x2(hi[4], hi[5]), pack_bf16x2(hi[6], hi[7])));
        }
    }
}

// Prepared Q6_K (prepare.cu): value = (d * sc) * (q - 32), left to right as
// dequant.rs:275-278.  Half h of the block is k-chunks 2h (groups 0, 1) and 2h+1 (2, 3).
__device__ __forceinline__ void dequant_store(const RawQ6KR &r, uint32_t h, uint32_t row, uint32_t tile_c0, uint32_t tile_c1) {
    const float d = f16_bits_to_f32((uint16_t)r.d);
#pragma unroll
    for (int tp = 0; tp < 2; ++tp) {
        const uint4 &W1 = r.rec[3 * tp], &W2 = r.rec[3 * tp + 1], &W3 = r.rec[3 * tp + 2];
        const uint32_t scw = tp ? r.sc.y : r.sc.x;
        float ds[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) ds[g] = __fmul_rn(d, (float)((int)(scw << (24 - 8 * g)) >> 24));
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) { // positions l = 16tp + 8hf .. +7
            float v[4][8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint32_t w1 = byte_of(W1, 8 * hf + b), w2 = byte_of(W2, 8 * hf + b), w3 = byte_of(W3, 8 * hf + b);
                const int q0 = (int)(w1 & 0x3f), q1 = (int)((w2 & 0xf) | ((w1 >> 6) << 4));
                const int q2 = (int)((w2 >> 4) | ((w3 >> 6) << 4)), q3 = (int)(w3 & 0x3f);
                v[0][b] = __fmul_rn(ds[0], (float)(q0 - 32));
                v[1][b] = __fmul_rn(ds[1], (float)(q1 - 32));
                v[2][b] = __fmul_rn(ds[2], (float)(q2 - 32));
                v[3][b] = __fmul_rn(ds[3], (float)(q3 - 32));
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint32_t tile = g < 2 ? tile_c0 : tile_c1;
                const uint32_t c16 = 4 * (g & 1) + 2 * tp + hf;
                st_a_sw128(tile, row, c16, make_uint4(pack_bf16x2(v[g][0], v[g][1]), pack_bf16x2(v[g][2], v[g][3]), pack_bf16x2(v[g][4], v[g][5]), pack_bf16x2(v[g][6], v[g][7])));
            }
        }
    }
}

template <int FMT> struct RawOf;
template <> struct RawOf<FMT_Q4K> { using type = RawQ4K; };
template <> struct RawOf<FMT_Q6KR> { using type = RawQ6KR; };

// grid (ceil(out / 128), ceil(s / 256)), 320 threads, dynamic smem: 4 x (16 KB A + 32 KB B)
template <int FMT>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_q_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
    using Raw = typename RawOf<FMT>::type;
    extern __shared__ __align__(1024) uint8_t gsm[];
    // dynamic smem is only guaranteed 16-byte aligned: round up to the 1024 B the swizzle atoms need
    uint8_t *base = (uint8_t *)(((uintptr_t)gsm + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tiles = base;                       // G_SLOTS x 16 KB
    uint8_t *b_tiles = base + G_SLOTS * G_A_BYTES; // G_SLOTS x 32 KB
    __shared__ uint64_t a_full[G_SLOTS], b_full[G_SLOTS], slot_free[G_SLOTS], acc_full;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m0 = blockIdx.x * GM, n0 = blockIdx.y * GN;
    const uint32_t nb = p.in_dim / QK_K, nchunks = nb * 4;

    if (tid == 0) {
        for (int i = 0; i < G_SLOTS; ++i) {
            mbar_init(&a_full[i], 128); // the 128 threads that own this chunk's half
            mbar_init(&b_full[i], 1);
            mbar_init(&slot_free[i], 1);
        }
        mbar_init(&acc_full, 1);
        abort_s = 0;
        mbar_fence_init();
    }
    if (warp == 1) { // TMEM: 256 columns of 128 lanes x 32 bit
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)GN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_s;

    if (warp == 0) {
        // ---- TMA producer: activation tile of every k-chunk ----
        if (lane == 0) {
            for (uint32_t g = 0; g < nchunks; ++g) {
                const uint32_t c = g % G_SLOTS;
                if (g >= G_SLOTS && !wait_or_timeout(&slot_free[c], ((g / G_SLOTS) - 1) & 1)) {
                    abort_s = 1;
                    *(volatile int *)p.status = DEV_TIMEOUT;
                    break;
                }
                mbar_arrive_expect_tx(&b_full[c], G_B_BYTES);
                tma_load_2d(b_tiles + c * G_B_BYTES, &xmap, (int)(g * GKC), (int)n0, &b_full[c]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc();
            bool ok = true;
            for (uint32_t g = 0; g < nchunks && ok; ++g) {
                const uint32_t c = g % G_SLOTS, par = (g / G_SLOTS) & 1;
                ok = wait_or_timeout(&a_full[c], par) && wait_or_timeout(&b_full[c], par);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = umma_desc_sw128(smem_u32(a_tiles + c * G_A_BYTES));
                const uint64_t bd = umma_desc_sw128(smem_u32(b_tiles + c * G_B_BYTES));
#pragma unroll
                for (uint32_t k = 0; k < GKC / 16; ++k) // K = 16 per instruction: 32 bytes along the swizzle row
                    umma_bf16(tmem_d, ad + 2 * k, bd + 2 * k, idesc, (g | k) != 0);
                umma_commit(&slot_free[c]); // operands of this slot may be overwritten once these MMAs are done
            }
            if (ok) umma_commit(&acc_full);
            else {
                abort_s = 1;
                *(volatile int *)p.status = DEV_TIMEOUT;
            }
        }
    } else {
        // ---- dequantization: thread = (row, half of each 256-k block) ----
        const uint32_t dt = tid - 64, row = dt & 127, h = dt >> 7;
        const bool in_range = m0 + row < p.out_dim;
        Raw cur, nxt;
        if (in_range) raw_load(cur, p.w, m0 + row, nb, 0, h);
        else raw_zero(cur);
        bool ok = true;
        for (uint32_t kb = 0; kb < nb && ok; ++kb) {
            if (kb + 1 < nb && in_range) raw_load(nxt, p.w, m0 + row, nb, kb + 1, h); // overlaps the math below
            const uint32_t c0 = 2 * h, c1 = 2 * h + 1;
            if (kb >= 1) ok = wait_or_timeout(&slot_free[c0], (kb - 1) & 1) && wait_or_timeout(&slot_free[c1], (kb - 1) & 1);
            if (!ok) break;
            dequant_store(cur, h, row, smem_u32(a_tiles + c0 * G_A_BYTES), smem_u32(a_tiles + c1 * G_A_BYTES));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the MMA
            mbar_arrive(&a_full[c0]);
            mbar_arrive(&a_full[c1]);
            if (in_range) cur = nxt;
        }
        if (!ok) {
            abort_s = 1;
            *(volatile int *)p.status = DEV_TIMEOUT;
        }
        // ---- epilogue: TMEM -> registers -> Y[token, row] ----
        if (ok && wait_or_timeout(&acc_full, 0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t q = warp & 3, colh = (warp - 2) >> 2; // TMEM lane quarter of this warp, column half
            const uint32_t orow = m0 + q * 32 + lane;
#pragma unroll 1
            for (uint32_t cb = 0; cb < 4; ++cb) {
                const uint32_t col0 = colh * 128 + cb * 32;
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
                if (orow < p.out_dim) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t tok = n0 + col0 + j;
                        if (tok < p.s) p.y[(size_t)tok * p.out_dim + orow] = __uint_as_float(v[j]);
                    }
                }
            }
        } else if (ok) {
            abort_s = 1;
            *(volatile int *)p.status = DEV_TIMEOUT;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)GN) : "memory");
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

bool gemm_tc_supported(int fmt, size_t out_dim, size_t in_dim, size_t s) {
    if (fmt != FMT_Q4K && fmt != FMT_Q6KR) return false;
    if (in_dim % QK_K || in_dim < QK_K || out_dim == 0 || s == 0) return false;
    if (fmt == FMT_Q6KR && in_dim % 2048) return false;
    return in_dim <= (1u << 30) && out_dim <= (1u << 30) && s <= (1u << 30);
}

size_t gemm_tc_scratch_bytes(size_t in_dim, size_t s) { return s * in_dim * 2; }

// d_w: FMT_Q4K verbatim rows or FMT_Q6KR prepared rows.  d_x f32 [s, in], d_y f32 [s, out],
// d_xb16: scratch of gemm_tc_scratch_bytes (256-byte aligned).
cudaError_t launch_gemm_tc(int fmt, const void *d_w, const float *d_x, float *d_y, void *d_xb16, size_t out_dim, size_t in_dim,
                           size_t s, int *d_status, cudaStream_t st) {
    if (!gemm_tc_supported(fmt, out_dim, in_dim, s)) return cudaErrorNotSupported;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    const size_t n = s * in_dim;
    cast_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256 + 1), 256, 0, st>>>(d_x, (__nv_bfloat16 *)d_xb16, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)in_dim, (cuuint64_t)s};
    const cuuint64_t gstride[1] = {(cuuint64_t)in_dim * 2};
    const cuuint32_t box[2] = {GKC, GN}, estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d_xb16, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    GemmParams p;
    p.w = (const uint8_t *)d_w, p.y = d_y, p.status = d_status;
    p.out_dim = (uint32_t)out_dim, p.in_dim = (uint32_t)in_dim, p.s = (uint32_t)s;
    const dim3 grid((unsigned)((out_dim + GM - 1) / GM), (unsigned)((s + GN - 1) / GN));
    const size_t smem = (size_t)G_SLOTS * (G_A_BYTES + G_B_BYTES) + 1024;
    if (fmt == FMT_Q4K) {
        static bool set = false;
        if (!set) {
            if ((e = cudaFuncSetAttribute(gemm_q_tc_kernel<FMT_Q4K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
            set = true;
        }
        gemm_q_tc_kernel<FMT_Q4K><<<grid, G_THREADS, smem, st>>>(p, map);
    } else {
        static bool set = false;
        if (!set) {
            if ((e = cudaFuncSetAttribute(gemm_q_tc_kernel<FMT_Q6KR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
            set = true;
        }
        gemm_q_tc_kernel<FMT_Q6KR><<<grid, G_THREADS, smem, st>>>(p, map);
    }
    return cudaGetLastError();
}

} // namespace ullm
