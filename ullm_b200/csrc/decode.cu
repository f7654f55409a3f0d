// One decode step of a dense Llama-family model with every weight resident and
// quantized (CPU form: crates/ullm-model/src/lib.rs:807-969; GPU surface:
// crates/ullm-metal/src/forward.rs:384-526).
//
// Per layer the step is five launches, all HBM-streaming matvecs except the
// attention:
//   [rmsnorm ->] W_qk x      (Q and K projections stored as one matrix)
//   [rmsnorm ->] W_v  x
//   bias / per-head norm / rope of q and k, K/V cache write, split-KV attention, split combine
//   W_o attn  (+ residual, in the epilogue)
//   [rmsnorm ->] W_gate|up x (rows interleaved at upload; silu(g)*u in the epilogue)
//   W_down h  (+ residual)
// and norm + output projection at the end.  A mixture-of-experts layer (MLX 4-bit) replaces the
// last two by the router matvec, the routing, the selected experts' gate|up and down kernels (x is
// RMS-normalised in their prologues) and the weighted combine (+ residual): moe.cu; its q, k and v
// projections are one stacked MLX matrix.  The position and the current token
// live in device memory, so the same CUDA graph is replayed for every token: one
// submission per decoded token, and greedy decoding (argmax -> embedding lookup)
// needs no host round trip at all.
#include "decode.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace ullm {

// ---------------------------------------------------------------------------
// Attention for one new token
// ---------------------------------------------------------------------------
constexpr int ATT_CHUNK = 32; // cache positions per CTA: a 1024-position context is 33 x n_kv_head CTAs, each with one batch per warp
constexpr int ATT_MAX_CTX = 8192;

template <typename T> __device__ __forceinline__ float kv_load(const T *p);
template <> __device__ __forceinline__ float kv_load<float>(const float *p) { return __ldcg(p); }
template <> __device__ __forceinline__ float kv_load<__half>(const __half *p) { return __half2float(__ldcg(p)); }
template <typename T> __device__ __forceinline__ T kv_make(float v);
template <> __device__ __forceinline__ float kv_make<float>(float v) { return v; }
template <> __device__ __forceinline__ __half kv_make<__half>(float v) { return __float2half_rn(v); }

// E consecutive cache elements (E = 2 or 4) as one load
template <typename T, int E> __device__ __forceinline__ void kv_load_vec(const T *p, float (&o)[E]);
template <> __device__ __forceinline__ void kv_load_vec<float, 2>(const float *p, float (&o)[2]) {
    const float2 v = __ldcg((const float2 *)p);
    o[0] = v.x, o[1] = v.y;
}
template <> __device__ __forceinline__ void kv_load_vec<float, 4>(const float *p, float (&o)[4]) {
    const float4 v = __ldcg((const float4 *)p);
    o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
}
template <> __device__ __forceinline__ void kv_load_vec<__half, 2>(const __half *p, float (&o)[2]) {
    const unsigned v = __ldcg((const unsigned *)p);
    const float2 f = __half22float2(*(const __half2 *)&v);
    o[0] = f.x, o[1] = f.y;
}
template <> __device__ __forceinline__ void kv_load_vec<__half, 4>(const __half *p, float (&o)[4]) {
    const uint2 v = __ldcg((const uint2 *)p);
    const float2 a = __half22float2(*(const __half2 *)&v.x), b = __half22float2(*(const __half2 *)&v.y);
    o[0] = a.x, o[1] = a.y, o[2] = b.x, o[3] = b.y;
}

template <typename T> __device__ __forceinline__ float kv_f(T v);
template <> __device__ __forceinline__ float kv_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float kv_f<__half>(__half v) { return __half2float(v); }

struct AttnParams {
    const float *q, *knew, *vnew; // projections of the new token (before RoPE)
    void *kcache, *vcache;        // this layer: [n_ctx][kv_dim]
    const float2 *rope;           // [n_ctx][HD/2] (cos, sin) of pos * theta^(-2i/HD)
    const int *pos_ptr;
    float scale;
    float *partial;               // [n_kv_head][n_split][KVMUL][HD + 2]
    unsigned *counters;           // [n_kv_head], zero between launches
    float *out;                   // [n_head * HD]
    int kv_dim, n_split;
    // optional model variants (crates/ullm-model/src/lib.rs:877-909), null / 0 = absent
    const float *q_bias, *k_bias, *v_bias; // added to the projections
    const float *q_norm, *k_norm;          // per-head RMSNorm weights [HD], applied before RoPE
    float eps;
    int neox;                              // rotate-half pairs (i, i + HD/2) instead of (2i, 2i+1)
};

// One head's projection -> (+ bias) -> (per-head RMSNorm) -> RoPE, in shared memory `dst[HD]`, by one
// warp (all 32 lanes call it).  Products and sums unfused as in math.rs:130-132 / :154-158; the norm
// as math.rs:82-86 (x * inv * w, inv = 1 / sqrt(mean(x^2) + eps)).
template <int HD>
__device__ __forceinline__ void head_prepare(const float *__restrict__ src, const float *__restrict__ bias,
                                             const float *__restrict__ norm_w, float eps, const float2 *__restrict__ rp, int neox,
                                             float *dst, int lane) {
    constexpr int E = HD / 32;
    float v[E], ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const int d = lane + 32 * e;
        v[e] = src[d] + (bias ? bias[d] : 0.f);
        ss += v[e] * v[e];
    }
    if (norm_w) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) v[e] = v[e] * inv * norm_w[lane + 32 * e];
    }
#pragma unroll
    for (int e = 0; e < E; ++e) dst[lane + 32 * e] = v[e];
    __syncwarp();
    for (int j = lane; j < HD / 2; j += 32) {
        const int ia = neox ? j : 2 * j, ib = neox ? j + HD / 2 : 2 * j + 1;
        const float a = dst[ia], b = dst[ib];
        const float2 cs = rp[j];
        dst[ia] = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
        dst[ib] = __fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
    }
    __syncwarp();
}

// Sums each of the 32 values over the warp; on return lane L holds the total of
// value index L.
__device__ __forceinline__ float warp_transpose_sum32(float (&v)[32], int lane) {
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
        const bool up = lane & half;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            float send = up ? v[i] : v[i + half];
            float keep = up ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
        }
    }
    return v[0];
}

// grid (n_kv_head, n_split), 128 threads.  CTA (h, s) owns cache positions
// [s*ATT_CHUNK, (s+1)*ATT_CHUNK) of kv head h for its KVMUL query heads; the CTA that owns `pos`
// applies RoPE to the new K, rounds K and V to the cache type and stores them;
// the last CTA of a head to finish merges the per-split softmax partials.
template <int HD, int KVMUL, typename KV_T>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnParams p) {
    constexpr int E = HD / 32;     // dims per lane
    constexpr int PB = 32 / KVMUL; // positions per transposed-reduction batch
    __shared__ float qs[KVMUL][HD];
    __shared__ float sc[KVMUL][ATT_CHUNK];
    __shared__ float red[4][KVMUL][HD];
    __shared__ float ml[KVMUL][2];
    __shared__ bool is_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, sp = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait_prior();
    const int pos = *p.pos_ptr;
    const int n_active = pos / ATT_CHUNK + 1;
    if (sp >= n_active) return;
    const int p0 = sp * ATT_CHUNK, p1 = min(p0 + ATT_CHUNK, pos + 1), np = p1 - p0;
    KV_T *kc = (KV_T *)p.kcache, *vc = (KV_T *)p.vcache;
    const float2 *rp = p.rope + (size_t)pos * (HD / 2);

    // The cache rows of this CTA's positions are requested before anything else: keys of the warp's score batches
    // and values of the warp's positions (warp, warp + 4, ...), so that their trip to memory overlaps the work on
    // the new token below.  The row of `pos` itself is written by this kernel: what is read of it here is stale and
    // is replaced from shared memory (kn / vn, rounded as the cache rounds) where it is used.
    constexpr int NB = (KVMUL + 3) / 4, VPW = ATT_CHUNK / 4; // score batches per warp, values per warp
    float kpre[NB][PB][E], vpre[VPW][E];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int j = 0; j < PB; ++j) {
            const int pp = min(p0 + (warp + 4 * nb) * PB + j, p1 - 1);
            kv_load_vec<KV_T, E>(kc + (size_t)pp * p.kv_dim + kvh * HD + lane * E, kpre[nb][j]);
        }
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
        const int pp = min(p0 + warp + 4 * i, p1 - 1);
        kv_load_vec<KV_T, E>(vc + (size_t)pp * p.kv_dim + kvh * HD + lane * E, vpre[i]);
    }
    const bool owns_pos = sp == n_active - 1;
    __shared__ float vn[HD];

    // the new token's q heads of this kv head (and, in the CTA that owns `pos`, its k and v): bias,
    // per-head norm and RoPE as the model asks, then the cache write
    __shared__ float kn[HD];
    const bool plain = !p.q_bias && !p.k_bias && !p.v_bias && !p.q_norm && !p.k_norm && !p.neox;
    if (plain) {
        // plain Llama: interleaved RoPE only, all pairs in parallel (products and sums unfused, math.rs:130-132)
        for (int i = tid; i < KVMUL * (HD / 2); i += 128) {
            const int h = i / (HD / 2), j = i % (HD / 2);
            const float *qp = p.q + (size_t)(kvh * KVMUL + h) * HD + 2 * j;
            const float a = qp[0], b = qp[1];
            const float2 cs = rp[j];
            qs[h][2 * j] = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
            qs[h][2 * j + 1] = __fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
        }
        if (owns_pos) {
            for (int j = tid; j < HD / 2; j += 128) {
                const float *kp = p.knew + (size_t)kvh * HD + 2 * j;
                const float a = kp[0], b = kp[1];
                const float2 cs = rp[j];
                KV_T *dst = kc + (size_t)pos * p.kv_dim + kvh * HD + 2 * j;
                const KV_T r0 = kv_make<KV_T>(__fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)));
                const KV_T r1 = kv_make<KV_T>(__fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x)));
                dst[0] = r0, dst[1] = r1;
                kn[2 * j] = kv_f<KV_T>(r0), kn[2 * j + 1] = kv_f<KV_T>(r1);
            }
            for (int j = tid; j < HD; j += 128) {
                const KV_T r = kv_make<KV_T>(p.vnew[(size_t)kvh * HD + j]);
                vc[(size_t)pos * p.kv_dim + kvh * HD + j] = r;
                vn[j] = kv_f<KV_T>(r);
            }
        }
    } else {
        for (int h = warp; h < KVMUL; h += 4)
            head_prepare<HD>(p.q + (size_t)(kvh * KVMUL + h) * HD, p.q_bias ? p.q_bias + (size_t)(kvh * KVMUL + h) * HD : nullptr,
                             p.q_norm, p.eps, rp, p.neox, qs[h], lane);
        if (owns_pos && warp == 3) {
            head_prepare<HD>(p.knew + (size_t)kvh * HD, p.k_bias ? p.k_bias + (size_t)kvh * HD : nullptr, p.k_norm, p.eps, rp, p.neox, kn, lane);
            for (int j = lane; j < HD; j += 32) {
                const KV_T rk = kv_make<KV_T>(kn[j]);
                kc[(size_t)pos * p.kv_dim + kvh * HD + j] = rk;
                kn[j] = kv_f<KV_T>(rk);
                const float vv = p.vnew[(size_t)kvh * HD + j] + (p.v_bias ? p.v_bias[(size_t)kvh * HD + j] : 0.f);
                const KV_T rv = kv_make<KV_T>(vv);
                vc[(size_t)pos * p.kv_dim + kvh * HD + j] = rv;
                vn[j] = kv_f<KV_T>(rv);
            }
        }
    }
    __syncthreads();

    // scores: lane owns dims [lane*E, lane*E+E) of every head
    float qr[KVMUL][E];
#pragma unroll
    for (int h = 0; h < KVMUL; ++h)
#pragma unroll
        for (int e = 0; e < E; ++e) qr[h][e] = qs[h][lane * E + e];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int b0 = (warp + 4 * nb) * PB;
        if (b0 >= np) break;
        float v[32];
#pragma unroll
        for (int j = 0; j < PB; ++j) {
            const int pp = min(p0 + b0 + j, p1 - 1);
            float kk[E];
#pragma unroll
            for (int e = 0; e < E; ++e) kk[e] = owns_pos && pp == pos ? kn[lane * E + e] : kpre[nb][j][e];
#pragma unroll
            for (int h = 0; h < KVMUL; ++h) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < E; ++e) s += qr[h][e] * kk[e];
                v[j * KVMUL + h] = s;
            }
        }
        const float tot = warp_transpose_sum32(v, lane);
        const int j = lane / KVMUL, h = lane % KVMUL;
        if (b0 + j < np) sc[h][b0 + j] = tot * p.scale;
    }
    __syncthreads();

    // per-head softmax partials over this CTA's positions
    for (int h = warp; h < KVMUL; h += 4) {
        float m = -INFINITY;
        for (int i = lane; i < np; i += 32) m = fmaxf(m, sc[h][i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < np; i += 32) {
            const float e = expf(sc[h][i] - m);
            sc[h][i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) ml[h][0] = m, ml[h][1] = l;
    }
    __syncthreads();

    // P V: positions split over the warps, dims over the lanes
    float acc[KVMUL][E];
#pragma unroll
    for (int h = 0; h < KVMUL; ++h)
#pragma unroll
        for (int e = 0; e < E; ++e) acc[h][e] = 0.f;
#pragma unroll
    for (int i = 0; i < VPW; ++i) {
        if (warp + 4 * i < np) {
#pragma unroll
            for (int h = 0; h < KVMUL; ++h) {
                const float a = sc[h][warp + 4 * i];
#pragma unroll
                for (int e = 0; e < E; ++e) acc[h][e] += a * (owns_pos && p0 + warp + 4 * i == pos ? vn[lane * E + e] : vpre[i][e]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < KVMUL; ++h)
#pragma unroll
        for (int e = 0; e < E; ++e) red[warp][h][lane * E + e] = acc[h][e];
    __syncthreads();
    if (n_active == 1) {
        // one split holds the whole context: its partial is the answer, no merge and no hand-over through memory
        for (int i = tid; i < KVMUL * HD; i += 128) {
            const int h = i / HD, d = i % HD;
            p.out[(size_t)(kvh * KVMUL + h) * HD + d] = (red[0][h][d] + red[1][h][d] + red[2][h][d] + red[3][h][d]) * (1.0f / ml[h][1]);
        }
        return;
    }
    float *mine = p.partial + ((size_t)(kvh * p.n_split + sp) * KVMUL) * (HD + 2);
    for (int i = tid; i < KVMUL * HD; i += 128) {
        const int h = i / HD, d = i % HD;
        mine[(size_t)h * (HD + 2) + d] = red[0][h][d] + red[1][h][d] + red[2][h][d] + red[3][h][d];
    }
    if (tid < KVMUL) {
        mine[(size_t)tid * (HD + 2) + HD] = ml[tid][0];
        mine[(size_t)tid * (HD + 2) + HD + 1] = ml[tid][1];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned t = atomicAdd(&p.counters[kvh], 1u);
        is_last = t == (unsigned)(n_active - 1);
        if (is_last) p.counters[kvh] = 0u; // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // merge the splits: w[h][s] = exp(m_s - M) * (1 / L), L = sum_s l_s exp(m_s - M).  The (m, l) pairs of all
    // splits come in with one 8-byte load each (all independent), one warp per head reduces them, then one
    // pass over the partial outputs.
    const float *base = p.partial + ((size_t)kvh * p.n_split * KVMUL) * (HD + 2);
    __shared__ float wgt[KVMUL][ATT_MAX_CTX / ATT_CHUNK], lsum[KVMUL][ATT_MAX_CTX / ATT_CHUNK];
    for (int i = tid; i < KVMUL * n_active; i += 128) {
        const int h = i / n_active, s2 = i % n_active;
        const float2 v = __ldcg((const float2 *)(base + ((size_t)s2 * KVMUL + h) * (HD + 2) + HD));
        wgt[h][s2] = v.x, lsum[h][s2] = v.y;
    }
    __syncthreads();
    for (int h = warp; h < KVMUL; h += 4) {
        float M = -INFINITY, L = 0.f;
        for (int s2 = lane; s2 < n_active; s2 += 32) M = fmaxf(M, wgt[h][s2]);
        M = warp_max(M);
        for (int s2 = lane; s2 < n_active; s2 += 32) {
            const float w = expf(wgt[h][s2] - M);
            L += lsum[h][s2] * w;
            wgt[h][s2] = w;
        }
        L = warp_sum(L);
        const float invL = 1.0f / L;
        for (int s2 = lane; s2 < n_active; s2 += 32) wgt[h][s2] *= invL;
    }
    __syncthreads();
    // every thread's outputs together, SU splits per batch: OPT * SU independent loads in flight instead of 8
    constexpr int NOUT = KVMUL * HD, OPT = (NOUT + 127) / 128, SU = OPT <= 2 ? 40 : 8;
    float o[OPT];
#pragma unroll
    for (int k = 0; k < OPT; ++k) o[k] = 0.f;
    for (int s0 = 0; s0 < n_active; s0 += SU) {
        float v[OPT][SU];
#pragma unroll
        for (int u = 0; u < SU; ++u) {
            const int s2 = min(s0 + u, n_active - 1);
#pragma unroll
            for (int k = 0; k < OPT; ++k) {
                const int i = min(tid + 128 * k, NOUT - 1), h = i / HD, d = i % HD;
                v[k][u] = __ldcg(base + ((size_t)s2 * KVMUL + h) * (HD + 2) + d);
            }
        }
#pragma unroll
        for (int u = 0; u < SU; ++u)
            if (s0 + u < n_active) {
#pragma unroll
                for (int k = 0; k < OPT; ++k) o[k] += v[k][u] * wgt[min(tid + 128 * k, NOUT - 1) / HD][s0 + u];
            }
    }
#pragma unroll
    for (int k = 0; k < OPT; ++k) {
        const int i = tid + 128 * k, h = i / HD, d = i % HD;
        if (i < NOUT) p.out[(size_t)(kvh * KVMUL + h) * HD + d] = o[k];
    }
}

// ---------------------------------------------------------------------------
// Small kernels
// ---------------------------------------------------------------------------
// Greedy sampling (crates/ullm-model/src/sample.rs:125-133: first index wins ties)
// and the bookkeeping that lets the next graph replay run without the host.
constexpr int ARGMAX_CTAS = 32;
__global__ void __launch_bounds__(256) argmax_step_kernel(const float *__restrict__ logits, int n, uint32_t *token, int *pos, int *step,
                                                         uint32_t *tokens_out, int max_steps, float2 *part, unsigned *counter) {
    __shared__ float bvs[8];
    __shared__ int bis[8];
    __shared__ bool is_last;
    pdl_wait_prior();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
    // each CTA scans a contiguous slice; the candidates meet in memory and the last CTA to arrive decides
    const int per = (n + gridDim.x - 1) / gridDim.x, i0 = blockIdx.x * per, i1 = min(n, i0 + per);
    for (int i = i0 + tid; i < i1; i += 256) {
        const float v = __ldcg(logits + i);
        if (better(v, i, bv, bi)) bv = v, bi = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) bvs[warp] = bv, bis[warp] = bi;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; ++w)
            if (better(bvs[w], bis[w], bv, bi)) bv = bvs[w], bi = bis[w];
        part[blockIdx.x] = make_float2(bv, __int_as_float(bi));
        __threadfence();
        const unsigned t = atomicAdd(counter, 1u);
        is_last = t == gridDim.x - 1;
        if (is_last) *counter = 0u; // ready for the next launch
    }
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    bv = -INFINITY, bi = 0x7fffffff;
    for (int c = lane; c < (int)gridDim.x; c += 32) {
        const float2 v = __ldcg(part + c);
        if (better(v.x, __float_as_int(v.y), bv, bi)) bv = v.x, bi = __float_as_int(v.y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0; // all NaN / -inf: the reference keeps index 0
        *token = (uint32_t)bi;
        const int s = *step;
        if (s < max_steps) tokens_out[s] = (uint32_t)bi;
        *step = s + 1;
        *pos = *pos + 1;
    }
}

__global__ void kv_fill_kernel(const float *__restrict__ src, void *dst, size_t n, int f16) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (f16) ((__half *)dst)[i] = __float2half_rn(src[i]);
    else ((float *)dst)[i] = src[i];
}

// ---------------------------------------------------------------------------
// Engine
// ---------------------------------------------------------------------------
static int fmt_of_dtype(int dtype) { return dtype == 12 ? FMT_Q4K : (dtype == 14 ? FMT_Q6K : (dtype == 1000 ? FMT_MLX4 : -1)); }

// x * (1 / sqrt(mean(x^2) + eps)) * w (math.rs:82-86) and a + b for one vector: the steps around a
// mixture-of-experts FFN, whose kernels take the normalised vector from memory, and the unfused
// fallback of Forward::mv
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps, int n,
                                                         float *__restrict__ y) {
    __shared__ float red[8];
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) ss += x[i] * x[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) y[i] = x[i] * inv * w[i];
}
__global__ void add_vec_kernel(const float *__restrict__ a, const float *__restrict__ b, int n, float *__restrict__ y) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = a[i] + b[i];
}
static size_t qbytes(int fmt, size_t out, size_t cols) {
    return out * (cols / QK_K) * (fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
}

template <int HD, int KVMUL> static cudaError_t launch_attn_t(const AttnParams &p, int n_kv_head, bool f16, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_kv_head, p.n_split), cfg.blockDim = dim3(128), cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl ? 1 : 0;
    // Same shared-memory carve-out as the streamed matvecs around it: a kernel that prefers a
    // different L1 / shared split makes the SMs drain and reconfigure between launches.
    static bool carved = false;
    if (!carved) {
        cudaFuncSetAttribute(attn_decode_kernel<HD, KVMUL, __half>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(attn_decode_kernel<HD, KVMUL, float>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carved = true;
    }
    if (f16) return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, KVMUL, __half>, p);
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, KVMUL, float>, p);
}
static cudaError_t launch_attn(const AttnParams &p, int hd, int kvmul, int n_kv_head, bool f16, cudaStream_t st, bool pdl) {
#define ULLM_ATT(H, K) \
    if (hd == H && kvmul == K) return launch_attn_t<H, K>(p, n_kv_head, f16, st, pdl);
    ULLM_ATT(64, 1) ULLM_ATT(64, 2) ULLM_ATT(64, 4) ULLM_ATT(64, 8)
    ULLM_ATT(128, 1) ULLM_ATT(128, 2) ULLM_ATT(128, 4) ULLM_ATT(128, 8)
#undef ULLM_ATT
    return cudaErrorNotSupported;
}

const char *Forward::check_params(const ForwardParams &p) {
    if (!p.n_embd || !p.n_layer || !p.n_head || !p.n_kv_head || !p.head_dim || (!p.n_ff && !p.n_experts) || !p.n_ctx || !p.vocab)
        return "zero hyperparameter";
    if (p.n_experts && (!p.n_experts_used || !p.moe_inter || p.n_experts_used > p.n_experts)) return "mixture-of-experts sizes";
    if (p.n_head % p.n_kv_head) return "n_head is not a multiple of n_kv_head";
    if (p.n_ctx > 8192) return "context longer than 8192 positions"; // the reference caps it there too (lib.rs:236)
    const size_t kvmul = p.n_head / p.n_kv_head;
    if (p.head_dim != 64 && p.head_dim != 128) return "head_dim must be 64 or 128";
    if (kvmul != 1 && kvmul != 2 && kvmul != 4 && kvmul != 8) return "n_head / n_kv_head must be 1, 2, 4 or 8";
    if (p.n_embd % QK_K || p.n_ff % QK_K || (p.n_head * p.head_dim) % QK_K) return "dimensions must be multiples of 256";
    return nullptr;
}

Forward::~Forward() {
    cudaSetDevice(device);
    if (graph_exec[0]) cudaGraphExecDestroy(graph_exec[0]);
    if (graph_exec[1]) cudaGraphExecDestroy(graph_exec[1]);
    for (void *q : owned)
        if (q) cudaFree(q);
    if (h_pin) cudaFreeHost(h_pin);
    if (h_x) cudaFreeHost(h_x);
    if (h_logits) cudaFreeHost(h_logits);
    if (h_status) cudaFreeHost((void *)h_status);
    if (stream) cudaStreamDestroy(stream);
}

cudaError_t Forward::dev_alloc(void **out, size_t bytes) {
    cudaError_t e = cudaMalloc(out, bytes ? bytes : 16);
    if (e == cudaSuccess) owned.push_back(*out);
    return e;
}

cudaError_t Forward::upload(const void *host, size_t bytes, void **out) {
    cudaError_t e = dev_alloc(out, bytes);
    if (e != cudaSuccess) return e;
    return cudaMemcpyAsync(*out, host, bytes, cudaMemcpyHostToDevice, stream);
}

// Makes `bytes` (rows of `fmt`) resident; Q6_K rows are prepared on the device
// (prepare.cu) when their length allows it.
cudaError_t Forward::upload_rows(const void *bytes, int fmt, size_t out_dim, size_t cols, Mat *out) {
    const size_t n = qbytes(fmt, out_dim, cols);
    out->fmt = fmt, out->out = out_dim, out->cols = cols;
    cudaError_t e = dev_alloc(&out->w, n);
    if (e != cudaSuccess) return e;
    if (fmt == FMT_Q6K && q6k_can_prepare(cols)) {
        void *tmp = nullptr;
        if ((e = cudaMalloc(&tmp, n)) != cudaSuccess) return e;
        e = cudaMemcpyAsync(tmp, bytes, n, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = launch_q6k_prepare(tmp, out->w, out_dim, cols, false, stream);
        cudaError_t e2 = cudaStreamSynchronize(stream);
        cudaFree(tmp);
        out->fmt = FMT_Q6KR;
        return e != cudaSuccess ? e : e2;
    }
    e = cudaMemcpyAsync(out->w, bytes, n, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream); // the caller's bytes may be a temporary
    return e;
}

// Two matrices of the same type stacked (`interleave` = false: rows of a then rows
// of b) or row-interleaved (a0 b0 a1 b1 ...) into one resident matrix.
cudaError_t Forward::upload_pair(const HostWeight &a, const HostWeight &b, bool interleave, Mat *out) {
    const int fmt = fmt_of_dtype(a.dtype);
    const size_t rb = (a.cols / QK_K) * (fmt == FMT_Q4K ? Q4K_BYTES : Q6K_BYTES);
    std::vector<uint8_t> tmp((a.out + b.out) * rb);
    if (!interleave) {
        memcpy(tmp.data(), a.bytes, a.out * rb);
        memcpy(tmp.data() + a.out * rb, b.bytes, b.out * rb);
    } else {
        for (size_t r = 0; r < a.out; ++r) {
            memcpy(tmp.data() + (2 * r) * rb, (const uint8_t *)a.bytes + r * rb, rb);
            memcpy(tmp.data() + (2 * r + 1) * rb, (const uint8_t *)b.bytes + r * rb, rb);
        }
    }
    return upload_rows(tmp.data(), fmt, a.out + b.out, a.cols, out);
}

cudaError_t Forward::upload_one(const HostWeight &a, Mat *out) {
    const int fmt = fmt_of_dtype(a.dtype);
    if (fmt != FMT_MLX4) return upload_rows(a.bytes, fmt, a.out, a.cols, out);
    // MLX 4-bit: packed words as they are, tables in the element type given (f32, or the bf16 bits of the file)
    out->fmt = fmt, out->out = a.out, out->cols = a.cols, out->group = a.group, out->tbl_bytes = mlx_table_bytes;
    const size_t tb = a.out * (a.cols / a.group) * (size_t)mlx_table_bytes;
    cudaError_t e = upload(a.bytes, a.out * a.cols / 2, &out->w);
    if (e == cudaSuccess) e = upload(a.scales, tb, &out->scales);
    if (e == cudaSuccess) e = upload(a.biases, tb, &out->biases);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return e;
}

// MLX matrices with the same row length and group size stacked row-wise: words after words, tables after tables.
cudaError_t Forward::upload_mlx_stack(const HostWeight *const *ws, int n, Mat *out) {
    const size_t cols = ws[0]->cols, group = ws[0]->group, tb = (size_t)mlx_table_bytes;
    size_t rows = 0;
    for (int i = 0; i < n; ++i) rows += ws[i]->out;
    std::vector<uint8_t> w(rows * cols / 2), sc(rows * (cols / group) * tb), bi(sc.size());
    size_t r = 0;
    for (int i = 0; i < n; ++i) {
        memcpy(w.data() + r * cols / 2, ws[i]->bytes, ws[i]->out * cols / 2);
        memcpy(sc.data() + r * (cols / group) * tb, ws[i]->scales, ws[i]->out * (cols / group) * tb);
        memcpy(bi.data() + r * (cols / group) * tb, ws[i]->biases, ws[i]->out * (cols / group) * tb);
        r += ws[i]->out;
    }
    HostWeight h = *ws[0];
    h.bytes = w.data(), h.scales = sc.data(), h.biases = bi.data(), h.out = rows;
    return upload_one(h, out); // synchronises: the vectors may go
}

// Stacked experts of one layer: nine arrays made resident, the description re-pointed at them.
cudaError_t Forward::upload_experts(const MoeExperts &h, MoeExperts *out) {
    *out = h;
    const size_t wb = h.n_experts * h.inter * h.hidden / 2;
    const size_t tg = h.n_experts * h.inter * (h.hidden / h.group) * (size_t)h.table_bytes;
    const size_t td = h.n_experts * h.hidden * (h.inter / h.group) * (size_t)h.table_bytes;
    const void *src[9] = {h.gate_w, h.gate_s, h.gate_b, h.up_w, h.up_s, h.up_b, h.down_w, h.down_s, h.down_b};
    const void **dst[9] = {&out->gate_w, &out->gate_s, &out->gate_b, &out->up_w, &out->up_s, &out->up_b, &out->down_w, &out->down_s, &out->down_b};
    const size_t len[9] = {wb, tg, tg, wb, tg, tg, wb, td, td};
    for (int i = 0; i < 9; ++i) {
        void *d = nullptr;
        cudaError_t e = upload(src[i], len[i], &d);
        if (e != cudaSuccess) return e;
        *dst[i] = d;
    }
    return cudaStreamSynchronize(stream);
}

cudaError_t Forward::init(const DeviceInfo &devinfo, int device_, const ForwardParams &params, const HostModel &m) {
    dev = devinfo, device = device_, P = params, mlx_table_bytes = m.mlx_table_bytes;
    if (const char *v = getenv("ULLM_DECODE_CHAIN")) use_chain = atoi(v) != 0; // comparison knob
    cudaError_t e;
#define TRY(x) \
    if ((e = (x)) != cudaSuccess) return e;
    TRY(cudaSetDevice(device));
    TRY(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    const size_t hd = P.head_dim, qd = P.n_head * hd, kvd = P.n_kv_head * hd;
    layers.resize(P.n_layer);
    for (size_t l = 0; l < P.n_layer; ++l) {
        const HostLayer &h = m.layers[l];
        Layer &L = layers[l];
        TRY(upload(h.attn_norm, P.n_embd * 4, (void **)&L.attn_norm));
        TRY(upload(h.ffn_norm, P.n_embd * 4, (void **)&L.ffn_norm));
        {
            const size_t qd_ = P.n_head * P.head_dim, kvd_ = P.n_kv_head * P.head_dim;
            if (h.q_bias) TRY(upload(h.q_bias, qd_ * 4, (void **)&L.q_bias));
            if (h.k_bias) TRY(upload(h.k_bias, kvd_ * 4, (void **)&L.k_bias));
            if (h.v_bias) TRY(upload(h.v_bias, kvd_ * 4, (void **)&L.v_bias));
            if (h.q_norm) TRY(upload(h.q_norm, P.head_dim * 4, (void **)&L.q_norm));
            if (h.k_norm) TRY(upload(h.k_norm, P.head_dim * 4, (void **)&L.k_norm));
        }
        const bool mlx = fmt_of_dtype(h.wq.dtype) == FMT_MLX4; // no stacked q|k for MLX matrices (tables would need stacking too)
        L.qk_fused = h.wq.dtype == h.wk.dtype && !mlx;
        L.qkv_fused = mlx && fmt_of_dtype(h.wk.dtype) == FMT_MLX4 && fmt_of_dtype(h.wv.dtype) == FMT_MLX4 && h.wq.group == h.wk.group &&
                      h.wq.group == h.wv.group;
        if (L.qkv_fused) {
            const HostWeight *ws[3] = {&h.wq, &h.wk, &h.wv};
            TRY(upload_mlx_stack(ws, 3, &L.wqk));
        } else if (L.qk_fused) {
            TRY(upload_pair(h.wq, h.wk, false, &L.wqk));
        } else {
            TRY(upload_one(h.wq, &L.wq));
            TRY(upload_one(h.wk, &L.wk));
        }
        if (!L.qkv_fused) TRY(upload_one(h.wv, &L.wv));
        TRY(upload_one(h.wo, &L.wo));
        if (h.experts) {
            L.moe = true;
            TRY(upload_one(h.moe_gate, &L.moe_gate));
            TRY(upload_experts(*h.experts, &L.experts));
            continue;
        }
        int gfmt = fmt_of_dtype(h.w_gate.dtype);
        if (gfmt == FMT_Q6K && q6k_can_prepare(P.n_embd)) gfmt = FMT_Q6KR;
        L.gu_fused = h.w_gate.dtype == h.w_up.dtype && gfmt != FMT_MLX4 && matvec_is_streamed(dev, gfmt, 2 * P.n_ff, P.n_embd, 0, 4, EPI_SWIGLU);
        if (L.gu_fused) {
            TRY(upload_pair(h.w_gate, h.w_up, true, &L.wgu));
        } else {
            TRY(upload_one(h.w_gate, &L.wg));
            TRY(upload_one(h.w_up, &L.wu));
        }
        TRY(upload_one(h.w_down, &L.wd));
    }
    TRY(upload_one(m.output, &output));
    TRY(upload(m.final_norm, P.n_embd * 4, (void **)&final_norm));

    // RoPE table with the host libm, as the CPU path computes it (math.rs:128-129)
    {
        std::vector<float2> tab(P.n_ctx * (hd / 2));
        for (size_t pos = 0; pos < P.n_ctx; ++pos)
            for (size_t j = 0; j < hd / 2; ++j) {
                const float freq = 1.0f / powf(P.rope_theta, (float)(2 * j) / (float)hd);
                const float ang = (float)pos * freq;
                tab[pos * (hd / 2) + j] = make_float2(cosf(ang), sinf(ang));
            }
        TRY(upload(tab.data(), tab.size() * sizeof(float2), (void **)&rope));
        TRY(cudaStreamSynchronize(stream));
    }
    const size_t kvb = P.kv_f16 ? 2 : 4;
    TRY(dev_alloc(&kcache, P.n_layer * P.n_ctx * kvd * kvb));
    TRY(dev_alloc(&vcache, P.n_layer * P.n_ctx * kvd * kvb));
    TRY(cudaMemsetAsync(kcache, 0, P.n_layer * P.n_ctx * kvd * kvb, stream));
    TRY(cudaMemsetAsync(vcache, 0, P.n_layer * P.n_ctx * kvd * kvb, stream));
    n_split = (int)((P.n_ctx + ATT_CHUNK - 1) / ATT_CHUNK);
    TRY(dev_alloc((void **)&x, P.n_embd * 4));
    TRY(dev_alloc((void **)&xb, P.n_embd * 4));
    TRY(dev_alloc((void **)&qk, (qd + 2 * kvd) * 4)); // q | k (| v when the three projections are one stacked matrix)
    TRY(dev_alloc((void **)&vbuf, kvd * 4));
    TRY(dev_alloc((void **)&attn, qd * 4));
    TRY(dev_alloc((void **)&hidden, P.n_ff * 4));
    TRY(dev_alloc((void **)&gate, P.n_ff * 4));
    TRY(dev_alloc((void **)&up, P.n_ff * 4));
    TRY(dev_alloc((void **)&tmpn, std::max(std::max(P.n_embd, qd), P.n_ff) * 4));
    TRY(dev_alloc((void **)&tmpo, std::max(P.n_embd, P.n_ff) * 4));
    if (P.n_experts) {
        size_t sb = 0;
        for (const Layer &L : layers)
            if (L.moe) sb = std::max(sb, moe_scratch_bytes(L.experts));
        TRY(dev_alloc((void **)&moe_logits, P.n_experts * 4));
        TRY(dev_alloc((void **)&moe_out, P.n_embd * 4));
        TRY(dev_alloc(&moe_scratch, sb));
    }
    TRY(dev_alloc((void **)&logits, P.vocab * 4));
    TRY(dev_alloc((void **)&partial, P.n_kv_head * n_split * (P.n_head / P.n_kv_head) * (hd + 2) * 4));
    TRY(dev_alloc((void **)&counters, (P.n_kv_head + 1) * 4)); // one per kv head (attention) + one for the argmax
    TRY(cudaMemsetAsync(counters, 0, (P.n_kv_head + 1) * 4, stream));
    TRY(dev_alloc((void **)&argmax_part, ARGMAX_CTAS * sizeof(float2)));
    TRY(dev_alloc((void **)&chain_sync, 256));
    TRY(cudaMemsetAsync(chain_sync, 0, 256, stream));
    TRY(dev_alloc((void **)&state, 64)); // [0] pos, [1] token, [2] step
    TRY(cudaMemsetAsync(state, 0, 64, stream));
    TRY(dev_alloc((void **)&tokens_out, MAX_GREEDY * 4));
    TRY(cudaHostAlloc((void **)&h_pin, 64, cudaHostAllocDefault));
    TRY(cudaHostAlloc((void **)&h_x, P.n_embd * 4, cudaHostAllocDefault));
    TRY(cudaHostAlloc((void **)&h_logits, P.vocab * 4, cudaHostAllocDefault));
    TRY(cudaHostAlloc((void **)&h_status, sizeof(int), cudaHostAllocMapped));
    owned_host = true;
    *h_status = 0;
    TRY(cudaHostGetDevicePointer((void **)&d_status, (void *)h_status, 0));
    TRY(cudaStreamSynchronize(stream));
#undef TRY
    return cudaSuccess;
}

cudaError_t Forward::mv(const Mat &m, const float *in, float *out, const float *norm_w, int epi, const float *res) {
    MatvecOpts o;
    o.pdl = use_pdl, o.norm_w = norm_w, o.eps = P.eps, o.epi = epi, o.res = res;
    MlxTables tb;
    tb.scales = m.scales, tb.biases = m.biases, tb.elem_bytes = m.tbl_bytes, tb.group = m.group;
    cudaError_t e = launch_matvec(dev, m.fmt, m.w, tb, in, out, m.out, m.cols, d_status, stream, o);
    ++launches;
    if (e != cudaErrorNotSupported || epi == EPI_SWIGLU) return e;
    // A shape the streamed kernel does not take has no fused prologue / epilogue: normalise into
    // memory first, add the residual afterwards.
    --launches;
    if (norm_w) {
        rmsnorm_vec_kernel<<<1, 256, 0, stream>>>(in, norm_w, P.eps, (int)m.cols, tmpn);
        in = tmpn, ++launches;
    }
    MatvecOpts plain;
    e = launch_matvec(dev, m.fmt, m.w, tb, in, epi == EPI_RESIDUAL ? tmpo : out, m.out, m.cols, d_status, stream, plain);
    ++launches;
    if (e == cudaSuccess && epi == EPI_RESIDUAL) {
        add_vec_kernel<<<(unsigned)((m.out + 255) / 256), 256, 0, stream>>>(res, tmpo, (int)m.out, out);
        ++launches;
    }
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Enqueues one token step on `stream`.  mode 0: x already holds the embedding,
// logits are left in `logits`.  mode 1 (greedy): embedding lookup of state.token
// first, argmax + bookkeeping last.
cudaError_t Forward::enqueue_step(int mode, const void *embd_table, int embd_dtype) {
    cudaError_t e;
#define TRY(x) \
    if ((e = (x)) != cudaSuccess) return e;
    const size_t hd = P.head_dim, qd = P.n_head * hd, kvd = P.n_kv_head * hd;
    int *pos_ptr = (int *)state;
    uint32_t *tok_ptr = (uint32_t *)state + 1;
    int *step_ptr = (int *)state + 2;
    launches = 0;
    if (mode == 1) {
        if (embd_dtype == 1000) {
            TRY(launch_dequant_row_mlx4(embd_table, embd_mlx.scales, embd_mlx.biases, embd_mlx.elem_bytes, embd_mlx.group, tok_ptr, P.n_embd, x, stream));
        } else {
            TRY(launch_dequant_row(embd_dtype, embd_table, tok_ptr, P.n_embd, x, stream));
        }
        ++launches;
    }
    const size_t kvb = P.kv_f16 ? 2 : 4;
    for (size_t l = 0; l < P.n_layer; ++l) {
        Layer &L = layers[l];
        // q|k and v read the same normed x and share nothing else: one persistent launch for both
        // (matvec_chain.cu) when the formats allow it, else one launch each
        bool chained = false;
        if (L.qk_fused && !L.qkv_fused && use_chain && matvec_chain_supported(L.wqk.fmt, L.wqk.out, L.wqk.cols, EPI_STORE) &&
            matvec_chain_supported(L.wv.fmt, L.wv.out, L.wv.cols, EPI_STORE)) {
            MatvecChainOp ops[2];
            ops[0].fmt = L.wqk.fmt, ops[0].w = L.wqk.w, ops[0].x = x, ops[0].y = qk, ops[0].out_dim = L.wqk.out, ops[0].in_dim = L.wqk.cols;
            ops[1].fmt = L.wv.fmt, ops[1].w = L.wv.w, ops[1].x = x, ops[1].y = vbuf, ops[1].out_dim = L.wv.out, ops[1].in_dim = L.wv.cols;
            ops[0].norm_w = ops[1].norm_w = L.attn_norm, ops[0].eps = ops[1].eps = P.eps;
            e = launch_matvec_chain(dev, 2, ops, chain_sync, d_status, stream, use_pdl);
            if (e == cudaSuccess) chained = true, ++launches;
            else if (e != cudaErrorNotSupported) return e;
            else cudaGetLastError();
        }
        if (L.qkv_fused) {
            TRY(mv(L.wqk, x, qk, L.attn_norm, EPI_STORE, nullptr));
        } else if (!chained) {
            if (L.qk_fused) {
                TRY(mv(L.wqk, x, qk, L.attn_norm, EPI_STORE, nullptr));
            } else {
                TRY(mv(L.wq, x, qk, L.attn_norm, EPI_STORE, nullptr));
                TRY(mv(L.wk, x, qk + qd, L.attn_norm, EPI_STORE, nullptr));
            }
            TRY(mv(L.wv, x, vbuf, L.attn_norm, EPI_STORE, nullptr));
        }
        AttnParams ap;
        ap.q = qk, ap.knew = qk + qd, ap.vnew = L.qkv_fused ? qk + qd + kvd : vbuf;
        ap.kcache = (uint8_t *)kcache + l * P.n_ctx * kvd * kvb;
        ap.vcache = (uint8_t *)vcache + l * P.n_ctx * kvd * kvb;
        ap.rope = rope, ap.pos_ptr = pos_ptr, ap.scale = 1.0f / sqrtf((float)hd);
        ap.partial = partial, ap.counters = counters, ap.out = attn, ap.kv_dim = (int)kvd, ap.n_split = n_split;
        ap.q_bias = L.q_bias, ap.k_bias = L.k_bias, ap.v_bias = L.v_bias, ap.q_norm = L.q_norm, ap.k_norm = L.k_norm;
        ap.eps = P.eps, ap.neox = P.rope_neox;
        TRY(launch_attn(ap, (int)hd, (int)(P.n_head / P.n_kv_head), (int)P.n_kv_head, P.kv_f16 != 0, stream, use_pdl));
        ++launches;
        TRY(mv(L.wo, attn, x, nullptr, EPI_RESIDUAL, x));
        if (L.moe) {
            // forward.rs:484-494: normalised x -> router logits -> top-k -> the selected experts' SwiGLU FFNs,
            // weighted by the softmax over the selected logits -> added to x
            // router and experts both normalise x themselves (fused prologues); shapes outside the streamed kernels
            // go through a normalised copy instead
            TRY(mv(L.moe_gate, x, moe_logits, L.ffn_norm, EPI_STORE, nullptr));
            e = launch_moe_ffn(dev, L.experts, x, moe_logits, 1, P.n_experts_used, x, nullptr, nullptr, moe_scratch, d_status, stream, false,
                               use_pdl, nullptr, x, L.ffn_norm, P.eps);
            if (e == cudaErrorNotSupported) {
                rmsnorm_vec_kernel<<<1, 256, 0, stream>>>(x, L.ffn_norm, P.eps, (int)P.n_embd, xb);
                ++launches;
                e = launch_moe_ffn(dev, L.experts, xb, moe_logits, 1, P.n_experts_used, x, nullptr, nullptr, moe_scratch, d_status, stream,
                                   false, use_pdl, nullptr, x);
            }
            TRY(e);
            launches += 4; // route, gate|up, down, combine (+ residual)
            TRY(cudaGetLastError());
            continue;
        }
        if (L.gu_fused) {
            TRY(mv(L.wgu, x, hidden, L.ffn_norm, EPI_SWIGLU, nullptr));
        } else {
            return cudaErrorNotSupported;
        }
        TRY(mv(L.wd, hidden, x, nullptr, EPI_RESIDUAL, x));
    }
    TRY(mv(output, x, logits, final_norm, EPI_STORE, nullptr));
    if (mode == 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ARGMAX_CTAS), cfg.blockDim = dim3(256), cfg.stream = stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at, cfg.numAttrs = use_pdl ? 1 : 0;
        cudaFuncSetAttribute(argmax_step_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        TRY(cudaLaunchKernelEx(&cfg, argmax_step_kernel, (const float *)logits, (int)P.vocab, tok_ptr, pos_ptr, step_ptr,
                               tokens_out, (int)MAX_GREEDY, (float2 *)argmax_part, counters + P.n_kv_head));
        ++launches;
    }
#undef TRY
    return cudaSuccess;
}

// Captures the step into a graph once per mode and replays it afterwards.
cudaError_t Forward::run_step(int mode, const void *embd_table, int embd_dtype) {
    if (!use_graph) return enqueue_step(mode, embd_table, embd_dtype);
    if (graph_exec[mode] && (mode == 0 || (graph_table == embd_table && graph_dtype == embd_dtype)))
        return cudaGraphLaunch(graph_exec[mode], stream);
    if (graph_exec[mode]) {
        cudaGraphExecDestroy(graph_exec[mode]);
        graph_exec[mode] = nullptr;
    }
    cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return e;
    cudaError_t body = enqueue_step(mode, embd_table, embd_dtype);
    cudaGraph_t g = nullptr;
    e = cudaStreamEndCapture(stream, &g);
    if (body != cudaSuccess) {
        if (g) cudaGraphDestroy(g);
        return body;
    }
    if (e != cudaSuccess) return e;
    e = cudaGraphInstantiate(&graph_exec[mode], g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return e;
    graph_launches = launches;
    if (mode == 1) graph_table = embd_table, graph_dtype = embd_dtype;
    return cudaGraphLaunch(graph_exec[mode], stream);
}

cudaError_t Forward::forward(const float *x_init, size_t pos, float *logits_host) {
    cudaError_t e;
    if ((e = cudaSetDevice(device)) != cudaSuccess) return e;
    ((int *)h_pin)[0] = (int)pos;
    if ((e = cudaMemcpyAsync(state, h_pin, 4, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
    // The caller's vectors are ordinary (pageable) memory as a rule: a direct copy would be staged by the driver in
    // small pieces.  They go through this object's page-locked buffers instead: one DMA each way plus a host memcpy.
    memcpy(h_x, x_init, P.n_embd * 4);
    if ((e = cudaMemcpyAsync(x, h_x, P.n_embd * 4, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
    if ((e = run_step(0, nullptr, 0)) != cudaSuccess) return e;
    if ((e = cudaMemcpyAsync(h_logits, logits, P.vocab * 4, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;
    memcpy(logits_host, h_logits, P.vocab * 4);
    return cudaSuccess;
}

cudaError_t Forward::greedy(const void *embd_table, int embd_dtype, uint32_t first_token, size_t pos, size_t n,
                            uint32_t *tokens_host) {
    cudaError_t e;
    if ((e = cudaSetDevice(device)) != cudaSuccess) return e;
    size_t done = 0;
    uint32_t tok = first_token;
    while (done < n) {
        const size_t chunk = n - done < MAX_GREEDY ? n - done : MAX_GREEDY;
        ((int *)h_pin)[0] = (int)(pos + done), ((uint32_t *)h_pin)[1] = tok, ((int *)h_pin)[2] = 0;
        if ((e = cudaMemcpyAsync(state, h_pin, 12, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
        for (size_t i = 0; i < chunk; ++i)
            if ((e = run_step(1, embd_table, embd_dtype)) != cudaSuccess) return e;
        if ((e = cudaMemcpyAsync(tokens_host + done, tokens_out, chunk * 4, cudaMemcpyDeviceToHost, stream)) != cudaSuccess)
            return e;
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;
        tok = tokens_host[done + chunk - 1];
        done += chunk;
    }
    return cudaSuccess;
}

cudaError_t Forward::set_kv(size_t pos0, size_t n, const float *k, const float *v) {
    cudaError_t e;
    if ((e = cudaSetDevice(device)) != cudaSuccess) return e;
    const size_t kvd = P.n_kv_head * P.head_dim, kvb = P.kv_f16 ? 2 : 4;
    float *tmp = nullptr;
    if ((e = cudaMalloc((void **)&tmp, n * kvd * 4)) != cudaSuccess) return e;
    for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
        const float *src = which ? v : k;
        uint8_t *cache = (uint8_t *)(which ? vcache : kcache);
        for (size_t l = 0; l < P.n_layer && e == cudaSuccess; ++l) {
            e = cudaMemcpyAsync(tmp, src + l * n * kvd, n * kvd * 4, cudaMemcpyHostToDevice, stream);
            if (e != cudaSuccess) break;
            const size_t cnt = n * kvd;
            kv_fill_kernel<<<(unsigned)((cnt + 255) / 256), 256, 0, stream>>>(tmp, cache + (l * P.n_ctx + pos0) * kvd * kvb, cnt,
                                                                             P.kv_f16);
            e = cudaGetLastError();
        }
    }
    cudaError_t e2 = cudaStreamSynchronize(stream);
    cudaFree(tmp);
    return e != cudaSuccess ? e : e2;
}

// ---------------------------------------------------------------------------
// forward_debug: layer 0 one op at a time (crates/ullm-metal/src/forward.rs:530-635)
// ---------------------------------------------------------------------------
// Non-finite counts and the largest finite magnitude of n values `stride` apart (one CTA).
__global__ void __launch_bounds__(256) debug_stat_kernel(const float *__restrict__ v, size_t n, size_t stride, DebugStat *out) {
    __shared__ unsigned long long s_nan[8], s_inf[8];
    __shared__ float s_mx[8];
    unsigned long long nan = 0, inf = 0;
    float mx = 0.f;
    for (size_t i = threadIdx.x; i < n; i += 256) {
        const float x = v[i * stride];
        if (isnan(x)) ++nan;
        else if (isinf(x)) ++inf;
        else mx = fmaxf(mx, fabsf(x));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        nan += __shfl_xor_sync(0xffffffffu, nan, o);
        inf += __shfl_xor_sync(0xffffffffu, inf, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) s_nan[threadIdx.x >> 5] = nan, s_inf[threadIdx.x >> 5] = inf, s_mx[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) nan += s_nan[i], inf += s_inf[i], mx = fmaxf(mx, s_mx[i]);
        out->nan = nan, out->inf = inf, out->maxabs = mx;
    }
}
// Per-head RMSNorm (math.rs:82-86) and RoPE (math.rs:116-162) of `n_heads` heads of `hd` values, unfused: the
// normalised heads go to `normed` (when norm_w is given), the rotated ones to `roped`.  One warp per head.
__global__ void debug_heads_kernel(const float *__restrict__ src, const float *__restrict__ norm_w, float eps, const float2 *__restrict__ rp,
                                   int neox, int hd, float *__restrict__ normed, float *__restrict__ roped) {
    const int h = blockIdx.x, lane = threadIdx.x;
    const float *s = src + (size_t)h * hd;
    float *nd = normed + (size_t)h * hd, *rd = roped + (size_t)h * hd;
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) ss += s[d] * s[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) nd[d] = norm_w ? s[d] * inv * norm_w[d] : s[d];
    __syncwarp();
    for (int j = lane; j < hd / 2; j += 32) {
        const int ia = neox ? j : 2 * j, ib = neox ? j + hd / 2 : 2 * j + 1;
        const float a = nd[ia], b = nd[ib];
        const float2 cs = rp[j];
        rd[ia] = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
        rd[ib] = __fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
    }
}
// scores[h][t] = scale * q[h] . K[t][h / kv_mul] for t <= pos, keys read from the cache.  One warp per (h, t).
template <typename KV_T>
__global__ void debug_scores_kernel(const float *__restrict__ q, const KV_T *__restrict__ kcache, int hd, int kv_dim, int kv_mul, int seqlen,
                                    float scale, float *__restrict__ scores) {
    const int h = blockIdx.y, t = blockIdx.x, lane = threadIdx.x;
    const KV_T *k = kcache + (size_t)t * kv_dim + (size_t)(h / kv_mul) * hd;
    float acc = 0.f;
    for (int d = lane; d < hd; d += 32) acc += q[(size_t)h * hd + d] * kv_f(k[d]);
    acc = warp_sum(acc);
    if (lane == 0) scores[(size_t)h * seqlen + t] = acc * scale;
}
__global__ void debug_glu_kernel(const float *__restrict__ gu, int n_ff, float *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_ff) {
        const float g = gu[2 * i], u = gu[2 * i + 1];
        out[i] = g / (1.0f + expf(-g)) * u; // silu(g) * u (math.rs:103-105)
    }
}

cudaError_t Forward::debug_layer0(const float *x_init, size_t pos, DebugStat *out, size_t cap, size_t *n_out) {
    cudaError_t e;
#define TRY(x) \
    if ((e = (x)) != cudaSuccess) return e;
    TRY(cudaSetDevice(device));
    const Layer &L = layers[0];
    if (L.moe || !L.gu_fused) return cudaErrorNotSupported;
    const size_t hd = P.head_dim, qd = P.n_head * hd, kvd = P.n_kv_head * hd, ne = P.n_embd, nf = P.n_ff, seqlen = pos + 1;
    // scratch: normed x | q k v projections | normed heads | rotated heads | scores | wo out | gate,up | glu | down | stats
    const size_t proj = qd + 2 * kvd;
    const size_t floats = ne + proj + proj + proj + P.n_head * P.n_ctx + ne + 2 * nf + nf + ne;
    if (!dbg) TRY(dev_alloc((void **)&dbg, floats * 4 + 32 * sizeof(DebugStat)));
    float *xn = dbg, *pr = xn + ne, *hn = pr + proj, *hr = hn + proj, *sc = hr + proj, *wo_out = sc + P.n_head * P.n_ctx, *gu = wo_out + ne,
          *glu = gu + 2 * nf, *down = glu + nf;
    DebugStat *d_stats = (DebugStat *)(down + ne);
    std::vector<DebugStat> host;
    auto stat = [&](const char *label, const float *v, size_t n, size_t stride) -> cudaError_t {
        if (host.size() >= cap || host.size() >= 32) return cudaErrorInvalidValue;
        DebugStat s{};
        snprintf(s.label, sizeof s.label, "%s", label);
        debug_stat_kernel<<<1, 256, 0, stream>>>(v, n, stride, d_stats + host.size());
        host.push_back(s);
        return cudaGetLastError();
    };
    auto plain = [&](const Mat &m, const float *in, float *o) -> cudaError_t {
        MlxTables tb;
        tb.scales = m.scales, tb.biases = m.biases, tb.elem_bytes = m.tbl_bytes, tb.group = m.group;
        return launch_matvec(dev, m.fmt, m.w, tb, in, o, m.out, m.cols, d_status, stream, MatvecOpts());
    };
    ((int *)h_pin)[0] = (int)pos;
    TRY(cudaMemcpyAsync(state, h_pin, 4, cudaMemcpyHostToDevice, stream));
    memcpy(h_x, x_init, ne * 4);
    TRY(cudaMemcpyAsync(x, h_x, ne * 4, cudaMemcpyHostToDevice, stream));
    TRY(stat("x_init", x, ne, 1));
    rmsnorm_vec_kernel<<<1, 256, 0, stream>>>(x, L.attn_norm, P.eps, (int)ne, xn);
    TRY(stat("attn_norm", xn, ne, 1));
    // projections, stored q | k | v in `pr` whatever way the engine keeps the matrices
    if (L.qkv_fused) {
        TRY(plain(L.wqk, xn, pr));
    } else {
        if (L.qk_fused) {
            TRY(plain(L.wqk, xn, pr));
        } else {
            TRY(plain(L.wq, xn, pr));
            TRY(plain(L.wk, xn, pr + qd));
        }
        TRY(plain(L.wv, xn, pr + qd + kvd));
    }
    TRY(stat("wq", pr, qd, 1));
    TRY(stat("wk", pr + qd, kvd, 1));
    const float2 *rp = rope + pos * (hd / 2);
    debug_heads_kernel<<<(unsigned)P.n_head, 32, 0, stream>>>(pr, L.q_norm, P.eps, rp, P.rope_neox, (int)hd, hn, hr);
    debug_heads_kernel<<<(unsigned)P.n_kv_head, 32, 0, stream>>>(pr + qd, L.k_norm, P.eps, rp, P.rope_neox, (int)hd, hn + qd, hr + qd);
    if (L.q_norm) TRY(stat("q_norm", hn, qd, 1));
    if (L.k_norm) TRY(stat("k_norm", hn + qd, kvd, 1));
    TRY(stat("rope_q", hr, qd, 1));
    TRY(stat("rope_k", hr + qd, kvd, 1));
    // the engine's own attention kernel (it rotates q / k itself and writes K / V of `pos` into the cache); as in the
    // reference's debug walk the projection biases are left out
    AttnParams ap;
    ap.q = pr, ap.knew = pr + qd, ap.vnew = pr + qd + kvd;
    ap.kcache = kcache, ap.vcache = vcache;
    ap.rope = rope, ap.pos_ptr = (int *)state, ap.scale = 1.0f / sqrtf((float)hd);
    ap.partial = partial, ap.counters = counters, ap.out = attn, ap.kv_dim = (int)kvd, ap.n_split = n_split;
    ap.q_bias = ap.k_bias = ap.v_bias = nullptr, ap.q_norm = L.q_norm, ap.k_norm = L.k_norm;
    ap.eps = P.eps, ap.neox = P.rope_neox;
    TRY(launch_attn(ap, (int)hd, (int)(P.n_head / P.n_kv_head), (int)P.n_kv_head, P.kv_f16 != 0, stream, false));
    const dim3 sg((unsigned)seqlen, (unsigned)P.n_head);
    if (P.kv_f16)
        debug_scores_kernel<__half><<<sg, 32, 0, stream>>>(hr, (const __half *)kcache, (int)hd, (int)kvd, (int)(P.n_head / P.n_kv_head), (int)seqlen,
                                                          ap.scale, sc);
    else
        debug_scores_kernel<float><<<sg, 32, 0, stream>>>(hr, (const float *)kcache, (int)hd, (int)kvd, (int)(P.n_head / P.n_kv_head), (int)seqlen,
                                                         ap.scale, sc);
    TRY(stat("attn_scores", sc, P.n_head * seqlen, 1));
    TRY(stat("attn_out", attn, qd, 1));
    TRY(plain(L.wo, attn, wo_out));
    TRY(stat("wo", wo_out, ne, 1));
    rmsnorm_vec_kernel<<<1, 256, 0, stream>>>(x, L.ffn_norm, P.eps, (int)ne, xn); // x is still x_init, as in the reference's walk
    TRY(stat("ffn_norm", xn, ne, 1));
    TRY(plain(L.wgu, xn, gu)); // rows interleaved (gate_j, up_j)
    TRY(stat("gate", gu, nf, 2));
    TRY(stat("up", gu + 1, nf, 2));
    debug_glu_kernel<<<(unsigned)((nf + 255) / 256), 256, 0, stream>>>(gu, (int)nf, glu);
    TRY(stat("glu", glu, nf, 1));
    TRY(plain(L.wd, glu, down));
    TRY(stat("w_down", down, ne, 1));
    std::vector<DebugStat> got(host.size());
    TRY(cudaMemcpyAsync(got.data(), d_stats, host.size() * sizeof(DebugStat), cudaMemcpyDeviceToHost, stream));
    TRY(cudaStreamSynchronize(stream));
    for (size_t i = 0; i < host.size(); ++i) {
        out[i] = got[i];
        memcpy(out[i].label, host[i].label, sizeof host[i].label);
    }
    *n_out = host.size();
#undef TRY
    return cudaSuccess;
}

} // namespace ullm
