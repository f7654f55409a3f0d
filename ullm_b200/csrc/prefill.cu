// Batched prefill of the resident decode engine: all prompt tokens through every layer in one
// pass (GpuForward::forward_batch, crates/ullm-metal/src/forward.rs:757-909; the CPU meaning is
// forward_llama run for positions 0..s-1, crates/ullm-model/src/lib.rs:807-969).
//
// Per layer: rmsnorm of every token -> [q|k] and v projections as tensor-core GEMMs on the
// quantized weights (gemm.cu) -> RoPE of q and k, K/V written to the cache -> causal
// attention of the s new tokens over the cache -> W_o GEMM + residual -> rmsnorm ->
// [gate|up] GEMM with silu(g)*u in its epilogue -> W_down GEMM + residual (epilogue).  Only the last token goes through
// the final norm and the output projection (a matvec).  Prompts longer than PREFILL_CHUNK
// tokens are processed in chunks; the attention reads earlier chunks from the cache.
#include "decode.h"

#include <cstring>

#include <cuda_fp16.h>

#include <algorithm>
#include <utility>

namespace ullm {

constexpr size_t PREFILL_CHUNK = 512;

// y[t, :] = x[t, :] * (1 / sqrt(mean(x[t, :]^2) + eps)) * w   (math.rs:82-86), one CTA per token
__global__ void __launch_bounds__(256) rmsnorm_batch_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps,
                                                           int n, float *__restrict__ y) {
    __shared__ float red[8];
    const float *xr = x + (size_t)blockIdx.x * n;
    float *yr = y + (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) yr[i] = xr[i] * inv * w[i];
}

template <typename T> __device__ __forceinline__ T kv_from(float v);
template <> __device__ __forceinline__ float kv_from<float>(float v) { return v; }
template <> __device__ __forceinline__ __half kv_from<__half>(float v) { return __float2half_rn(v); }
template <typename T> __device__ __forceinline__ float kv_to(T v);
template <> __device__ __forceinline__ float kv_to<float>(float v) { return v; }
template <> __device__ __forceinline__ float kv_to<__half>(__half v) { return __half2float(v); }

// One head: (+ bias) -> (per-head RMSNorm, math.rs:82-86) -> RoPE on interleaved or rotate-half pairs
// (math.rs:116-162, products and sums unfused), in shared memory, by one warp.  Same steps as the
// decode kernel's prologue (decode.cu), so both paths fill the cache with the same values.
template <int HD>
__device__ __forceinline__ void head_prepare_batch(const float *__restrict__ src, const float *__restrict__ bias,
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

struct RopeBatchParams {
    float *qk;            // [s, qd + kvd]: q heads then k heads of every token; q is rewritten in place
    const float *v;       // [s, kvd]
    const float2 *rope;
    void *kc, *vc;        // this layer's cache
    const float *q_bias, *k_bias, *v_bias, *q_norm, *k_norm; // optional
    float eps;
    int pos0, n_head, n_kv_head, neox;
};

// one CTA per token, one warp per head in turn; k and v go to the cache
template <int HD, typename KV_T> __global__ void __launch_bounds__(256) rope_kv_batch_kernel(const RopeBatchParams p) {
    __shared__ float buf[8][HD];
    const int t = blockIdx.x, pos = p.pos0 + t, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qd = p.n_head * HD, kvd = p.n_kv_head * HD;
    float *row = p.qk + (size_t)t * (qd + kvd);
    const float2 *rp = p.rope + (size_t)pos * (HD / 2);
    KV_T *kc = (KV_T *)p.kc, *vc = (KV_T *)p.vc;
    for (int hh = warp; hh < p.n_head + p.n_kv_head; hh += 8) {
        const bool is_q = hh < p.n_head;
        const int hk = hh - p.n_head;
        const float *bias = is_q ? (p.q_bias ? p.q_bias + (size_t)hh * HD : nullptr) : (p.k_bias ? p.k_bias + (size_t)hk * HD : nullptr);
        head_prepare_batch<HD>(row + (size_t)hh * HD, bias, is_q ? p.q_norm : p.k_norm, p.eps, rp, p.neox, buf[warp], lane);
        for (int d = lane; d < HD; d += 32) {
            if (is_q) row[(size_t)hh * HD + d] = buf[warp][d];
            else kc[(size_t)pos * kvd + (size_t)hk * HD + d] = kv_from<KV_T>(buf[warp][d]);
        }
        __syncwarp();
    }
    for (int i = threadIdx.x; i < kvd; i += 256)
        vc[(size_t)pos * kvd + i] = kv_from<KV_T>(p.v[(size_t)t * kvd + i] + (p.v_bias ? p.v_bias[i] : 0.f));
}

// Eight consecutive cache values of one position -> f32 (one 16- or 32-byte load)
__device__ __forceinline__ void kv_load8(const float *p, float (&o)[8]) {
    const float4 a = *(const float4 *)p, b = *(const float4 *)(p + 4);
    o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
}
__device__ __forceinline__ void kv_load8(const __half *p, float (&o)[8]) {
    const uint4 v = *(const uint4 *)p;
    const __half2 *h = (const __half2 *)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        o[2 * i] = f.x, o[2 * i + 1] = f.y;
    }
}

// Causal attention of the chunk's queries over cache positions 0 .. pos0 + t (lib.rs:916-938: scores
// q.k / sqrt(hd), softmax, weighted sum of v).  grid (n_head, ceil(s / 8)), 8 warps: one query per
// warp; keys in blocks of 32 staged in shared memory for the CTA's 8 queries (vector loads from the
// cache, rows padded so that 128-bit reads one row apart hit distinct banks); lane j scores key j of
// the block, the block's probabilities are then broadcast lane by lane for the P.V sum, where every
// lane owns HD / 32 output dimensions.  Running max / sum as in any streaming softmax.
template <int HD, typename KV_T>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float *__restrict__ qk, const KV_T *__restrict__ kc,
                                                          const KV_T *__restrict__ vc, float *__restrict__ out, int s, int pos0,
                                                          int qd, int kvd, int kvmul, float scale) {
    constexpr int E = HD / 32, KP = HD + 4; // padded K row: 16-byte aligned, 4 banks apart per row
    __shared__ __align__(16) float ks[32][KP];
    __shared__ __align__(16) float vs[32][HD];
    const int h = blockIdx.x, kvh = h / kvmul, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y * 8 + warp;
    const bool valid = t < s;
    const int qpos = pos0 + (valid ? t : s - 1);
    const int last_q = pos0 + min(s - 1, (int)blockIdx.y * 8 + 7); // the CTA's keys end at its last query
    float q[HD];
    {
        const float4 *qp = (const float4 *)(qk + (size_t)(valid ? t : 0) * (qd + kvd) + (size_t)h * HD);
#pragma unroll
        for (int d = 0; d < HD / 4; ++d) {
            const float4 v = qp[d];
            q[4 * d] = v.x * scale, q[4 * d + 1] = v.y * scale, q[4 * d + 2] = v.z * scale, q[4 * d + 3] = v.w * scale;
        }
    }
    float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;
    for (int k0 = 0; k0 <= last_q; k0 += 32) {
        __syncthreads(); // the previous block's tiles are no longer read
        for (int i = threadIdx.x; i < 32 * (HD / 8); i += 256) { // 8 values per thread and matrix
            const int j = i / (HD / 8), d = (i % (HD / 8)) * 8, kp = min(k0 + j, last_q);
            float kk[8], vv[8];
            kv_load8(kc + (size_t)kp * kvd + (size_t)kvh * HD + d, kk);
            kv_load8(vc + (size_t)kp * kvd + (size_t)kvh * HD + d, vv);
            *(float4 *)&ks[j][d] = make_float4(kk[0], kk[1], kk[2], kk[3]);
            *(float4 *)&ks[j][d + 4] = make_float4(kk[4], kk[5], kk[6], kk[7]);
            *(float4 *)&vs[j][d] = make_float4(vv[0], vv[1], vv[2], vv[3]);
            *(float4 *)&vs[j][d + 4] = make_float4(vv[4], vv[5], vv[6], vv[7]);
        }
        __syncthreads();
        if (k0 > qpos) continue; // this query's keys are exhausted (other warps of the CTA still need the tiles)
        float sc = 0.f;
#pragma unroll
        for (int d = 0; d < HD / 4; ++d) {
            const float4 kv = *(const float4 *)&ks[lane][4 * d];
            sc += q[4 * d] * kv.x + q[4 * d + 1] * kv.y + q[4 * d + 2] * kv.z + q[4 * d + 3] * kv.w;
        }
        if (k0 + lane > qpos) sc = -INFINITY;
        const float mb = warp_max(sc), mn = fmaxf(m, mb);
        const float pj = expf(sc - mn), corr = expf(m - mn);
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] *= corr;
        m = mn;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const float pb = __shfl_sync(0xffffffffu, pj, j);
            if constexpr (E == 2) {
                const float2 v2 = *(const float2 *)&vs[j][lane * 2];
                acc[0] += pb * v2.x, acc[1] += pb * v2.y;
            } else {
                const float4 v4 = *(const float4 *)&vs[j][lane * 4];
                acc[0] += pb * v4.x, acc[1] += pb * v4.y, acc[2] += pb * v4.z, acc[3] += pb * v4.w;
            }
        }
    }
    if (valid) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int e = 0; e < E; ++e) out[(size_t)t * qd + (size_t)h * HD + lane * E + e] = acc[e] * inv;
    }
}

bool Forward::batch_supported() const {
    for (const Layer &L : layers) {
        if (!L.qk_fused || !L.gu_fused) return false;
        const size_t qd = P.n_head * P.head_dim, kvd = P.n_kv_head * P.head_dim;
        if (!gemm_tc_supported(L.wqk.fmt, qd + kvd, P.n_embd, 1) || !gemm_tc_supported(L.wv.fmt, kvd, P.n_embd, 1) ||
            !gemm_tc_supported(L.wo.fmt, P.n_embd, qd, 1) || !gemm_tc_supported(L.wgu.fmt, 2 * P.n_ff, P.n_embd, 1) ||
            !gemm_tc_supported(L.wd.fmt, P.n_embd, P.n_ff, 1))
            return false;
    }
    return P.head_dim == 64 || P.head_dim == 128;
}

cudaError_t Forward::forward_batch(const float *embeds_host, size_t s, float *logits_host) {
    cudaError_t e;
#define TRY(x) \
    if ((e = (x)) != cudaSuccess) return e;
    TRY(cudaSetDevice(device));
    if (!batch_supported()) return cudaErrorNotSupported;
    if (s == 0 || s > P.n_ctx) return cudaErrorInvalidValue;
    const size_t hd = P.head_dim, qd = P.n_head * hd, kvd = P.n_kv_head * hd, E = P.n_embd, F = P.n_ff, B = PREFILL_CHUNK;
    const size_t kvb = P.kv_f16 ? 2 : 4;
    if (!bx) { // activation buffers for one chunk, allocated on first use
        size_t scratch = 0;
        for (const auto &d : {std::pair<size_t, size_t>{qd + kvd, E}, {kvd, E}, {E, qd}, {2 * F, E}, {E, F}})
            for (size_t n = 1; n <= B; ++n) // the split-K factor, and with it the partial-sum area, depends on the token count
                scratch = std::max(scratch, gemm_tc_scratch_bytes(d.first, d.second, n, dev.sm_count));
        TRY(dev_alloc((void **)&bx, B * E * 4));
        TRY(dev_alloc((void **)&bxn, B * std::max(E, qd) * 4));
        TRY(dev_alloc((void **)&bqk, B * (qd + kvd) * 4));
        TRY(dev_alloc((void **)&bv, B * kvd * 4));
        TRY(dev_alloc((void **)&bh, B * F * 4));
        TRY(dev_alloc(&bscratch, scratch));
    }
    auto gemm = [&](const Mat &m, const float *in, float *out, size_t n, int epi = EPI_STORE, const float *res = nullptr) {
        ++launches;
        return launch_gemm_tc(m.fmt, m.w, in, out, bscratch, m.out, m.cols, n, dev.sm_count, d_status, stream, epi, res);
    };
    const float scale = 1.0f / sqrtf((float)hd);
    for (size_t c0 = 0; c0 < s; c0 += B) {
        const size_t n = std::min(B, s - c0);
        TRY(cudaMemcpyAsync(bx, embeds_host + c0 * E, n * E * 4, cudaMemcpyHostToDevice, stream));
        for (size_t l = 0; l < P.n_layer; ++l) {
            Layer &L = layers[l];
            uint8_t *kc = (uint8_t *)kcache + l * P.n_ctx * kvd * kvb, *vc = (uint8_t *)vcache + l * P.n_ctx * kvd * kvb;
            rmsnorm_batch_kernel<<<(unsigned)n, 256, 0, stream>>>(bx, L.attn_norm, P.eps, (int)E, bxn);
            TRY(gemm(L.wqk, bxn, bqk, n));
            TRY(gemm(L.wv, bxn, bv, n));
            const dim3 ag((unsigned)P.n_head, (unsigned)((n + 7) / 8));
            const int kvmul = (int)(P.n_head / P.n_kv_head);
            RopeBatchParams rb;
            rb.qk = bqk, rb.v = bv, rb.rope = rope, rb.kc = kc, rb.vc = vc;
            rb.q_bias = L.q_bias, rb.k_bias = L.k_bias, rb.v_bias = L.v_bias, rb.q_norm = L.q_norm, rb.k_norm = L.k_norm;
            rb.eps = P.eps, rb.pos0 = (int)c0, rb.n_head = (int)P.n_head, rb.n_kv_head = (int)P.n_kv_head, rb.neox = P.rope_neox;
            if (P.kv_f16) {
                if (hd == 64) {
                    rope_kv_batch_kernel<64, __half><<<(unsigned)n, 256, 0, stream>>>(rb);
                    attn_prefill_kernel<64, __half><<<ag, 256, 0, stream>>>(bqk, (const __half *)kc, (const __half *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                } else {
                    rope_kv_batch_kernel<128, __half><<<(unsigned)n, 256, 0, stream>>>(rb);
                    attn_prefill_kernel<128, __half><<<ag, 256, 0, stream>>>(bqk, (const __half *)kc, (const __half *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                }
            } else {
                if (hd == 64) {
                    rope_kv_batch_kernel<64, float><<<(unsigned)n, 256, 0, stream>>>(rb);
                    attn_prefill_kernel<64, float><<<ag, 256, 0, stream>>>(bqk, (const float *)kc, (const float *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                } else {
                    rope_kv_batch_kernel<128, float><<<(unsigned)n, 256, 0, stream>>>(rb);
                    attn_prefill_kernel<128, float><<<ag, 256, 0, stream>>>(bqk, (const float *)kc, (const float *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                }
            }
            TRY(cudaGetLastError());
            // the attention output [n, qd] sits in bxn; residual adds and silu(g)*u happen in the GEMM epilogues
            TRY(gemm(L.wo, bxn, bx, n, EPI_RESIDUAL, bx));
            rmsnorm_batch_kernel<<<(unsigned)n, 256, 0, stream>>>(bx, L.ffn_norm, P.eps, (int)E, bxn);
            TRY(gemm(L.wgu, bxn, bh, n, EPI_SWIGLU));
            TRY(gemm(L.wd, bh, bx, n, EPI_RESIDUAL, bx));
            TRY(cudaGetLastError());
        }
        if (c0 + n == s) { // the last token's hidden state -> final norm + output projection
            TRY(cudaMemcpyAsync(x, bx + (n - 1) * E, E * 4, cudaMemcpyDeviceToDevice, stream));
            TRY(mv(output, x, logits, final_norm, EPI_STORE, nullptr));
        }
    }
    TRY(cudaMemcpyAsync(h_logits, logits, P.vocab * 4, cudaMemcpyDeviceToHost, stream)); // page-locked staging, as in forward()
    TRY(cudaStreamSynchronize(stream));
#undef TRY
    memcpy(logits_host, h_logits, P.vocab * 4);
    return cudaSuccess;
}

} // namespace ullm
