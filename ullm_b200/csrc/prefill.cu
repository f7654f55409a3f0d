// Batched prefill of the resident decode engine: all prompt tokens through every layer in one
// pass (GpuForward::forward_batch, crates/ullm-metal/src/forward.rs:757-909; the CPU meaning is
// forward_llama run for positions 0..s-1, crates/ullm-model/src/lib.rs:807-969).
//
// Per layer: rmsnorm of every token -> [q|k] and v projections as tensor-core GEMMs on the
// quantized weights (gemm.cu) -> RoPE of q and k, K/V written to the cache -> causal
// attention of the s new tokens over the cache -> W_o GEMM + residual -> rmsnorm ->
// [gate|up] GEMM -> silu(g)*u -> W_down GEMM + residual.  Only the last token goes through
// the final norm and the output projection (a matvec).  Prompts longer than PREFILL_CHUNK
// tokens are processed in chunks; the attention reads earlier chunks from the cache.
#include "decode.h"

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

// RoPE on interleaved pairs (math.rs:116-136, products and sums unfused) of q (in place) and of
// k, which goes to the cache together with v.  qk: [s, qd + kvd], v: [s, kvd]; one CTA per token.
template <typename KV_T>
__global__ void __launch_bounds__(256) rope_kv_batch_kernel(float *__restrict__ qk, const float *__restrict__ v,
                                                           const float2 *__restrict__ rope, KV_T *__restrict__ kc,
                                                           KV_T *__restrict__ vc, int pos0, int hd, int qd, int kvd) {
    const int t = blockIdx.x, pos = pos0 + t;
    float *row = qk + (size_t)t * (qd + kvd);
    const float2 *rp = rope + (size_t)pos * (hd / 2);
    for (int i = threadIdx.x; i < (qd + kvd) / 2; i += 256) {
        const int e = 2 * i, j = (e % hd) / 2; // heads are hd wide in both the q and the k part (qd is a multiple of hd)
        const float a = row[e], b = row[e + 1];
        const float2 cs = rp[j];
        const float r0 = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)), r1 = __fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
        if (e < qd) {
            row[e] = r0, row[e + 1] = r1;
        } else {
            KV_T *dst = kc + (size_t)pos * kvd + (e - qd);
            dst[0] = kv_from<KV_T>(r0), dst[1] = kv_from<KV_T>(r1);
        }
    }
    for (int i = threadIdx.x; i < kvd; i += 256) vc[(size_t)pos * kvd + i] = kv_from<KV_T>(v[(size_t)t * kvd + i]);
}

// Causal attention of the chunk's queries over cache positions 0 .. pos0 + t (lib.rs:916-938: scores
// q.k / sqrt(hd), softmax, weighted sum of v).  grid (n_head, ceil(s / 8)), 8 warps: one query per
// warp; keys in blocks of 32 staged in shared memory for the CTA's 8 queries; lane j scores key j of
// the block, the block's probabilities are then broadcast lane by lane for the P.V sum, where every
// lane owns HD / 32 output dimensions.  Running max / sum as in any streaming softmax.
template <int HD, typename KV_T>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float *__restrict__ qk, const KV_T *__restrict__ kc,
                                                          const KV_T *__restrict__ vc, float *__restrict__ out, int s, int pos0,
                                                          int qd, int kvd, int kvmul, float scale) {
    constexpr int E = HD / 32;
    __shared__ float ks[32][HD + 1];
    __shared__ float vs[32][HD];
    const int h = blockIdx.x, kvh = h / kvmul, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y * 8 + warp;
    const bool valid = t < s;
    const int qpos = pos0 + (valid ? t : s - 1);
    const int last_q = pos0 + min(s - 1, (int)blockIdx.y * 8 + 7); // the CTA's keys end at its last query
    float q[HD];
    {
        const float *qp = qk + (size_t)(valid ? t : 0) * (qd + kvd) + (size_t)h * HD;
#pragma unroll
        for (int d = 0; d < HD; ++d) q[d] = qp[d] * scale;
    }
    float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;
    for (int k0 = 0; k0 <= last_q; k0 += 32) {
        __syncthreads(); // the previous block's tiles are no longer read
        for (int i = threadIdx.x; i < 32 * HD; i += 256) {
            const int j = i / HD, d = i % HD, kp = min(k0 + j, last_q);
            ks[j][d] = kv_to<KV_T>(kc[(size_t)kp * kvd + (size_t)kvh * HD + d]);
            vs[j][d] = kv_to<KV_T>(vc[(size_t)kp * kvd + (size_t)kvh * HD + d]);
        }
        __syncthreads();
        if (k0 > qpos) continue; // this query's keys are exhausted (other warps of the CTA still need the tiles)
        float sc = 0.f;
#pragma unroll
        for (int d = 0; d < HD; ++d) sc += q[d] * ks[lane][d];
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
#pragma unroll
            for (int e = 0; e < E; ++e) acc[e] += pb * vs[j][lane * E + e];
        }
    }
    if (valid) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int e = 0; e < E; ++e) out[(size_t)t * qd + (size_t)h * HD + lane * E + e] = acc[e] * inv;
    }
}

__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ y, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        float4 a = *(float4 *)(x + i);
        const float4 b = *(const float4 *)(y + i);
        a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
        *(float4 *)(x + i) = a;
    } else {
        for (size_t j = i; j < n; ++j) x[j] += y[j];
    }
}

// gu: [s, 2 * ff] with rows of the matrix interleaved (gate_j, up_j) -> h[s, ff] = silu(g) * u (math.rs:103-105)
__global__ void swiglu_batch_kernel(const float *__restrict__ gu, float *__restrict__ h, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float2 p = *(const float2 *)(gu + 2 * i);
    h[i] = p.x / (1.0f + expf(-p.x)) * p.y;
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
        TRY(dev_alloc((void **)&bgu, B * 2 * F * 4));
        TRY(dev_alloc((void **)&bh, B * F * 4));
        TRY(dev_alloc((void **)&bt, B * E * 4));
        TRY(dev_alloc(&bscratch, scratch));
    }
    auto gemm = [&](const Mat &m, const float *in, float *out, size_t n) {
        ++launches;
        return launch_gemm_tc(m.fmt, m.w, in, out, bscratch, m.out, m.cols, n, dev.sm_count, d_status, stream);
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
            if (P.kv_f16) {
                rope_kv_batch_kernel<__half><<<(unsigned)n, 256, 0, stream>>>(bqk, bv, rope, (__half *)kc, (__half *)vc, (int)c0, (int)hd, (int)qd, (int)kvd);
                if (hd == 64) attn_prefill_kernel<64, __half><<<ag, 256, 0, stream>>>(bqk, (const __half *)kc, (const __half *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                else attn_prefill_kernel<128, __half><<<ag, 256, 0, stream>>>(bqk, (const __half *)kc, (const __half *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
            } else {
                rope_kv_batch_kernel<float><<<(unsigned)n, 256, 0, stream>>>(bqk, bv, rope, (float *)kc, (float *)vc, (int)c0, (int)hd, (int)qd, (int)kvd);
                if (hd == 64) attn_prefill_kernel<64, float><<<ag, 256, 0, stream>>>(bqk, (const float *)kc, (const float *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
                else attn_prefill_kernel<128, float><<<ag, 256, 0, stream>>>(bqk, (const float *)kc, (const float *)vc, bxn, (int)n, (int)c0, (int)qd, (int)kvd, kvmul, scale);
            }
            TRY(cudaGetLastError());
            TRY(gemm(L.wo, bxn, bt, n)); // attention output [n, qd] sits in bxn
            add_inplace_kernel<<<(unsigned)((n * E / 4 + 255) / 256 + 1), 256, 0, stream>>>(bx, bt, n * E);
            rmsnorm_batch_kernel<<<(unsigned)n, 256, 0, stream>>>(bx, L.ffn_norm, P.eps, (int)E, bxn);
            TRY(gemm(L.wgu, bxn, bgu, n));
            swiglu_batch_kernel<<<(unsigned)((n * F + 255) / 256), 256, 0, stream>>>(bgu, bh, n * F);
            TRY(gemm(L.wd, bh, bt, n));
            add_inplace_kernel<<<(unsigned)((n * E / 4 + 255) / 256 + 1), 256, 0, stream>>>(bx, bt, n * E);
            TRY(cudaGetLastError());
        }
        if (c0 + n == s) { // the last token's hidden state -> final norm + output projection
            TRY(cudaMemcpyAsync(x, bx + (n - 1) * E, E * 4, cudaMemcpyDeviceToDevice, stream));
            TRY(mv(output, x, logits, final_norm, EPI_STORE, nullptr));
        }
    }
    TRY(cudaMemcpyAsync(logits_host, logits, P.vocab * 4, cudaMemcpyDeviceToHost, stream));
#undef TRY
    return cudaStreamSynchronize(stream);
}

} // namespace ullm
