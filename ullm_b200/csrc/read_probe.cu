// Read-only bandwidth probe: what this GPU delivers to kernels that only READ a large buffer, the
// access pattern of a batch-1 quantized matvec (weights are read once and never written).  The copy
// bandwidth a roofline is usually quoted against counts reads and writes of a copy; a pure reader has
// its own ceiling, and the two ways of reading differ:
//   mode 0  plain 16-byte loads, grid-stride, 16 CTAs of 512 threads per SM (evict-first);
//   mode 1  one warp per SM feeding a shared-memory ring with bulk copies (cp.async.bulk), each stage
//           requested again as soon as it has landed: the producer side of matvec_chain_kernel /
//           matvec_stream_kernel with the arithmetic taken away, i.e. the ceiling of that design.
// Measurement tool only (bench.py reports the two rates beside the kernel's); nothing in the product
// path calls it.
#include "../../include/ullm_cuda.h"
#include "common.cuh"
#include "engine.h"
#include "kernels.h"

#include <algorithm>
#include <vector>

namespace ullm {

template <int U>
__global__ void __launch_bounds__(512) read_probe_ld_kernel(const uint4 *__restrict__ p, size_t n16, unsigned *sink) {
    unsigned acc = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x * U;
    for (size_t i = (size_t)blockIdx.x * blockDim.x * U + threadIdx.x; i < n16; i += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t j = i + (size_t)u * blockDim.x;
            v[u] = j < n16 ? __ldcs(p + j) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    if (acc == 0x12345678u) *sink = acc; // keeps the loads alive; the buffer holds no such pattern
}

// CTA b streams tiles [t0, t1) of `stage_bytes` each through S stages; no consumer.
__global__ void __launch_bounds__(32) read_probe_ring_kernel(const uint8_t *p, size_t bytes, uint32_t stage_bytes, uint32_t S,
                                                             uint32_t chunk, int *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem;
    uint8_t *ring = smem + 128;
    const uint32_t lane = threadIdx.x;
    if (lane == 0) {
        for (uint32_t s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncwarp();
    const size_t ntiles = bytes / stage_bytes, per = (ntiles + gridDim.x - 1) / gridDim.x;
    const size_t t0 = per * blockIdx.x, t1 = min(ntiles, t0 + per);
    auto issue = [&](size_t t, uint32_t s) {
        if (lane == 0) mbar_arrive_expect_tx(&full[s], stage_bytes);
        __syncwarp();
        const uint8_t *src = p + t * stage_bytes;
        uint8_t *dst = ring + (size_t)s * stage_bytes;
        for (uint32_t off = lane * chunk; off < stage_bytes; off += 32 * chunk)
            bulk_g2s(dst + off, src + off, min(chunk, stage_bytes - off), &full[s]);
    };
    size_t t = t0;
    for (uint32_t s = 0; s < S && t < t1; ++s, ++t) issue(t, s);
    uint32_t s = 0, ph = 0;
    for (size_t c = t0; c < t1; ++c) {
        bool ok = true;
        if (lane == 0) { // bounded: about half a second of polling
            const long long st = clock64();
            while (!mbar_try_wait(&full[s], ph))
                if (clock64() - st > (1ll << 30)) {
                    ok = false;
                    break;
                }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
            if (lane == 0) *(volatile int *)status = DEV_TIMEOUT;
            return;
        }
        if (t < t1) issue(t++, s);
        if (++s == S) s = 0, ph ^= 1u;
    }
}

} // namespace ullm

// us_out[0..2] = median, min, max over `reps` launches, each after a write of 256 MB (more than the L2 holds).
extern "C" int ullm_cuda_debug_read_probe(ullm_cuda_ctx *c, int mode, size_t bytes, int stage_bytes, int stages, int chunk, int reps,
                                          float *us_out) {
    using namespace ullm;
    if (!c || !us_out || reps < 1 || reps > 1000 || bytes < ((size_t)16 << 20) || bytes > ((size_t)4 << 30)) return ULLM_ERR_INVALID;
    if (mode == 1) {
        if (stage_bytes < 1024 || stage_bytes % 16 || chunk < 1024 || chunk % 16 || stages < 1 || stages > 16) return ULLM_ERR_INVALID;
        if (128 + (size_t)stage_bytes * stages > (size_t)c->dev.max_smem_optin) return ULLM_ERR_INVALID;
    } else if (mode != 0) return ULLM_ERR_INVALID;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    uint8_t *buf = nullptr, *flush = nullptr;
    unsigned *sink = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    const size_t flush_bytes = (size_t)256 << 20;
    int rc = ULLM_OK;
    std::vector<float> us;
    cudaError_t e = cudaMalloc(&buf, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&flush, flush_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&sink, 4);
    if (e == cudaSuccess) e = cudaMemsetAsync(buf, 1, bytes, c->stream);
    if (e == cudaSuccess) e = cudaEventCreate(&a);
    if (e == cudaSuccess) e = cudaEventCreate(&b);
    if (e == cudaSuccess && mode == 1)
        e = cudaFuncSetAttribute(read_probe_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 + stage_bytes * stages);
    for (int i = 0; e == cudaSuccess && i < reps + 2; ++i) {
        cudaMemsetAsync(flush, i, flush_bytes, c->stream);
        cudaEventRecord(a, c->stream);
        if (mode == 0)
            read_probe_ld_kernel<8><<<c->dev.sm_count * 16, 512, 0, c->stream>>>((const uint4 *)buf, bytes / 16, sink);
        else
            read_probe_ring_kernel<<<c->dev.sm_count, 32, 128 + (size_t)stage_bytes * stages, c->stream>>>(
                buf, bytes, (uint32_t)stage_bytes, (uint32_t)stages, (uint32_t)chunk, c->d_status);
        cudaEventRecord(b, c->stream);
        e = cudaEventSynchronize(b);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (i >= 2) us.push_back(ms * 1e3f); // the first two launches warm up
    }
    if (e != cudaSuccess) {
        snprintf(c->err, sizeof c->err, "read probe: %s", cudaGetErrorString(e));
        rc = ULLM_ERR_CUDA;
    } else if (c->h_status && *c->h_status == DEV_TIMEOUT) {
        rc = ULLM_ERR_TIMEOUT;
    } else {
        std::sort(us.begin(), us.end());
        us_out[0] = us[us.size() / 2], us_out[1] = us.front(), us_out[2] = us.back();
    }
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    cudaFree(sink), cudaFree(flush), cudaFree(buf);
    cudaSetDevice(prev);
    return rc;
}
