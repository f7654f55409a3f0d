// Host-side objects behind the opaque handles of the C ABI.
#pragma once

#include "common.cuh"
#include "kernels.h"

#include <cstdarg>
#include <cstdio>

struct ullm_cuda_buf {
    void *ptr = nullptr;
    size_t len = 0;
};

struct ullm_cuda_ctx {
    int device = 0;
    char name[256] = {0};
    ullm::DeviceInfo dev;
    cudaStream_t stream = nullptr;
    // Status word the kernels write when a bounded wait expires: mapped pinned
    // host memory, so the host reads it without a copy.
    volatile int *h_status = nullptr;
    int *d_status = nullptr;
    char err[512] = {0};
    // Grow-only device staging areas for the host-buffer entry points.
    struct Scratch {
        void *ptr = nullptr;
        size_t cap = 0;
    } scratch[8];
    bool force_generic = false;
    bool use_pdl = true;  // programmatic dependent launch between the library's kernels (ULLM_OPT_PDL)
    bool no_prepare = false; // keep Q6_K weights in their verbatim bytes (tests)
    bool no_chain = false;   // run op lists one kernel per op (tests, comparisons)
    bool no_host_kernels = false; // host vectors always through cudaMemcpyAsync (comparisons)
    unsigned *d_sync = nullptr; // grid-barrier counter of the chain kernel
    int plan_wr = 0, plan_rw = 0, plan_stages = 0;
    int shard_timeout_ms = 2000; // ULLM_OPT_SHARD_TIMEOUT_MS
    int shard_gemm_exchange = 0; // prefill form's block transfer: 0 chosen per block, 1 copy engines, 2 copy kernel (comparisons)
    bool shard_no_tagged = false; // sharded matvec steps through the flag protocol only (tests, comparisons)
    int gemm_min_s = 32; // batches below this many tokens use per-token matvecs
    ullm::MatvecPlan last_plan;
};

// A weight matrix resident on the device (the `WBuf` of the reference, forward.rs:119-126).
struct ullm_cuda_weight {
    int fmt = 0;          // kernel format, FMT_Q6KR when the rows were prepared
    int dtype = 0;        // ullm_dtype the caller gave
    void *w = nullptr;
    void *scales = nullptr, *biases = nullptr;
    int table_bytes = 4;
    size_t group = 0, out = 0, cols = 0, nbytes = 0, tbytes = 0;
    // Row-sharded weights (ullm_cuda_shard_weight_create): this object holds rows
    // [row0, row0 + out) of a matrix of out_total rows; out_total == 0 for ordinary weights.
    size_t row0 = 0, out_total = 0;
};

inline int ctx_fail(ullm_cuda_ctx *c, int code, const char *fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof c->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define ULLM_CUDA_TRY(ctx, expr)                                                                   \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            cudaGetLastError();                                                                    \
            return ctx_fail((ctx), e__ == cudaErrorMemoryAllocation ? 5 /*OOM*/ : 3 /*CUDA*/,      \
                            "%s failed: %s", #expr, cudaGetErrorString(e__));                      \
        }                                                                                          \
    } while (0)

// Device staging area `slot`, at least `bytes` large (never shrinks).
inline int ctx_scratch(ullm_cuda_ctx *c, int slot, size_t bytes, void **out) {
    auto &s = c->scratch[slot];
    if (s.cap < bytes) {
        if (s.ptr) {
            cudaStreamSynchronize(c->stream);
            cudaFree(s.ptr);
            s.ptr = nullptr, s.cap = 0;
        }
        size_t cap = bytes < 4096 ? 4096 : bytes;
        cudaError_t e = cudaMalloc(&s.ptr, cap);
        if (e != cudaSuccess) {
            cudaGetLastError();
            s.ptr = nullptr;
            return ctx_fail(c, 5, "cudaMalloc(%zu) for staging failed: %s", cap, cudaGetErrorString(e));
        }
        s.cap = cap;
    }
    *out = s.ptr;
    return 0;
}

// After a synchronize: turns a device-side timeout into ULLM_ERR_TIMEOUT.
inline int ctx_check_status(ullm_cuda_ctx *c) {
    if (c->h_status && *c->h_status != ullm::DEV_OK) {
        *c->h_status = ullm::DEV_OK;
        if (c->d_sync) cudaMemset(c->d_sync, 0, 256); // a chain that gave up may have left its barrier half-way
        return ctx_fail(c, 4, "a device-side bounded wait expired (kernel gave up instead of hanging)");
    }
    return 0;
}
