// C ABI of the backend (see include/ullm_cuda.h).  Thin, validating wrappers:
// shapes and pointers are checked on the host before anything is launched, CUDA
// failures are turned into status codes with a message, and nothing here ever
// computes on the CPU.
#include "../../include/ullm_cuda.h"
#include "../../include/ullm_gguf.h"
#include "../../include/ullm_safetensors.h"
#include "decode.h"
#include "engine.h"
#include "host_copy.cuh"

#include <algorithm>
#include <string>
#include <vector>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

using namespace ullm;

// ---- context ---------------------------------------------------------------
int ullm_cuda_ctx_create(int device, ullm_cuda_ctx **out) {
    if (!out) return ULLM_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return ULLM_ERR_UNSUPPORTED; // "no CUDA device available"
    }
    if (device < 0 || device >= n) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = new (std::nothrow) ullm_cuda_ctx();
    if (!c) return ULLM_ERR_OOM;
    c->device = device;
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete c;
        return ULLM_ERR_CUDA;
    }
    if (prop.major != 10) { // the kernels are sm_100a only; no other path exists
        delete c;
        return ULLM_ERR_UNSUPPORTED;
    }
    snprintf(c->name, sizeof c->name, "%s", prop.name);
    c->dev.sm_count = prop.multiProcessorCount;
    c->dev.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    c->dev.max_smem_sm = (int)prop.sharedMemPerMultiprocessor;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaHostAlloc((void **)&c->h_status, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void **)&c->d_status, (void *)c->h_status, 0) != cudaSuccess) {
        ullm_cuda_ctx_destroy(c);
        return ULLM_ERR_CUDA;
    }
    *c->h_status = 0;
    *out = c;
    return ULLM_OK;
}

void ullm_cuda_ctx_destroy(ullm_cuda_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) {
        cudaStreamSynchronize(c->stream);
        cudaStreamDestroy(c->stream);
    }
    if (c->h_status) cudaFreeHost((void *)c->h_status);
    if (c->d_sync) cudaFree(c->d_sync);
    for (auto &s : c->scratch)
        if (s.ptr) cudaFree(s.ptr);
    delete c;
}

const char *ullm_cuda_last_error(const ullm_cuda_ctx *c) { return c ? c->err : "null context"; }

int ullm_cuda_ctx_set_option(ullm_cuda_ctx *c, int option, int value) {
    if (!c) return ULLM_ERR_INVALID;
    switch (option) {
    case ULLM_OPT_PDL: c->use_pdl = value != 0; return ULLM_OK;
    case ULLM_OPT_SHARD_TIMEOUT_MS:
        if (value < 1) return ctx_fail(c, ULLM_ERR_INVALID, "the time limit must be at least 1 ms");
        c->shard_timeout_ms = value;
        return ULLM_OK;
    default: return ctx_fail(c, ULLM_ERR_INVALID, "unknown option %d", option);
    }
}

int ullm_cuda_device_name(const ullm_cuda_ctx *c, char *name, size_t cap) {
    if (!c || !name || cap == 0) return ULLM_ERR_INVALID;
    snprintf(name, cap, "%s", c->name);
    return ULLM_OK;
}
int ullm_cuda_sm_count(const ullm_cuda_ctx *c) { return c ? c->dev.sm_count : 0; }

int ullm_cuda_synchronize(ullm_cuda_ctx *c) {
    if (!c) return ULLM_ERR_INVALID;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

// ---- buffers ---------------------------------------------------------------
int ullm_cuda_alloc(ullm_cuda_ctx *c, size_t len, ullm_cuda_buf **out) {
    if (!c || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ullm_cuda_buf *b = new (std::nothrow) ullm_cuda_buf();
    if (!b) return ULLM_ERR_OOM;
    b->len = len;
    cudaError_t e = cudaMalloc(&b->ptr, len ? len : 16);
    if (e != cudaSuccess) {
        delete b;
        cudaGetLastError();
        return ctx_fail(c, e == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "cudaMalloc(%zu): %s", len,
                        cudaGetErrorString(e));
    }
    *out = b;
    return ULLM_OK;
}
int ullm_cuda_upload(ullm_cuda_ctx *c, const void *bytes, size_t len, ullm_cuda_buf **out) {
    if (!c || !out || (!bytes && len)) return ULLM_ERR_INVALID;
    int rc = ullm_cuda_alloc(c, len, out);
    if (rc) return rc;
    if (len) {
        cudaError_t e = cudaMemcpyAsync((*out)->ptr, bytes, len, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) {
            ullm_cuda_buf_free(c, *out);
            *out = nullptr;
            return ctx_fail(c, ULLM_ERR_CUDA, "upload: %s", cudaGetErrorString(e));
        }
    }
    return ULLM_OK;
}
int ullm_cuda_download(ullm_cuda_ctx *c, const ullm_cuda_buf *b, size_t offset, void *host, size_t len) {
    if (!c || !b || (!host && len)) return ULLM_ERR_INVALID;
    if (offset > b->len || len > b->len - offset) return ctx_fail(c, ULLM_ERR_FORMAT, "download: range outside buffer");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(host, (const uint8_t *)b->ptr + offset, len, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ULLM_OK;
}
void *ullm_cuda_buf_ptr(const ullm_cuda_buf *b) { return b ? b->ptr : nullptr; }
size_t ullm_cuda_buf_len(const ullm_cuda_buf *b) { return b ? b->len : 0; }
void ullm_cuda_buf_free(ullm_cuda_ctx *c, ullm_cuda_buf *b) {
    if (!b) return;
    if (c) cudaSetDevice(c->device);
    if (b->ptr) cudaFree(b->ptr);
    delete b;
}

// ---- helpers ---------------------------------------------------------------
static int fmt_of(int dtype) {
    switch (dtype) {
    case ULLM_DTYPE_Q4_K: return FMT_Q4K;
    case ULLM_DTYPE_Q6_K: return FMT_Q6K;
    case ULLM_DTYPE_MLX_U32: return FMT_MLX4;
    default: return -1;
    }
}
static size_t weight_bytes(int fmt, size_t out_dim, size_t in_dim) {
    if (fmt == FMT_Q4K) return out_dim * (in_dim / QK_K) * Q4K_BYTES;
    if (fmt == FMT_Q6K) return out_dim * (in_dim / QK_K) * Q6K_BYTES;
    return out_dim * (in_dim / 8) * 4;
}

// ---- dequantization --------------------------------------------------------
int ullm_cuda_dequantize(ullm_cuda_ctx *c, int dtype, const void *data, size_t data_len, float *out, size_t n) {
    if (!c || (!data && data_len) || (!out && n)) return ULLM_ERR_INVALID;
    size_t block, ts;
    switch (dtype) {
    case ULLM_DTYPE_F32: block = 1, ts = 4; break;
    case ULLM_DTYPE_F16: case ULLM_DTYPE_BF16: block = 1, ts = 2; break;
    case ULLM_DTYPE_Q4_K: block = QK_K, ts = Q4K_BYTES; break;
    case ULLM_DTYPE_Q6_K: block = QK_K, ts = Q6K_BYTES; break;
    default: return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "dequantization of dtype %d is not implemented", dtype);
    }
    // crates/ullm-core/src/dequant.rs:65-77
    if (n % block) return ctx_fail(c, ULLM_ERR_FORMAT, "element count %zu is not a multiple of block size %zu", n, block);
    size_t need = n / block * ts;
    if (data_len < need) return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu bytes, have %zu", need, data_len);
    if (n == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    void *d_in = nullptr, *d_out = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, need, &d_in)) || (rc = ctx_scratch(c, 1, n * 4, &d_out))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_in, data, need, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, launch_dequant(dtype, d_in, (float *)d_out, n, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(out, d_out, n * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ULLM_OK;
}

int ullm_cuda_dequantize_mlx4(ullm_cuda_ctx *c, const uint32_t *weight, const float *scales, const float *biases,
                              size_t out_dim, size_t in_dim, size_t group, float *y) {
    if (!c || !weight || !scales || !biases || !y) return ULLM_ERR_INVALID;
    if (const char *m = matvec_shape_error(FMT_MLX4, out_dim, in_dim, group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    size_t wb = out_dim * (in_dim / 8) * 4, tb = out_dim * (in_dim / group) * 4, yb = out_dim * in_dim * 4;
    void *d_w = nullptr, *d_s = nullptr, *d_b = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, wb, &d_w)) || (rc = ctx_scratch(c, 1, yb, &d_y)) || (rc = ctx_scratch(c, 2, tb, &d_s)) ||
        (rc = ctx_scratch(c, 3, tb, &d_b)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_w, weight, wb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_s, scales, tb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_b, biases, tb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, launch_dequant_mlx4((const uint32_t *)d_w, (const float *)d_s, (const float *)d_b, (float *)d_y,
                                         out_dim, in_dim, group, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, yb, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ULLM_OK;
}

// ---- matvec ----------------------------------------------------------------
int ullm_cuda_matvec_dev(ullm_cuda_ctx *c, int dtype, const void *d_w, const void *d_scales, const void *d_biases,
                         int table_dtype, size_t group, const float *d_x, float *d_y, size_t out_dim, size_t in_dim,
                         void *stream) {
    if (!c || !d_w || !d_x || !d_y) return ULLM_ERR_INVALID;
    int fmt = fmt_of(dtype);
    if (fmt < 0) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA kernel for dtype %d yet", dtype);
    MlxTables tb;
    if (fmt == FMT_MLX4) {
        if (!d_scales || !d_biases) return ULLM_ERR_INVALID;
        if (table_dtype != ULLM_DTYPE_F32 && table_dtype != ULLM_DTYPE_BF16)
            return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "MLX tables must be f32 or bf16");
        tb.scales = d_scales, tb.biases = d_biases, tb.group = group;
        tb.elem_bytes = table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
    }
    if (const char *m = matvec_shape_error(fmt, out_dim, in_dim, group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    if ((uintptr_t)d_w % 16 || (uintptr_t)d_x % 16 || (uintptr_t)d_y % 4)
        return ctx_fail(c, ULLM_ERR_FORMAT, "device pointers must be 16-byte aligned");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    MatvecOpts mo;
    mo.force_generic = c->force_generic, mo.pdl = c->use_pdl, mo.plan_out = &c->last_plan;
    mo.plan_wr = c->plan_wr, mo.plan_rw = c->plan_rw, mo.plan_stages = c->plan_stages;
    ULLM_CUDA_TRY(c, launch_matvec(c->dev, fmt, d_w, tb, d_x, d_y, out_dim, in_dim, c->d_status, st, mo));
    return ULLM_OK;
}

// x (host) -> device scratch, run, y -> host, wait.
static int matvec_host(ullm_cuda_ctx *c, int dtype, const void *d_w, const void *d_s, const void *d_b, int tdt,
                       size_t group, const float *x, float *y, size_t out_dim, size_t in_dim) {
    void *d_x = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, in_dim * 4, &d_x)) || (rc = ctx_scratch(c, 5, out_dim * 4, &d_y))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_x, x, in_dim * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = ullm_cuda_matvec_dev(c, dtype, d_w, d_s, d_b, tdt, group, (const float *)d_x, (float *)d_y, out_dim, in_dim,
                                   nullptr)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, out_dim * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_matvec_resident(ullm_cuda_ctx *c, int dtype, const ullm_cuda_buf *w, const float *x, float *y,
                              size_t out_dim, size_t in_dim) {
    if (!c || !w || !x || !y) return ULLM_ERR_INVALID;
    int fmt = fmt_of(dtype);
    // MetalContext::pso_for (crates/ullm-metal/src/lib.rs:268-276): only the k-quants
    if (fmt != FMT_Q4K && fmt != FMT_Q6K) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA kernel for dtype %d yet", dtype);
    if (const char *m = matvec_shape_error(fmt, out_dim, in_dim, 0)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    if (w->len < weight_bytes(fmt, out_dim, in_dim))
        return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu weight bytes, have %zu", weight_bytes(fmt, out_dim, in_dim), w->len);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    return matvec_host(c, dtype, w->ptr, nullptr, nullptr, 0, 0, x, y, out_dim, in_dim);
}

int ullm_cuda_matvec_quant(ullm_cuda_ctx *c, int dtype, const void *w_bytes, size_t w_len, const float *x, float *y,
                           size_t out_dim, size_t in_dim) {
    if (!c || !w_bytes || !x || !y) return ULLM_ERR_INVALID;
    int fmt = fmt_of(dtype);
    if (fmt != FMT_Q4K && fmt != FMT_Q6K) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA kernel for dtype %d yet", dtype);
    if (const char *m = matvec_shape_error(fmt, out_dim, in_dim, 0)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    size_t need = weight_bytes(fmt, out_dim, in_dim);
    if (w_len < need) return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu weight bytes, have %zu", need, w_len);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    void *d_w = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, need, &d_w))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_w, w_bytes, need, cudaMemcpyHostToDevice, c->stream));
    return matvec_host(c, dtype, d_w, nullptr, nullptr, 0, 0, x, y, out_dim, in_dim);
}

int ullm_cuda_matvec_mlx4(ullm_cuda_ctx *c, const void *w, const float *scales, const float *biases, const float *x,
                          float *y, size_t out_dim, size_t in_dim, size_t group) {
    if (!c || !w || !scales || !biases || !x || !y) return ULLM_ERR_INVALID;
    if (const char *m = matvec_shape_error(FMT_MLX4, out_dim, in_dim, group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    size_t wb = weight_bytes(FMT_MLX4, out_dim, in_dim), tb = out_dim * (in_dim / group) * 4;
    void *d_w = nullptr, *d_s = nullptr, *d_b = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, wb, &d_w)) || (rc = ctx_scratch(c, 2, tb, &d_s)) || (rc = ctx_scratch(c, 3, tb, &d_b)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_w, w, wb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_s, scales, tb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_b, biases, tb, cudaMemcpyHostToDevice, c->stream));
    return matvec_host(c, ULLM_DTYPE_MLX_U32, d_w, d_s, d_b, ULLM_DTYPE_F32, group, x, y, out_dim, in_dim);
}

// ---- resident weights ------------------------------------------------------

int ullm_cuda_weight_create(ullm_cuda_ctx *c, const ullm_gpu_weight *gw, int mlx_table_dtype, ullm_cuda_weight **out) {
    if (!c || !gw || !out || !gw->bytes) return ULLM_ERR_INVALID;
    *out = nullptr;
    int fmt = fmt_of(gw->dtype);
    if (fmt < 0) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA forward kernel for dtype %d", gw->dtype); // forward.rs:376-378
    if (const char *m = matvec_shape_error(fmt, gw->out, gw->cols, gw->mlx_group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    const size_t need = weight_bytes(fmt, gw->out, gw->cols);
    if (gw->len < need) return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu weight bytes, have %zu", need, gw->len);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ullm_cuda_weight *w = new (std::nothrow) ullm_cuda_weight();
    if (!w) return ULLM_ERR_OOM;
    w->fmt = fmt, w->dtype = gw->dtype, w->out = gw->out, w->cols = gw->cols, w->nbytes = need, w->group = gw->mlx_group;
    cudaError_t e = cudaMalloc(&w->w, need);
    if (e == cudaSuccess && fmt == FMT_MLX4) {
        if (!gw->mlx_scales || !gw->mlx_biases || (mlx_table_dtype != ULLM_DTYPE_F32 && mlx_table_dtype != ULLM_DTYPE_BF16)) {
            ullm_cuda_weight_destroy(c, w);
            return ctx_fail(c, ULLM_ERR_FORMAT, "MLX weights need scale and bias tables (f32 or bf16)");
        }
        w->table_bytes = mlx_table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
        w->tbytes = gw->out * (gw->cols / gw->mlx_group) * w->table_bytes;
        e = cudaMalloc(&w->scales, w->tbytes);
        if (e == cudaSuccess) e = cudaMalloc(&w->biases, w->tbytes);
        if (e == cudaSuccess) e = cudaMemcpyAsync(w->scales, gw->mlx_scales, w->tbytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(w->biases, gw->mlx_biases, w->tbytes, cudaMemcpyHostToDevice, c->stream);
    }
    if (e == cudaSuccess && fmt == FMT_Q6K && q6k_can_prepare(gw->cols) && !c->no_prepare) {
        void *tmp = nullptr; // raw bytes land in staging, the prepared rows in the weight
        int rc = ctx_scratch(c, 0, need, &tmp);
        if (rc) {
            ullm_cuda_weight_destroy(c, w);
            return rc;
        }
        e = cudaMemcpyAsync(tmp, gw->bytes, need, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = launch_q6k_prepare(tmp, w->w, gw->out, gw->cols, false, c->stream);
        w->fmt = FMT_Q6KR;
    } else if (e == cudaSuccess) {
        e = cudaMemcpyAsync(w->w, gw->bytes, need, cudaMemcpyHostToDevice, c->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        ullm_cuda_weight_destroy(c, w);
        return ctx_fail(c, e == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "weight upload: %s", cudaGetErrorString(e));
    }
    *out = w;
    return ULLM_OK;
}

int ullm_cuda_weight_create_st(ullm_cuda_ctx *c, const ullm_st *st, const char *name, size_t group, ullm_cuda_weight **out) {
    if (!c || !st || !name || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    char msg[256] = {0};
    ullm_st_mlx_weight mw;
    if (ullm_st_mlx_weight_get(st, name, group, &mw, msg, sizeof msg)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
    ullm_gpu_weight gw;
    memset(&gw, 0, sizeof gw);
    gw.dtype = ULLM_DTYPE_MLX_U32, gw.bytes = mw.weight, gw.len = (size_t)(mw.out * (mw.in / 8) * 4), gw.out = (size_t)mw.out, gw.cols = (size_t)mw.in;
    gw.mlx_scales = (const float *)mw.scales, gw.mlx_biases = (const float *)mw.biases, gw.mlx_group = group; // bf16 bits, said so below
    return ullm_cuda_weight_create(c, &gw, ULLM_DTYPE_BF16, out);
}

void ullm_cuda_weight_destroy(ullm_cuda_ctx *c, ullm_cuda_weight *w) {
    if (!w) return;
    if (c) cudaSetDevice(c->device);
    if (w->w) cudaFree(w->w);
    if (w->scales) cudaFree(w->scales);
    if (w->biases) cudaFree(w->biases);
    delete w;
}

size_t ullm_cuda_weight_bytes(const ullm_cuda_weight *w) { return w ? w->nbytes : 0; }

int ullm_cuda_weight_matvec_dev(ullm_cuda_ctx *c, const ullm_cuda_weight *w, const float *d_x, float *d_y, void *stream) {
    if (!c || !w || !d_x || !d_y) return ULLM_ERR_INVALID;
    if ((uintptr_t)d_x % 16 || (uintptr_t)d_y % 4) return ctx_fail(c, ULLM_ERR_FORMAT, "device pointers must be 16-byte aligned");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    MlxTables tb;
    tb.scales = w->scales, tb.biases = w->biases, tb.elem_bytes = w->table_bytes, tb.group = w->group;
    MatvecOpts mo;
    mo.force_generic = c->force_generic && w->fmt != FMT_Q6KR, mo.pdl = c->use_pdl, mo.plan_out = &c->last_plan;
    mo.plan_wr = c->plan_wr, mo.plan_rw = c->plan_rw, mo.plan_stages = c->plan_stages;
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    ULLM_CUDA_TRY(c, launch_matvec(c->dev, w->fmt, w->w, tb, d_x, d_y, w->out, w->cols, c->d_status, st, mo));
    return ULLM_OK;
}

// The grid barrier counter of the chain kernel (one unsigned per context, allocated on first use).
static int ctx_sync_word(ullm_cuda_ctx *c, unsigned **out) {
    if (!c->d_sync) {
        cudaError_t e = cudaMalloc((void **)&c->d_sync, 256);
        if (e == cudaSuccess) e = cudaMemset(c->d_sync, 0, 256);
        if (e != cudaSuccess) {
            cudaGetLastError();
            c->d_sync = nullptr;
            return ctx_fail(c, ULLM_ERR_OOM, "cudaMalloc for the chain barrier failed: %s", cudaGetErrorString(e));
        }
    }
    *out = c->d_sync;
    return ULLM_OK;
}

int ullm_cuda_weight_matvec_chain_dev(ullm_cuda_ctx *c, size_t n, const ullm_chain_op *ops, void *stream) {
    if (!c || (n && !ops)) return ULLM_ERR_INVALID;
    if (n == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    std::vector<MatvecChainOp> v(n);
    bool chain_ok = !c->force_generic && !c->no_chain;
    for (size_t i = 0; i < n; ++i) {
        const ullm_chain_op &o = ops[i];
        if (!o.w || !o.d_x || !o.d_y) return ULLM_ERR_INVALID;
        if (o.epi < ULLM_EPI_STORE || o.epi > ULLM_EPI_SWIGLU) return ctx_fail(c, ULLM_ERR_INVALID, "op %zu: unknown epilogue %d", i, o.epi);
        if (o.epi == ULLM_EPI_RESIDUAL && !o.d_res) return ctx_fail(c, ULLM_ERR_INVALID, "op %zu: residual epilogue without d_res", i);
        MatvecChainOp &m = v[i];
        m.fmt = o.w->fmt, m.w = o.w->w, m.x = o.d_x, m.y = o.d_y, m.out_dim = o.w->out, m.in_dim = o.w->cols;
        m.norm_w = o.d_norm_w, m.eps = o.eps, m.epi = o.epi, m.res = o.d_res, m.dep = o.dep != 0;
        chain_ok = chain_ok && matvec_chain_supported(m.fmt, m.out_dim, m.in_dim, m.epi);
    }
    // one persistent launch per run of at most 12 ops; anything it cannot take goes op by op
    if (chain_ok) {
        unsigned *d_sync = nullptr;
        int rc = ctx_sync_word(c, &d_sync);
        if (rc) return rc;
        size_t i = 0;
        bool fell_back = false;
        while (i < n) {
            const size_t m = std::min<size_t>(12, n - i);
            if (i > 0) v[i].dep = false; // ordered after the previous launch by the stream
            cudaError_t e = launch_matvec_chain(c->dev, (int)m, v.data() + i, d_sync, c->d_status, st, c->use_pdl);
            if (e == cudaErrorNotSupported) {
                cudaGetLastError();
                fell_back = true;
                break;
            }
            if (e != cudaSuccess) {
                cudaGetLastError();
                return ctx_fail(c, ULLM_ERR_CUDA, "matvec chain launch: %s", cudaGetErrorString(e));
            }
            i += m;
        }
        if (!fell_back) {
            c->last_plan = MatvecPlan();
            c->last_plan.streamed = true, c->last_plan.warps = 16, c->last_plan.grid = -2; // marks the chain kernel
            return ULLM_OK;
        }
        if (i > 0) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "matvec chain: ops %zu.. cannot be streamed", i);
    }
    for (size_t i = 0; i < n; ++i) {
        const ullm_chain_op &o = ops[i];
        MlxTables tb;
        tb.scales = o.w->scales, tb.biases = o.w->biases, tb.group = o.w->group, tb.elem_bytes = o.w->table_bytes;
        MatvecOpts mo;
        mo.force_generic = c->force_generic && o.w->fmt != FMT_Q6KR, mo.pdl = c->use_pdl, mo.plan_out = &c->last_plan;
        mo.norm_w = o.d_norm_w, mo.eps = o.eps, mo.epi = o.epi, mo.res = o.d_res;
        cudaError_t e = launch_matvec(c->dev, o.w->fmt, o.w->w, tb, o.d_x, o.d_y, o.w->out, o.w->cols, c->d_status, st, mo);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return ctx_fail(c, e == cudaErrorNotSupported ? ULLM_ERR_UNSUPPORTED : ULLM_ERR_CUDA, "matvec %zu of the chain: %s", i,
                            cudaGetErrorString(e));
        }
    }
    return ULLM_OK;
}

int ullm_cuda_weight_matvec_batch_dev(ullm_cuda_ctx *c, size_t n, const ullm_cuda_weight *const *w, const float *const *d_x,
                                      float *const *d_y, void *stream) {
    if (!c || (n && (!w || !d_x || !d_y))) return ULLM_ERR_INVALID;
    std::vector<ullm_chain_op> ops(n);
    for (size_t i = 0; i < n; ++i) {
        if (!w[i]) return ULLM_ERR_INVALID;
        ops[i] = ullm_chain_op{};
        ops[i].w = w[i], ops[i].d_x = d_x[i], ops[i].d_y = d_y[i];
    }
    return ullm_cuda_weight_matvec_chain_dev(c, n, ops.data(), stream);
}

int ullm_cuda_weight_matvec(ullm_cuda_ctx *c, const ullm_cuda_weight *w, const float *x, float *y) {
    if (!c || !w || !x || !y) return ULLM_ERR_INVALID;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    void *d_x = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, w->cols * 4, &d_x)) || (rc = ctx_scratch(c, 5, w->out * 4, &d_y))) return rc;
    const float *xv = c->no_host_kernels ? nullptr : device_view_of_host(x);
    float *yv = c->no_host_kernels ? nullptr : (float *)device_view_of_host(y);
    if (xv) ULLM_CUDA_TRY(c, vec_copy(xv, (float *)d_x, w->cols, c->stream));
    else ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_x, x, w->cols * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = ullm_cuda_weight_matvec_dev(c, w, (const float *)d_x, (float *)d_y, nullptr))) return rc;
    if (yv) ULLM_CUDA_TRY(c, vec_copy((const float *)d_y, yv, w->out, c->stream));
    else ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, w->out * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_weight_matvec_batch(ullm_cuda_ctx *c, size_t n, const ullm_cuda_weight *const *w, const float *const *x, float *const *y) {
    if (!c || (n && (!w || !x || !y))) return ULLM_ERR_INVALID;
    if (n == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    // one staging area for all inputs and one for all outputs, every vector 16-byte aligned inside it
    size_t xin = 0, yout = 0;
    for (size_t i = 0; i < n; ++i) {
        if (!w[i] || !x[i] || !y[i]) return ULLM_ERR_INVALID;
        xin += (w[i]->cols + 3) & ~(size_t)3, yout += (w[i]->out + 3) & ~(size_t)3;
    }
    void *d_x = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, xin * 4, &d_x)) || (rc = ctx_scratch(c, 5, yout * 4, &d_y))) return rc;
    std::vector<ullm_chain_op> ops(n);
    std::vector<const float *> xv(n);
    std::vector<float *> yv(n);
    size_t xo = 0, yo = 0;
    bool all_mapped = !c->no_host_kernels;
    for (size_t i = 0; i < n; ++i) {
        ops[i] = ullm_chain_op{};
        ops[i].w = w[i], ops[i].d_x = (float *)d_x + xo, ops[i].d_y = (float *)d_y + yo;
        xo += (w[i]->cols + 3) & ~(size_t)3, yo += (w[i]->out + 3) & ~(size_t)3;
        xv[i] = all_mapped ? device_view_of_host(x[i]) : nullptr;
        yv[i] = all_mapped ? (float *)device_view_of_host(y[i]) : nullptr;
        all_mapped = all_mapped && xv[i] && yv[i] && w[i]->cols <= 0xffffffffull && w[i]->out <= 0xffffffffull;
    }
    // page-locked vectors move in one small kernel per direction (up to 16 vectors each); pageable ones by the copy engines
    if (all_mapped) {
        for (size_t i = 0; i < n; i += VEC_COPY_MAX) {
            VecCopyList l{};
            const int m = (int)std::min<size_t>(VEC_COPY_MAX, n - i);
            for (int k = 0; k < m; ++k) l.src[k] = xv[i + k], l.dst[k] = (float *)ops[i + k].d_x, l.n[k] = (unsigned)w[i + k]->cols;
            ULLM_CUDA_TRY(c, vec_copy_multi(l, m, c->stream, c->use_pdl));
        }
    } else {
        for (size_t i = 0; i < n; ++i) ULLM_CUDA_TRY(c, cudaMemcpyAsync((void *)ops[i].d_x, x[i], w[i]->cols * 4, cudaMemcpyHostToDevice, c->stream));
    }
    if ((rc = ullm_cuda_weight_matvec_chain_dev(c, n, ops.data(), nullptr))) return rc;
    if (all_mapped) {
        for (size_t i = 0; i < n; i += VEC_COPY_MAX) {
            VecCopyList l{};
            const int m = (int)std::min<size_t>(VEC_COPY_MAX, n - i);
            for (int k = 0; k < m; ++k) l.src[k] = ops[i + k].d_y, l.dst[k] = yv[i + k], l.n[k] = (unsigned)w[i + k]->out;
            ULLM_CUDA_TRY(c, vec_copy_multi(l, m, c->stream, c->use_pdl));
        }
    } else {
        for (size_t i = 0; i < n; ++i) ULLM_CUDA_TRY(c, cudaMemcpyAsync(y[i], ops[i].d_y, w[i]->out * 4, cudaMemcpyDeviceToHost, c->stream));
    }
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_weight_export(ullm_cuda_ctx *c, const ullm_cuda_weight *w, void *bytes, size_t len) {
    if (!c || !w || !bytes) return ULLM_ERR_INVALID;
    if (len < w->nbytes) return ctx_fail(c, ULLM_ERR_FORMAT, "need room for %zu bytes, have %zu", w->nbytes, len);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    const void *src = w->w;
    if (w->fmt == FMT_Q6KR) {
        void *tmp = nullptr;
        int rc = ctx_scratch(c, 0, w->nbytes, &tmp);
        if (rc) return rc;
        ULLM_CUDA_TRY(c, launch_q6k_prepare(w->w, tmp, w->out, w->cols, true, c->stream));
        src = tmp;
    }
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(bytes, src, w->nbytes, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ULLM_OK;
}

// ---- batched matmul --------------------------------------------------------
// Runs the tensor-core GEMM on weights in kernel format `fmt` (FMT_Q4K verbatim or
// FMT_Q6KR prepared); ULLM_ERR_UNSUPPORTED (silently, no message) when the shape or
// the batch is outside what it takes, so callers can fall back to per-token matvecs.
static int gemm_try(ullm_cuda_ctx *c, int fmt, const void *d_w, const float *d_x, float *d_y, size_t out_dim, size_t in_dim,
                    size_t s, cudaStream_t st, const MlxTables *mlx = nullptr) {
    if (c->force_generic || s < (size_t)c->gemm_min_s) return ULLM_ERR_UNSUPPORTED;
    if (fmt == FMT_MLX4 ? !(mlx && gemm_tc_supported_mlx4(out_dim, in_dim, s, *mlx)) : !gemm_tc_supported(fmt, out_dim, in_dim, s)) return ULLM_ERR_UNSUPPORTED;
    void *xb = nullptr;
    int rc = ctx_scratch(c, 7, gemm_tc_scratch_bytes(out_dim, in_dim, s, c->dev.sm_count), &xb);
    if (rc) return rc;
    cudaError_t e = launch_gemm_tc(fmt, d_w, d_x, d_y, xb, out_dim, in_dim, s, c->dev.sm_count, c->d_status, st, EPI_STORE, nullptr, 0, nullptr, mlx);
    if (e == cudaErrorNotSupported) {
        cudaGetLastError();
        return ULLM_ERR_UNSUPPORTED;
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return ctx_fail(c, ULLM_ERR_CUDA, "tensor-core GEMM launch: %s", cudaGetErrorString(e));
    }
    c->last_plan = MatvecPlan();
    c->last_plan.streamed = true, c->last_plan.warps = 10, c->last_plan.rows_per_tile = 128, c->last_plan.stages = 4;
    c->last_plan.grid = -1; // marks the GEMM kernel
    return ULLM_OK;
}

int ullm_cuda_matmul_dev(ullm_cuda_ctx *c, int dtype, const void *d_w, const void *d_scales, const void *d_biases,
                         int table_dtype, size_t group, const float *d_x, float *d_y, size_t out_dim, size_t in_dim,
                         size_t s, void *stream) {
    if (!c || !d_w || !d_x || !d_y) return ULLM_ERR_INVALID;
    int fmt = fmt_of(dtype);
    if (fmt < 0) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA kernel for dtype %d yet", dtype);
    if (const char *m = matvec_shape_error(fmt, out_dim, in_dim, group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    // Prefill-sized batches go to the tcgen05 GEMM (dequantize to bf16 in shared memory,
    // accumulate in TMEM); Q6_K rows are first re-ordered into the prepared layout.
    if (fmt == FMT_Q4K || (fmt == FMT_Q6K && q6k_can_prepare(in_dim))) {
        const void *gw = d_w;
        int gfmt = fmt, rc = ULLM_OK;
        if (fmt == FMT_Q6K && s >= (size_t)c->gemm_min_s && !c->force_generic) {
            void *prep = nullptr;
            if ((rc = ctx_scratch(c, 6, weight_bytes(fmt, out_dim, in_dim), &prep))) return rc;
            ULLM_CUDA_TRY(c, launch_q6k_prepare(d_w, prep, out_dim, in_dim, false, st));
            gw = prep, gfmt = FMT_Q6KR;
        }
        rc = gemm_try(c, gfmt, gw, d_x, d_y, out_dim, in_dim, s, st);
        if (rc != ULLM_ERR_UNSUPPORTED) return rc;
    }
    // MLX 4-bit words with group 64 (matmul_mlx4, crates/ullm-metal/src/shader.metal:568): the same tensor-core kernel,
    // values q * scale + bias formed in its dequantization stage
    if (fmt == FMT_MLX4 && d_scales && d_biases && (table_dtype == ULLM_DTYPE_F32 || table_dtype == ULLM_DTYPE_BF16)) {
        MlxTables tb;
        tb.scales = d_scales, tb.biases = d_biases, tb.group = group, tb.elem_bytes = table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
        int rc = gemm_try(c, FMT_MLX4, d_w, d_x, d_y, out_dim, in_dim, s, st, &tb);
        if (rc != ULLM_ERR_UNSUPPORTED) return rc;
    }
    // Otherwise the product is formed one token column at a time with the matvec kernel
    // (same arithmetic, weights re-read per token).
    for (size_t t = 0; t < s; ++t) {
        int rc = ullm_cuda_matvec_dev(c, dtype, d_w, d_scales, d_biases, table_dtype, group, d_x + t * in_dim,
                                      d_y + t * out_dim, out_dim, in_dim, stream);
        if (rc) return rc;
    }
    return ULLM_OK;
}

int ullm_cuda_weight_matmul_dev(ullm_cuda_ctx *c, const ullm_cuda_weight *w, const float *d_x, float *d_y, size_t s, void *stream) {
    if (!c || !w || !d_x || !d_y) return ULLM_ERR_INVALID;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    MlxTables tb;
    tb.scales = w->scales, tb.biases = w->biases, tb.elem_bytes = w->table_bytes, tb.group = w->group;
    int rc = gemm_try(c, w->fmt, w->w, d_x, d_y, w->out, w->cols, s, st, w->fmt == FMT_MLX4 ? &tb : nullptr);
    if (rc != ULLM_ERR_UNSUPPORTED) return rc;
    for (size_t t = 0; t < s; ++t)
        if ((rc = ullm_cuda_weight_matvec_dev(c, w, d_x + t * w->cols, d_y + t * w->out, stream))) return rc;
    return ULLM_OK;
}

int ullm_cuda_weight_matmul(ullm_cuda_ctx *c, const ullm_cuda_weight *w, const float *x, float *y, size_t s) {
    if (!c || !w || (s && (!x || !y))) return ULLM_ERR_INVALID;
    if (s == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    void *d_x = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, s * w->cols * 4, &d_x)) || (rc = ctx_scratch(c, 5, s * w->out * 4, &d_y))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_x, x, s * w->cols * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = ullm_cuda_weight_matmul_dev(c, w, (const float *)d_x, (float *)d_y, s, nullptr))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, s * w->out * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

static int matmul_host(ullm_cuda_ctx *c, int dtype, const void *d_w, const void *d_s, const void *d_b, int tdt,
                       size_t group, const float *x, float *y, size_t out_dim, size_t in_dim, size_t s) {
    void *d_x = nullptr, *d_y = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, s * in_dim * 4, &d_x)) || (rc = ctx_scratch(c, 5, s * out_dim * 4, &d_y))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_x, x, s * in_dim * 4, cudaMemcpyHostToDevice, c->stream));
    if ((rc = ullm_cuda_matmul_dev(c, dtype, d_w, d_s, d_b, tdt, group, (const float *)d_x, (float *)d_y, out_dim, in_dim,
                                   s, nullptr)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, s * out_dim * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_matmul_quant(ullm_cuda_ctx *c, int dtype, const void *w_bytes, size_t w_len, const float *x, float *y,
                           size_t out_dim, size_t in_dim, size_t s) {
    if (!c || !w_bytes || (s && (!x || !y))) return ULLM_ERR_INVALID;
    int fmt = fmt_of(dtype);
    if (fmt != FMT_Q4K && fmt != FMT_Q6K) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA kernel for dtype %d yet", dtype);
    if (const char *m = matvec_shape_error(fmt, out_dim, in_dim, 0)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    size_t need = weight_bytes(fmt, out_dim, in_dim);
    if (w_len < need) return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu weight bytes, have %zu", need, w_len);
    if (s == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    void *d_w = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, need, &d_w))) return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_w, w_bytes, need, cudaMemcpyHostToDevice, c->stream));
    return matmul_host(c, dtype, d_w, nullptr, nullptr, 0, 0, x, y, out_dim, in_dim, s);
}

int ullm_cuda_matmul_mlx4(ullm_cuda_ctx *c, const void *w, const float *scales, const float *biases, const float *x,
                          float *y, size_t out_dim, size_t in_dim, size_t group, size_t s) {
    if (!c || !w || !scales || !biases || (s && (!x || !y))) return ULLM_ERR_INVALID;
    if (const char *m = matvec_shape_error(FMT_MLX4, out_dim, in_dim, group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    if (s == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    size_t wb = weight_bytes(FMT_MLX4, out_dim, in_dim), tb = out_dim * (in_dim / group) * 4;
    void *d_w = nullptr, *d_s = nullptr, *d_b = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 0, wb, &d_w)) || (rc = ctx_scratch(c, 2, tb, &d_s)) || (rc = ctx_scratch(c, 3, tb, &d_b)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_w, w, wb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_s, scales, tb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_b, biases, tb, cudaMemcpyHostToDevice, c->stream));
    return matmul_host(c, ULLM_DTYPE_MLX_U32, d_w, d_s, d_b, ULLM_DTYPE_F32, group, x, y, out_dim, in_dim, s);
}

// How the persistent matvec launch would deal `grid` CTAs out to `n` independent matrices (dtype: ULLM_DTYPE_Q4_K
// or ULLM_DTYPE_Q6_K; at most 12; n <= grid).  Host arithmetic only: needs no device, so the CPU tests can pin it.
extern "C" int ullm_cuda_debug_chain_deal(int n, const int *dtype, const size_t *out_dim, const size_t *in_dim, int grid, unsigned *ncta) {
    if (n < 1 || n > 12 || grid < n || !dtype || !out_dim || !in_dim || !ncta) return ULLM_ERR_INVALID;
    MatvecChainOp ops[12];
    for (int i = 0; i < n; ++i) {
        if (dtype[i] != ULLM_DTYPE_Q4_K && dtype[i] != ULLM_DTYPE_Q6_K) return ULLM_ERR_UNSUPPORTED;
        ops[i].fmt = dtype[i] == ULLM_DTYPE_Q4_K ? FMT_Q4K : FMT_Q6KR, ops[i].out_dim = out_dim[i], ops[i].in_dim = in_dim[i];
    }
    matvec_chain_deal(n, ops, (uint32_t)grid, ncta);
    return ULLM_OK;
}

// ---- test knobs (not part of the mirrored surface; every one is per context) ----
extern "C" int ullm_cuda_debug_set(ullm_cuda_ctx *c, const char *key, int value) {
    if (!c || !key) return ULLM_ERR_INVALID;
    if (!strcmp(key, "force_generic")) c->force_generic = value != 0;
    else if (!strcmp(key, "no_prepare")) c->no_prepare = value != 0;
    else if (!strcmp(key, "gemm_min_s")) c->gemm_min_s = value;
    else if (!strcmp(key, "no_chain")) c->no_chain = value != 0;
    else if (!strcmp(key, "shard_no_tagged")) c->shard_no_tagged = value != 0;
    else if (!strcmp(key, "shard_gemm_exchange")) c->shard_gemm_exchange = value;
    else if (!strcmp(key, "q6k_cost_permille")) matvec_chain_set_q6k_cost(value / 1000.0);
    else if (!strcmp(key, "chain_prefetch_tiles")) matvec_chain_set_prefetch(value);
    else if (!strcmp(key, "chain_chunk")) matvec_chain_set_chunk(value);
    else if (!strcmp(key, "chain_overlap_image")) matvec_chain_set_overlap(value);
    else if (!strcmp(key, "stream_chunk")) matvec_stream_set_chunk(value);
    else if (!strcmp(key, "no_host_kernels")) c->no_host_kernels = value != 0;
    else if (!strcmp(key, "plan_wr")) c->plan_wr = value;
    else if (!strcmp(key, "plan_rw")) c->plan_rw = value;
    else if (!strcmp(key, "plan_stages")) c->plan_stages = value;
    else return ULLM_ERR_INVALID;
    return ULLM_OK;
}
extern "C" int ullm_cuda_debug_last_plan(const ullm_cuda_ctx *c, int *vals, int n) {
    if (!c || !vals) return ULLM_ERR_INVALID;
    const int v[6] = {c->last_plan.streamed, c->last_plan.rows_per_tile, c->last_plan.warps,
                      c->last_plan.stages,   c->last_plan.smem_bytes,    c->last_plan.grid};
    for (int i = 0; i < n && i < 6; ++i) vals[i] = v[i];
    return ULLM_OK;
}

// ---- mixture of experts ------------------------------------------------------
struct ullm_cuda_experts {
    MoeExperts e;
    void *blob = nullptr;    // one allocation holding the nine arrays
    void *scratch = nullptr; // routing table + per-pair intermediates
};

int ullm_cuda_experts_create(ullm_cuda_ctx *c, const ullm_moe_experts_input *in, ullm_cuda_experts **out) {
    if (!c || !in || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    const void *src[9] = {in->gate_w, in->gate_scales, in->gate_biases, in->up_w,       in->up_scales,
                          in->up_biases, in->down_w,   in->down_scales, in->down_biases};
    for (auto p : src)
        if (!p) return ULLM_ERR_INVALID;
    if (in->table_dtype != ULLM_DTYPE_F32 && in->table_dtype != ULLM_DTYPE_BF16)
        return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "MLX tables must be f32 or bf16");
    MoeExperts e;
    e.table_bytes = in->table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
    e.n_experts = in->n_experts, e.hidden = in->hidden, e.inter = in->inter, e.group = in->group;
    if (const char *m = moe_shape_error(e, 1, 1)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    const size_t wb = e.n_experts * e.inter * e.hidden / 2; // same for gate, up and down
    const size_t tb = e.n_experts * e.inter * (e.hidden / e.group) * e.table_bytes;
    const size_t tbd = e.n_experts * e.hidden * (e.inter / e.group) * e.table_bytes;
    const size_t sizes[9] = {wb, tb, tb, wb, tb, tb, wb, tbd, tbd};
    size_t offs[9], total = 0;
    for (int i = 0; i < 9; ++i) {
        offs[i] = total;
        total += (sizes[i] + 255) / 256 * 256;
    }
    ullm_cuda_experts *x = new (std::nothrow) ullm_cuda_experts();
    if (!x) return ULLM_ERR_OOM;
    cudaError_t err = cudaMalloc(&x->blob, total);
    if (err == cudaSuccess) err = cudaMalloc(&x->scratch, moe_scratch_bytes(e));
    for (int i = 0; i < 9 && err == cudaSuccess; ++i)
        err = cudaMemcpyAsync((uint8_t *)x->blob + offs[i], src[i], sizes[i], cudaMemcpyHostToDevice, c->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(c->stream);
    if (err != cudaSuccess) {
        cudaGetLastError();
        ullm_cuda_experts_destroy(c, x);
        return ctx_fail(c, err == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "experts upload: %s",
                        cudaGetErrorString(err));
    }
    const uint8_t *b = (const uint8_t *)x->blob;
    e.gate_w = b + offs[0], e.gate_s = b + offs[1], e.gate_b = b + offs[2];
    e.up_w = b + offs[3], e.up_s = b + offs[4], e.up_b = b + offs[5];
    e.down_w = b + offs[6], e.down_s = b + offs[7], e.down_b = b + offs[8];
    x->e = e;
    *out = x;
    return ULLM_OK;
}

int ullm_cuda_experts_create_st(ullm_cuda_ctx *c, const ullm_st *st, const char *prefix, size_t n_experts, size_t hidden, size_t inter,
                                size_t group, ullm_cuda_experts **out) {
    if (!c || !st || !prefix || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    char msg[256] = {0};
    ullm_st_mlx_weight g, u, d;
    const std::string p(prefix);
    if (ullm_st_mlx_experts_get(st, (p + ".gate_proj").c_str(), n_experts, inter, hidden, group, n_experts, &g, msg, sizeof msg) ||
        ullm_st_mlx_experts_get(st, (p + ".up_proj").c_str(), n_experts, inter, hidden, group, n_experts, &u, msg, sizeof msg) ||
        ullm_st_mlx_experts_get(st, (p + ".down_proj").c_str(), n_experts, hidden, inter, group, n_experts, &d, msg, sizeof msg))
        return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
    ullm_moe_experts_input in;
    memset(&in, 0, sizeof in);
    in.gate_w = g.weight, in.gate_scales = g.scales, in.gate_biases = g.biases;
    in.up_w = u.weight, in.up_scales = u.scales, in.up_biases = u.biases;
    in.down_w = d.weight, in.down_scales = d.scales, in.down_biases = d.biases;
    in.table_dtype = ULLM_DTYPE_BF16, in.n_experts = n_experts, in.hidden = hidden, in.inter = inter, in.group = group;
    return ullm_cuda_experts_create(c, &in, out);
}

void ullm_cuda_experts_destroy(ullm_cuda_ctx *c, ullm_cuda_experts *x) {
    if (!x) return;
    if (c) cudaSetDevice(c->device);
    if (x->blob) cudaFree(x->blob);
    if (x->scratch) cudaFree(x->scratch);
    delete x;
}

int ullm_cuda_moe_ffn_dev(ullm_cuda_ctx *c, const ullm_cuda_experts *x, const float *d_x, const float *d_logits,
                          size_t n_tok, size_t k, float *d_y, uint32_t *d_idx, float *d_wts, void *stream) {
    if (!c || !x || !d_x || !d_logits || !d_y) return ULLM_ERR_INVALID;
    if (const char *m = moe_shape_error(x->e, n_tok, k)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    if ((uintptr_t)d_x % 16 || (uintptr_t)d_y % 4 || (uintptr_t)d_logits % 4 || (uintptr_t)d_idx % 4 || (uintptr_t)d_wts % 4)
        return ctx_fail(c, ULLM_ERR_FORMAT, "d_x must be 16-byte aligned, d_logits / d_y / d_idx / d_wts 4-byte aligned");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    int streamed = 0;
    ULLM_CUDA_TRY(c, launch_moe_ffn(c->dev, x->e, d_x, d_logits, n_tok, k, d_y, d_idx, d_wts, x->scratch, c->d_status, st,
                                    c->force_generic, c->use_pdl, &streamed));
    c->last_plan = MatvecPlan();
    c->last_plan.streamed = streamed != 0;
    return ULLM_OK;
}

int ullm_cuda_moe_ffn(ullm_cuda_ctx *c, const ullm_cuda_experts *x, const float *xs, const float *logits, size_t n_tok,
                      size_t k, float *y, uint32_t *idx, float *wts) {
    if (!c || !x || !xs || !logits || !y) return ULLM_ERR_INVALID;
    if (const char *m = moe_shape_error(x->e, n_tok, k)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", m);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    const size_t xb = n_tok * x->e.hidden * 4, lb = n_tok * x->e.n_experts * 4, kb = n_tok * k * 4;
    void *d_x = nullptr, *d_l = nullptr, *d_y = nullptr, *d_i = nullptr, *d_w = nullptr;
    int rc;
    if ((rc = ctx_scratch(c, 4, xb, &d_x)) || (rc = ctx_scratch(c, 5, xb, &d_y)) || (rc = ctx_scratch(c, 6, lb, &d_l)) ||
        (rc = ctx_scratch(c, 2, kb, &d_i)) || (rc = ctx_scratch(c, 3, kb, &d_w)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_x, xs, xb, cudaMemcpyHostToDevice, c->stream));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(d_l, logits, lb, cudaMemcpyHostToDevice, c->stream));
    if ((rc = ullm_cuda_moe_ffn_dev(c, x, (const float *)d_x, (const float *)d_l, n_tok, k, (float *)d_y, (uint32_t *)d_i,
                                    (float *)d_w, nullptr)))
        return rc;
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(y, d_y, xb, cudaMemcpyDeviceToHost, c->stream));
    if (idx) ULLM_CUDA_TRY(c, cudaMemcpyAsync(idx, d_i, kb, cudaMemcpyDeviceToHost, c->stream));
    if (wts) ULLM_CUDA_TRY(c, cudaMemcpyAsync(wts, d_w, kb, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

// ---- decode step -------------------------------------------------------------
struct ullm_cuda_fwd {
    ullm_cuda_ctx *ctx = nullptr;
    Forward f;
};

static int fwd_fail(ullm_cuda_fwd *f, cudaError_t e, const char *what) {
    cudaGetLastError();
    return ctx_fail(f->ctx, e == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "%s: %s", what,
                    cudaGetErrorString(e));
}
static int fwd_status(ullm_cuda_fwd *f) {
    if (f->f.h_status && *f->f.h_status != DEV_OK) {
        *f->f.h_status = DEV_OK;
        return ctx_fail(f->ctx, ULLM_ERR_TIMEOUT, "a device-side bounded wait expired during the decode step");
    }
    return ULLM_OK;
}

int ullm_cuda_forward_create(ullm_cuda_ctx *c, const ullm_gpu_model_input *in, ullm_cuda_fwd **out) {
    if (!c || !in || !out || !in->layers || !in->final_norm) return ULLM_ERR_INVALID;
    *out = nullptr;
    const ullm_gpu_params &gp = in->params;
    // Flags no benchmark configuration uses are refused, not ignored.
    if (gp.sandwich_norm) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "sandwich norms are not built");
    if (gp.geglu) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "GeGLU is not built");
    if (gp.sliding_window) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "sliding-window attention is not built");
    if (in->mlx_table_dtype != ULLM_DTYPE_F32 && in->mlx_table_dtype != ULLM_DTYPE_BF16)
        return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "MLX tables must be f32 or bf16");
    ForwardParams P;
    P.n_embd = gp.n_embd, P.n_layer = gp.n_layer, P.n_head = gp.n_head, P.n_kv_head = gp.n_kv_head, P.head_dim = gp.head_dim;
    P.n_ff = gp.n_ff, P.n_ctx = gp.n_ctx, P.vocab = gp.vocab, P.rope_theta = gp.rope_theta, P.eps = gp.eps, P.kv_f16 = gp.kv_f16;
    P.rope_neox = gp.rope_neox != 0, P.qk_norm = gp.qk_norm != 0;
    P.n_experts = gp.n_experts, P.n_experts_used = gp.n_experts_used, P.moe_inter = gp.moe_inter;
    if (const char *m = Forward::check_params(P)) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "%s", m);
    const size_t qd = P.n_head * P.head_dim, kvd = P.n_kv_head * P.head_dim;
    auto conv = [&](const ullm_gpu_weight &w, size_t out_dim, size_t cols, HostWeight *hw, const char *name) -> int {
        if (!w.bytes || w.out != out_dim || w.cols != cols) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: expected shape [%zu, %zu]", name, out_dim, cols);
        hw->dtype = w.dtype, hw->bytes = w.bytes, hw->out = out_dim, hw->cols = cols;
        if (w.dtype == ULLM_DTYPE_MLX_U32) { // GpuWeight with mlx_scales / mlx_biases / mlx_group (forward.rs:56-64)
            if (!w.mlx_scales || !w.mlx_biases) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: MLX weights need scale and bias tables", name);
            if (const char *m = matvec_shape_error(FMT_MLX4, out_dim, cols, w.mlx_group)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: %s", name, m);
            if (w.len < out_dim * cols / 2) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: need %zu bytes, have %zu", name, out_dim * cols / 2, w.len);
            hw->scales = w.mlx_scales, hw->biases = w.mlx_biases, hw->group = w.mlx_group;
            return ULLM_OK;
        }
        if (w.mlx_scales || w.mlx_biases) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: MLX tables on a weight of dtype %d", name, w.dtype);
        if (w.dtype != ULLM_DTYPE_Q4_K && w.dtype != ULLM_DTYPE_Q6_K)
            return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "%s: no CUDA forward kernel for dtype %d", name, w.dtype); // forward.rs:376-378
        if (cols % QK_K) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: in_dim is not a multiple of the 256-element super-block", name);
        const size_t need = out_dim * (cols / QK_K) * (w.dtype == ULLM_DTYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES);
        if (w.len < need) return ctx_fail(c, ULLM_ERR_FORMAT, "%s: need %zu bytes, have %zu", name, need, w.len);
        return ULLM_OK;
    };
    HostModel hm;
    hm.mlx_table_bytes = in->mlx_table_dtype == ULLM_DTYPE_BF16 ? 2 : 4;
    std::vector<MoeExperts> experts(P.n_layer); // host-pointer descriptions, alive until init() has copied them
    int rc;
    if ((rc = conv(in->output, P.vocab, P.n_embd, &hm.output, "output"))) return rc;
    hm.final_norm = in->final_norm;
    hm.layers.resize(P.n_layer);
    for (size_t l = 0; l < P.n_layer; ++l) {
        const ullm_gpu_layer_input &li = in->layers[l];
        HostLayer &hl = hm.layers[l];
        if (!li.attn_norm || !li.ffn_norm) return ULLM_ERR_INVALID;
        hl.attn_norm = li.attn_norm, hl.ffn_norm = li.ffn_norm;
        hl.q_bias = li.q_bias, hl.k_bias = li.k_bias, hl.v_bias = li.v_bias;
        if (P.qk_norm) {
            if (!li.q_norm || !li.k_norm) return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: qk_norm is set but q_norm / k_norm are missing", l);
            hl.q_norm = li.q_norm, hl.k_norm = li.k_norm;
        } else if (li.q_norm || li.k_norm) {
            return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: q_norm / k_norm given but params.qk_norm is not set", l);
        }
        if ((rc = conv(li.wq, qd, P.n_embd, &hl.wq, "wq")) || (rc = conv(li.wk, kvd, P.n_embd, &hl.wk, "wk")) ||
            (rc = conv(li.wv, kvd, P.n_embd, &hl.wv, "wv")) || (rc = conv(li.wo, P.n_embd, qd, &hl.wo, "wo")))
            return rc;
        if (li.experts) {
            const ullm_moe_experts_input &xi = *li.experts;
            if (!P.n_experts) return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: experts given but params.n_experts is 0", l);
            if (xi.n_experts != P.n_experts || xi.hidden != P.n_embd || xi.inter != P.moe_inter)
                return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: experts are not %zu x [%zu, %zu]", l, P.n_experts, P.moe_inter, P.n_embd);
            if (xi.table_dtype != ULLM_DTYPE_F32 && xi.table_dtype != ULLM_DTYPE_BF16) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "MLX tables must be f32 or bf16");
            const void *ptrs[9] = {xi.gate_w, xi.gate_scales, xi.gate_biases, xi.up_w, xi.up_scales, xi.up_biases, xi.down_w, xi.down_scales, xi.down_biases};
            for (auto q : ptrs)
                if (!q) return ULLM_ERR_INVALID;
            MoeExperts &e = experts[l];
            e.gate_w = xi.gate_w, e.gate_s = xi.gate_scales, e.gate_b = xi.gate_biases, e.up_w = xi.up_w, e.up_s = xi.up_scales, e.up_b = xi.up_biases;
            e.down_w = xi.down_w, e.down_s = xi.down_scales, e.down_b = xi.down_biases;
            e.table_bytes = xi.table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
            e.n_experts = xi.n_experts, e.hidden = xi.hidden, e.inter = xi.inter, e.group = xi.group;
            if (const char *m = moe_shape_error(e, 1, P.n_experts_used)) return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: %s", l, m);
            if ((rc = conv(li.moe_gate, P.n_experts, P.n_embd, &hl.moe_gate, "moe_gate"))) return rc;
            hl.experts = &e;
            continue;
        }
        if (!P.n_ff) return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: neither experts nor a dense FFN (n_ff is 0)", l);
        if ((rc = conv(li.w_gate, P.n_ff, P.n_embd, &hl.w_gate, "w_gate")) ||
            (rc = conv(li.w_up, P.n_ff, P.n_embd, &hl.w_up, "w_up")) ||
            (rc = conv(li.w_down, P.n_embd, P.n_ff, &hl.w_down, "w_down")))
            return rc;
        if (hl.w_gate.dtype == ULLM_DTYPE_MLX_U32 || hl.w_up.dtype == ULLM_DTYPE_MLX_U32 || hl.w_down.dtype == ULLM_DTYPE_MLX_U32)
            return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "layer %zu: a dense FFN of MLX 4-bit matrices is not built", l);
    }
    ullm_cuda_fwd *f = new (std::nothrow) ullm_cuda_fwd();
    if (!f) return ULLM_ERR_OOM;
    f->ctx = c;
    f->f.use_pdl = !c->force_generic; // programmatic dependent launch between the kernels of a step
    cudaError_t e = f->f.init(c->dev, c->device, P, hm);
    if (e != cudaSuccess) {
        int code = fwd_fail(f, e, "uploading the model");
        delete f;
        return code;
    }
    *out = f;
    return ULLM_OK;
}

int ullm_cuda_forward_create_st(ullm_cuda_ctx *c, const ullm_st *st, int kv_f16, ullm_cuda_fwd **out) {
    if (!c || !st || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    char msg[256] = {0};
    ullm_st_mlx_params mp;
    int rc = ullm_st_mlx_params_get(st, &mp, msg, sizeof msg);
    if (rc == ULLM_ST_ERR_UNSUPPORTED) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "%s", msg);
    if (rc) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
    const size_t qd = mp.n_head * mp.head_dim, kvd = mp.n_kv_head * mp.head_dim, gs = (size_t)mp.group;
    // read_bf16 (mlx.rs:14-24): a bf16 vector widened to f32
    std::vector<std::vector<float>> norms;
    norms.reserve(4 * mp.n_layer + 1);
    auto norm = [&](const std::string &name, size_t n, const float **dst) -> int {
        ullm_st_tensor t;
        if (ullm_st_tensor_find(st, name.c_str(), &t)) return ctx_fail(c, ULLM_ERR_FORMAT, "missing tensor '%s'", name.c_str());
        if (t.dtype != ULLM_DTYPE_BF16 || !t.data || t.nbytes != n * 2)
            return ctx_fail(c, ULLM_ERR_FORMAT, "tensor '%s' is not %zu bf16 values", name.c_str(), n);
        norms.emplace_back(n);
        for (size_t i = 0; i < n; ++i) {
            const uint32_t b = (uint32_t)((const uint16_t *)t.data)[i] << 16;
            memcpy(&norms.back()[i], &b, 4);
        }
        *dst = norms.back().data();
        return ULLM_OK;
    };
    auto weight = [&](const std::string &name, size_t out_dim, size_t cols, ullm_gpu_weight *w) -> int {
        ullm_st_mlx_weight mw;
        if (ullm_st_mlx_weight_get(st, name.c_str(), gs, &mw, msg, sizeof msg)) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
        if (mw.out != out_dim || mw.in != cols) return ctx_fail(c, ULLM_ERR_FORMAT, "'%s' is not [%zu, %zu]", name.c_str(), out_dim, cols);
        memset(w, 0, sizeof *w);
        w->dtype = ULLM_DTYPE_MLX_U32, w->bytes = mw.weight, w->len = out_dim * cols / 2, w->out = out_dim, w->cols = cols;
        w->mlx_scales = (const float *)mw.scales, w->mlx_biases = (const float *)mw.biases, w->mlx_group = gs; // bf16 bits: mlx_table_dtype below
        return ULLM_OK;
    };
    std::vector<ullm_gpu_layer_input> layers(mp.n_layer);
    std::vector<ullm_moe_experts_input> experts(mp.n_layer);
    for (size_t i = 0; i < mp.n_layer; ++i) {
        const std::string p = "model.layers." + std::to_string(i);
        ullm_gpu_layer_input &l = layers[i];
        memset(&l, 0, sizeof l);
        if ((rc = norm(p + ".input_layernorm.weight", mp.n_embd, &l.attn_norm)) ||
            (rc = norm(p + ".post_attention_layernorm.weight", mp.n_embd, &l.ffn_norm)) ||
            (rc = norm(p + ".self_attn.q_norm.weight", mp.head_dim, &l.q_norm)) || (rc = norm(p + ".self_attn.k_norm.weight", mp.head_dim, &l.k_norm)) ||
            (rc = weight(p + ".self_attn.q_proj", qd, mp.n_embd, &l.wq)) || (rc = weight(p + ".self_attn.k_proj", kvd, mp.n_embd, &l.wk)) ||
            (rc = weight(p + ".self_attn.v_proj", kvd, mp.n_embd, &l.wv)) || (rc = weight(p + ".self_attn.o_proj", mp.n_embd, qd, &l.wo)) ||
            (rc = weight(p + ".mlp.gate", mp.n_experts, mp.n_embd, &l.moe_gate)))
            return rc;
        ullm_moe_experts_input &x = experts[i];
        memset(&x, 0, sizeof x);
        ullm_st_mlx_weight g, u, d;
        const std::string sw = p + ".mlp.switch_mlp";
        if (ullm_st_mlx_experts_get(st, (sw + ".gate_proj").c_str(), mp.n_experts, mp.moe_inter, mp.n_embd, gs, mp.n_experts, &g, msg, sizeof msg) ||
            ullm_st_mlx_experts_get(st, (sw + ".up_proj").c_str(), mp.n_experts, mp.moe_inter, mp.n_embd, gs, mp.n_experts, &u, msg, sizeof msg) ||
            ullm_st_mlx_experts_get(st, (sw + ".down_proj").c_str(), mp.n_experts, mp.n_embd, mp.moe_inter, gs, mp.n_experts, &d, msg, sizeof msg))
            return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
        x.gate_w = g.weight, x.gate_scales = g.scales, x.gate_biases = g.biases, x.up_w = u.weight, x.up_scales = u.scales, x.up_biases = u.biases;
        x.down_w = d.weight, x.down_scales = d.scales, x.down_biases = d.biases;
        x.table_dtype = ULLM_DTYPE_BF16, x.n_experts = mp.n_experts, x.hidden = mp.n_embd, x.inter = mp.moe_inter, x.group = gs;
        l.experts = &x;
    }
    ullm_gpu_model_input in;
    memset(&in, 0, sizeof in);
    ullm_gpu_params &gp = in.params;
    gp.n_embd = mp.n_embd, gp.n_layer = mp.n_layer, gp.n_head = mp.n_head, gp.n_kv_head = mp.n_kv_head, gp.head_dim = mp.head_dim;
    gp.n_ff = 0, gp.n_ctx = mp.n_ctx, gp.vocab = mp.vocab, gp.rope_theta = mp.rope_theta, gp.eps = mp.eps, gp.kv_f16 = kv_f16 ? 1 : 0;
    gp.rope_neox = 1, gp.qk_norm = 1; // mlx.rs:228, :197-198
    gp.n_experts = mp.n_experts, gp.n_experts_used = mp.n_experts_used, gp.moe_inter = mp.moe_inter;
    if ((rc = norm("model.norm.weight", mp.n_embd, &in.final_norm)) || (rc = weight("lm_head", mp.vocab, mp.n_embd, &in.output))) return rc;
    in.layers = layers.data();
    in.mlx_table_dtype = ULLM_DTYPE_BF16;
    return ullm_cuda_forward_create(c, &in, out);
}

void ullm_cuda_forward_destroy(ullm_cuda_fwd *f) { delete f; }

int ullm_cuda_forward(ullm_cuda_fwd *f, const float *x_init, size_t pos, float *logits) {
    if (!f || !x_init || !logits) return ULLM_ERR_INVALID;
    if (pos >= f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "position %zu is outside the context of %zu", pos, f->f.P.n_ctx);
    cudaError_t e = f->f.forward(x_init, pos, logits);
    if (e == cudaErrorNotSupported) return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "a layer shape is outside the fused decode path");
    if (e != cudaSuccess) return fwd_fail(f, e, "decode step");
    return fwd_status(f);
}

int ullm_cuda_forward_debug(ullm_cuda_fwd *f, const float *x_init, size_t pos, ullm_debug_stat *out, size_t cap, size_t *n_out) {
    if (!f || !x_init || !out || !n_out) return ULLM_ERR_INVALID;
    *n_out = 0;
    if (pos >= f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "position %zu is outside the context of %zu", pos, f->f.P.n_ctx);
    static_assert(sizeof(ullm_debug_stat) == sizeof(DebugStat), "debug record layout");
    cudaError_t e = f->f.debug_layer0(x_init, pos, (DebugStat *)out, cap, n_out);
    if (e == cudaErrorNotSupported) return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "forward_debug walks a dense layer 0 only");
    if (e == cudaErrorInvalidValue) return ctx_fail(f->ctx, ULLM_ERR_INVALID, "room for %zu entries is not enough", cap);
    if (e != cudaSuccess) return fwd_fail(f, e, "forward_debug");
    return fwd_status(f);
}

int ullm_cuda_forward_set_kv(ullm_cuda_fwd *f, size_t pos0, size_t n, const float *k, const float *v) {
    if (!f || !k || !v) return ULLM_ERR_INVALID;
    if (pos0 + n > f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "positions beyond the context");
    cudaError_t e = f->f.set_kv(pos0, n, k, v);
    if (e != cudaSuccess) return fwd_fail(f, e, "filling the KV cache");
    return ULLM_OK;
}

// GpuForward::supports_batched_prefill (forward.rs:744-749)
int ullm_cuda_forward_supports_batched_prefill(const ullm_cuda_fwd *f) { return f && f->f.batch_supported() ? 1 : 0; }

// GpuForward::forward_batch (forward.rs:757-909): positions 0..s-1, last token's logits
int ullm_cuda_forward_batch(ullm_cuda_fwd *f, const float *embeds, size_t s, float *logits) {
    if (!f || !embeds || !logits) return ULLM_ERR_INVALID;
    if (s == 0) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "empty prompt");
    if (s > f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "%zu prompt tokens exceed the context of %zu", s, f->f.P.n_ctx);
    if (!f->f.batch_supported()) return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "batched prefill is not available for this model's weight types");
    cudaError_t e = f->f.forward_batch(embeds, s, logits);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return ctx_fail(f->ctx, e == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "forward_batch: %s", cudaGetErrorString(e));
    }
    return fwd_status(f);
}

int ullm_cuda_forward_greedy(ullm_cuda_fwd *f, const ullm_cuda_buf *embd, int embd_dtype, uint32_t first_token, size_t pos,
                             size_t n, uint32_t *tokens_out) {
    if (!f || !embd || (n && !tokens_out)) return ULLM_ERR_INVALID;
    if (embd_dtype != ULLM_DTYPE_Q4_K && embd_dtype != ULLM_DTYPE_Q6_K)
        return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "embedding table dtype %d has no device lookup", embd_dtype);
    const size_t rb = (f->f.P.n_embd / QK_K) * (embd_dtype == ULLM_DTYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES);
    if (embd->len < f->f.P.vocab * rb) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "embedding table is shorter than vocab rows");
    if (first_token >= f->f.P.vocab) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "token id outside the vocabulary");
    if (pos + n > f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "positions beyond the context");
    cudaError_t e = f->f.greedy(embd->ptr, embd_dtype, first_token, pos, n, tokens_out);
    if (e == cudaErrorNotSupported) return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "a layer shape is outside the fused decode path");
    if (e != cudaSuccess) return fwd_fail(f, e, "greedy decode");
    return fwd_status(f);
}

int ullm_cuda_forward_greedy_weight(ullm_cuda_fwd *f, const ullm_cuda_weight *embd, uint32_t first_token, size_t pos, size_t n,
                                    uint32_t *tokens_out) {
    if (!f || !embd || (n && !tokens_out)) return ULLM_ERR_INVALID;
    if (embd->fmt != FMT_Q4K && embd->fmt != FMT_Q6K && embd->fmt != FMT_MLX4)
        return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "embedding table: rows re-ordered for the matvec kernels have no device lookup");
    if (embd->out < f->f.P.vocab || embd->cols != f->f.P.n_embd) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "embedding table is not [vocab, n_embd]");
    if (first_token >= f->f.P.vocab) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "token id outside the vocabulary");
    if (pos + n > f->f.P.n_ctx) return ctx_fail(f->ctx, ULLM_ERR_FORMAT, "positions beyond the context");
    f->f.embd_mlx.scales = embd->scales, f->f.embd_mlx.biases = embd->biases, f->f.embd_mlx.elem_bytes = embd->table_bytes, f->f.embd_mlx.group = embd->group;
    cudaError_t e = f->f.greedy(embd->w, embd->dtype, first_token, pos, n, tokens_out);
    if (e == cudaErrorNotSupported) return ctx_fail(f->ctx, ULLM_ERR_UNSUPPORTED, "a layer shape is outside the fused decode path");
    if (e != cudaSuccess) return fwd_fail(f, e, "greedy decode");
    return fwd_status(f);
}

// ---------------------------------------------------------------------------
// GpuForward straight from a GGUF file (LlamaModel::from_gguf + build_gpu,
// crates/ullm-model/src/lib.rs:174-301 and :712-805)
// ---------------------------------------------------------------------------
static float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, mant = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) bits = sign;
        else { // subnormal: mant * 2^-24 (crates/ullm-core/src/dequant.rs:20)
            float f = (float)mant * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (mant << 13);
    else bits = sign | ((exp + 112u) << 23) | (mant << 13);
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

int ullm_cuda_forward_create_gguf(ullm_cuda_ctx *c, const ullm_gguf *g, int kv_f16, ullm_cuda_fwd **out) {
    if (!c || !g || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    char msg[256] = {0};
    ullm_gguf_llama_params lp;
    int rc = ullm_gguf_llama_params_get(g, &lp, msg, sizeof msg);
    if (rc == ULLM_GGUF_ERR_UNSUPPORTED) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "%s", msg);
    if (rc) return ctx_fail(c, ULLM_ERR_FORMAT, "%s", msg);
    const size_t qd = lp.n_head * lp.head_dim, kvd = lp.n_kv_head * lp.head_dim;
    // f32 view of a norm vector (tensor_f32: F32 as is, F16 / BF16 widened)
    std::vector<std::vector<float>> norms;
    norms.reserve(7 * lp.n_layer + 1); // pointers into it are handed out: it must never reallocate
    auto norm = [&](const std::string &name, size_t n, const float **dst) -> int {
        ullm_gguf_tensor t;
        if (ullm_gguf_tensor_find(g, name.c_str(), &t)) return ctx_fail(c, ULLM_ERR_FORMAT, "missing tensor '%s'", name.c_str());
        uint64_t cnt = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) cnt *= t.shape[d];
        if (cnt != n) return ctx_fail(c, ULLM_ERR_FORMAT, "tensor '%s' has %llu elements, expected %zu", name.c_str(), (unsigned long long)cnt, n);
        norms.emplace_back(n);
        std::vector<float> &v = norms.back();
        if (t.dtype == ULLM_DTYPE_F32) memcpy(v.data(), t.data, n * 4);
        else if (t.dtype == ULLM_DTYPE_F16)
            for (size_t i = 0; i < n; ++i) v[i] = half_bits_to_float(((const uint16_t *)t.data)[i]);
        else if (t.dtype == ULLM_DTYPE_BF16)
            for (size_t i = 0; i < n; ++i) {
                const uint32_t b = (uint32_t)((const uint16_t *)t.data)[i] << 16;
                memcpy(&v[i], &b, 4);
            }
        else return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "tensor '%s': norm weights of ggml type %d", name.c_str(), t.dtype);
        *dst = v.data();
        return ULLM_OK;
    };
    auto weight = [&](const std::string &name, size_t out_dim, size_t cols, ullm_gpu_weight *w, bool optional) -> int {
        ullm_gguf_tensor t;
        if (ullm_gguf_tensor_find(g, name.c_str(), &t)) return optional ? -1 : ctx_fail(c, ULLM_ERR_FORMAT, "missing tensor '%s'", name.c_str());
        if (t.n_dims != 2 || t.shape[0] != out_dim || t.shape[1] != cols)
            return ctx_fail(c, ULLM_ERR_FORMAT, "tensor '%s' is not [%zu, %zu]", name.c_str(), out_dim, cols);
        memset(w, 0, sizeof *w);
        w->dtype = t.dtype, w->bytes = t.data, w->len = (size_t)t.nbytes, w->out = out_dim, w->cols = cols;
        return ULLM_OK;
    };
    std::vector<ullm_gpu_layer_input> layers(lp.n_layer);
    for (size_t i = 0; i < lp.n_layer; ++i) {
        const std::string b = "blk." + std::to_string(i) + ".";
        ullm_gpu_layer_input &l = layers[i];
        memset(&l, 0, sizeof l);
        if ((rc = norm(b + "attn_norm.weight", lp.n_embd, &l.attn_norm)) || (rc = norm(b + "ffn_norm.weight", lp.n_embd, &l.ffn_norm)) ||
            (rc = weight(b + "attn_q.weight", qd, lp.n_embd, &l.wq, false)) || (rc = weight(b + "attn_k.weight", kvd, lp.n_embd, &l.wk, false)) ||
            (rc = weight(b + "attn_v.weight", kvd, lp.n_embd, &l.wv, false)) || (rc = weight(b + "attn_output.weight", lp.n_embd, qd, &l.wo, false)) ||
            (rc = weight(b + "ffn_gate.weight", lp.n_ff, lp.n_embd, &l.w_gate, false)) ||
            (rc = weight(b + "ffn_up.weight", lp.n_ff, lp.n_embd, &l.w_up, false)) ||
            (rc = weight(b + "ffn_down.weight", lp.n_embd, lp.n_ff, &l.w_down, false)))
            return rc;
        // optional tensors (lib.rs:277-281: `.ok()`): Qwen2 projection biases, per-head Q/K norm weights
        auto optional = [&](const char *suffix, size_t n, const float **dst) -> int {
            ullm_gguf_tensor t;
            if (ullm_gguf_tensor_find(g, (b + suffix).c_str(), &t) != ULLM_GGUF_OK) return ULLM_OK;
            return norm(b + suffix, n, dst);
        };
        if ((rc = optional("attn_q.bias", qd, &l.q_bias)) || (rc = optional("attn_k.bias", kvd, &l.k_bias)) ||
            (rc = optional("attn_v.bias", kvd, &l.v_bias)) || (rc = optional("attn_q_norm.weight", lp.head_dim, &l.q_norm)) ||
            (rc = optional("attn_k_norm.weight", lp.head_dim, &l.k_norm)))
            return rc;
        if (!l.q_norm != !l.k_norm) return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: only one of attn_q_norm / attn_k_norm is present", i);
        if (i > 0 && !l.q_norm != !layers[0].q_norm) // qk_norm is one flag for the model (build_gpu, lib.rs:714)
            return ctx_fail(c, ULLM_ERR_FORMAT, "layer %zu: attn_q_norm present in some layers only", i);
        // tensors this backend has no kernel for are refused, not ignored
        for (const char *extra : {"post_attention_norm.weight", "post_ffw_norm.weight"}) {
            ullm_gguf_tensor t;
            if (ullm_gguf_tensor_find(g, (b + extra).c_str(), &t) == ULLM_GGUF_OK)
                return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "tensor '%s%s': sandwich norms are not built", b.c_str(), extra);
        }
    }
    ullm_gpu_model_input in;
    memset(&in, 0, sizeof in);
    in.params.n_embd = lp.n_embd, in.params.n_layer = lp.n_layer, in.params.n_head = lp.n_head, in.params.n_kv_head = lp.n_kv_head;
    in.params.head_dim = lp.head_dim, in.params.n_ff = lp.n_ff, in.params.n_ctx = lp.n_ctx, in.params.vocab = lp.vocab;
    in.params.rope_theta = lp.rope_theta, in.params.eps = lp.eps, in.params.kv_f16 = kv_f16 ? 1 : 0;
    in.params.qk_norm = lp.n_layer && layers[0].q_norm ? 1 : 0; // rope_neox stays 0: GGUF Llama / Qwen weights are permuted for interleaved RoPE (lib.rs:313-315)
    if ((rc = norm("output_norm.weight", lp.n_embd, &in.final_norm))) return rc;
    // some models tie the output projection to the input embeddings (lib.rs:303-304)
    rc = weight("output.weight", lp.vocab, lp.n_embd, &in.output, true);
    if (rc == -1) rc = weight("token_embd.weight", lp.vocab, lp.n_embd, &in.output, false);
    if (rc) return rc;
    in.layers = layers.data();
    return ullm_cuda_forward_create(c, &in, out);
}
