// Row-sharded matrices over the GPUs of one node (ullm_cuda_shard_*, include/ullm_cuda.h).
//
// The split is the reference's own: output rows are independent (crates/ullm-model/src/math.rs:11-21)
// and a row is a self-contained byte range (math.rs:29-31).  Each rank keeps out/N rows of a matrix,
// computes them with the ordinary kernels, and the kernels' epilogues store the results into every
// rank's gather buffer through peer mappings (plain st.global over NVLink, nothing is read from a
// peer); a step number published to every rank's control block, and a bounded wait on the ranks'
// numbers, replace the all-gather.  Host side here: the group object, the exchange of buffer
// addresses (CUDA IPC handles between processes, direct pointers inside one process), the small
// publish / wait / copy kernels for paths without a fused epilogue, and an NCCL all-gather as the
// comparison arm (libnccl loaded at run time).
#include "../../include/ullm_cuda.h"
#include "engine.h"
#include "host_copy.cuh"
#include "shard_dev.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

using namespace ullm;

// ---------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------
namespace ullm {

__global__ void shard_signal_kernel(const ShardDev sh, int *status) {
    pdl_wait_prior();
    if (threadIdx.x == 0 && !shard_publish(sh)) *(volatile int *)status = DEV_TIMEOUT;
}

__global__ void shard_wait_kernel(const ShardDev sh, int *status) {
    pdl_wait_prior();
    if (threadIdx.x == 0) {
        const unsigned step = *(volatile unsigned *)(sh.ctl + SHARD_CTL_STEP);
        if (!shard_wait_all(sh, step)) *(volatile int *)status = DEV_TIMEOUT;
    }
}

constexpr int SCATTER_MAX_REGIONS = 16;
struct ScatterParams {
    ShardDev sh;
    int n;
    ShardRegion reg[SCATTER_MAX_REGIONS];
    int *status;
};
// Every CTA copies a share of every region from this rank's buffer into the other ranks'; float4
// where source, destination and row length allow it.  The last CTA to finish publishes.
__global__ void __launch_bounds__(256) shard_scatter_kernel(const __grid_constant__ ScatterParams p) {
    pdl_wait_prior();
    const size_t nthr = (size_t)gridDim.x * blockDim.x, gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int i = 0; i < p.n; ++i) {
        const ShardRegion &g = p.reg[i];
        const bool vec = ((uintptr_t)g.ptr % 16 == 0) && (g.width % 4 == 0) && (g.stride % 4 == 0);
        if (vec) {
            const size_t w4 = g.width / 4, total = w4 * g.height;
            for (size_t e = gtid; e < total; e += nthr) {
                const size_t row = e / w4, col = e % w4;
                float4 *src = (float4 *)(g.ptr + row * g.stride) + col;
                const float4 v = *src;
                for (int r = 0; r < p.sh.world; ++r)
                    if (r != p.sh.rank) *(float4 *)((char *)src + p.sh.delta[r]) = v;
            }
        } else {
            const size_t total = (size_t)g.width * g.height;
            for (size_t e = gtid; e < total; e += nthr) {
                float *src = g.ptr + (e / g.width) * g.stride + e % g.width;
                const float v = *src;
                for (int r = 0; r < p.sh.world; ++r)
                    if (r != p.sh.rank) *(float *)((char *)src + p.sh.delta[r]) = v;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && !shard_cta_done(p.sh, false)) *(volatile int *)p.status = DEV_TIMEOUT;
}

static cudaError_t launch_small(const void *fn, dim3 grid, dim3 block, void **args, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

cudaError_t launch_shard_signal(const ShardDev &sh, int *d_status, cudaStream_t st) {
    void *args[2] = {(void *)&sh, (void *)&d_status};
    return launch_small((const void *)shard_signal_kernel, dim3(1), dim3(32), args, st, false);
}
cudaError_t launch_shard_wait(const ShardDev &sh, int *d_status, cudaStream_t st) {
    void *args[2] = {(void *)&sh, (void *)&d_status};
    return launch_small((const void *)shard_wait_kernel, dim3(1), dim3(32), args, st, false);
}
cudaError_t launch_shard_scatter(const DeviceInfo &dev, const ShardDev &sh, int n, const ShardRegion *regions, int *d_status,
                                 cudaStream_t st) {
    if (n < 0 || n > SCATTER_MAX_REGIONS) return cudaErrorInvalidValue;
    ScatterParams p;
    p.sh = sh, p.n = n, p.status = d_status;
    size_t floats = 0;
    for (int i = 0; i < n; ++i) p.reg[i] = regions[i], floats += (size_t)regions[i].width * regions[i].height;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>((size_t)dev.sm_count * 4, (floats / 4 + 255) / 256));
    void *args[1] = {(void *)&p};
    return launch_small((const void *)shard_scatter_kernel, dim3(grid), dim3(256), args, st, false);
}

} // namespace ullm

// ---------------------------------------------------------------------------
// NCCL, loaded at run time (comparison arm and asynchronous-error polling)
// ---------------------------------------------------------------------------
namespace {
struct NcclId128 { // ncclUniqueId: 128 opaque bytes, passed by value
    char b[128];
};
struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, NcclId128, int) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*CommGetAsyncError)(void *, int *) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*CommAbort)(void *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;
const NcclApi &nccl_api() {
    std::call_once(g_nccl_once, [] {
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            g_nccl.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (g_nccl.lib) break;
        }
        if (!g_nccl.lib) return;
        auto sym = [&](const char *n) { return dlsym(g_nccl.lib, n); };
        *(void **)&g_nccl.GetUniqueId = sym("ncclGetUniqueId");
        *(void **)&g_nccl.CommInitRank = sym("ncclCommInitRank");
        *(void **)&g_nccl.AllGather = sym("ncclAllGather");
        *(void **)&g_nccl.CommGetAsyncError = sym("ncclCommGetAsyncError");
        *(void **)&g_nccl.CommDestroy = sym("ncclCommDestroy");
        *(void **)&g_nccl.CommAbort = sym("ncclCommAbort");
        *(void **)&g_nccl.GetErrorString = sym("ncclGetErrorString");
        g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllGather && g_nccl.CommGetAsyncError && g_nccl.CommDestroy &&
                    g_nccl.GetErrorString;
    });
    return g_nccl;
}
constexpr int kNcclFloat = 7; // ncclFloat32
} // namespace

// ---------------------------------------------------------------------------
// the group object
// ---------------------------------------------------------------------------
struct ullm_cuda_shard {
    ullm_cuda_ctx *ctx = nullptr;
    int world = 0, rank = 0;
    void *base = nullptr; // [control block SHARD_CTL_BYTES][y_floats floats][pair area: 2 x y_floats pairs, when pair_bytes]
    size_t y_floats = 0;
    size_t pair_bytes = 0; // 0: no pair area (gather buffers beyond kPairMaxFloats, i.e. prefill-sized ones)
    void *peer_base[SHARD_MAX_RANKS] = {};
    bool peer_ipc[SHARD_MAX_RANKS] = {}; // opened with cudaIpcOpenMemHandle: closed on destroy
    bool connected = false;
    ShardDev dev;
    void *nccl_comm = nullptr;
    // the prefill form pushes finished blocks to the peers with the copy engines on a stream of its own, so that
    // the transfer of one matrix' block overlaps the next matrix' GEMM
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // one more stream per peer, made at the first use: the copies to different peers go over different links and
    // can use different copy engines, so they are issued side by side and meet again on copy_stream
    cudaStream_t peer_stream[SHARD_MAX_RANKS] = {};
    cudaEvent_t ev_peer[SHARD_MAX_RANKS] = {};
    bool copies_pending = false; // copy_stream has work the compute stream has not been joined with
};

static float *shard_y(const ullm_cuda_shard *s) { return (float *)((uint8_t *)s->base + SHARD_CTL_BYTES); }
static size_t shard_y_bytes(const ullm_cuda_shard *s) { return (s->y_floats * 4 + 255) & ~(size_t)255; }
// The tagged exchange of the batch-1 form needs 16 bytes of pair area per float of the gather buffer: kept to
// buffers of vector size (a prefill-sized buffer of [tokens, out] floats uses the flag protocol and copy engines).
constexpr size_t kPairMaxFloats = (size_t)1 << 22;

static void shard_wire(ullm_cuda_shard *s) {
    ShardDev &d = s->dev;
    d.world = s->world, d.rank = s->rank;
    d.ctl = (unsigned *)s->base;
    for (int r = 0; r < s->world; ++r) {
        d.delta[r] = (long long)((intptr_t)s->peer_base[r] - (intptr_t)s->base);
        d.peer_flag[r] = (unsigned *)s->peer_base[r] + s->rank * SHARD_CTL_STRIDE;
    }
    for (int r = 0; r < s->world; ++r) { // made here, outside any stream capture; a failure is retried at the first use
        if (r == s->rank || s->peer_stream[r]) continue;
        if (cudaStreamCreateWithFlags(&s->peer_stream[r], cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->ev_peer[r], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            if (s->peer_stream[r]) cudaStreamDestroy(s->peer_stream[r]);
            s->peer_stream[r] = nullptr;
        }
    }
    d.ybase = shard_y(s);
    d.pairs = s->pair_bytes ? (uint2 *)((uint8_t *)s->base + SHARD_CTL_BYTES + shard_y_bytes(s)) : nullptr;
    d.pair_floats = (unsigned)s->y_floats;
    s->connected = true;
}
static void shard_timeout(ullm_cuda_shard *s, ShardDev &d) { d.timeout_ns = (unsigned long long)s->ctx->shard_timeout_ms * 1000000ull; }

int ullm_cuda_shard_row_range(size_t out, int world, int rank, size_t *row0, size_t *rows) {
    if (world < 1 || rank < 0 || rank >= world || !row0 || !rows) return ULLM_ERR_INVALID;
    if (out % (size_t)world) return ULLM_ERR_FORMAT;
    *rows = out / (size_t)world;
    *row0 = *rows * (size_t)rank;
    return ULLM_OK;
}

int ullm_cuda_shard_create(ullm_cuda_ctx *c, int world, int rank, size_t y_floats, ullm_cuda_shard **out) {
    if (!c || !out) return ULLM_ERR_INVALID;
    *out = nullptr;
    if (world < 1 || world > SHARD_MAX_RANKS || rank < 0 || rank >= world)
        return ctx_fail(c, ULLM_ERR_INVALID, "a sharded group has 1..%d ranks and 0 <= rank < world", SHARD_MAX_RANKS);
    if (y_floats == 0) return ctx_fail(c, ULLM_ERR_INVALID, "empty gather buffer");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ullm_cuda_shard *s = new (std::nothrow) ullm_cuda_shard();
    if (!s) return ULLM_ERR_OOM;
    s->ctx = c, s->world = world, s->rank = rank, s->y_floats = y_floats;
    s->pair_bytes = y_floats <= kPairMaxFloats ? 2 * y_floats * sizeof(uint2) : 0;
    const size_t bytes = SHARD_CTL_BYTES + shard_y_bytes(s) + s->pair_bytes;
    cudaError_t e = cudaMalloc(&s->base, bytes);
    if (e == cudaSuccess) e = cudaMemset(s->base, 0, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (s->base) cudaFree(s->base);
        delete s;
        return ctx_fail(c, e == cudaErrorMemoryAllocation ? ULLM_ERR_OOM : ULLM_ERR_CUDA, "gather buffer: %s", cudaGetErrorString(e));
    }
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->ev_join, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        cudaGetLastError();
        ullm_cuda_shard_destroy(s);
        return ctx_fail(c, ULLM_ERR_CUDA, "copy stream: %s", cudaGetErrorString(e));
    }
    s->peer_base[rank] = s->base;
    if (world == 1) shard_wire(s);
    *out = s;
    return ULLM_OK;
}

void ullm_cuda_shard_destroy(ullm_cuda_shard *s) {
    if (!s) return;
    cudaSetDevice(s->ctx->device);
    cudaStreamSynchronize(s->ctx->stream);
    if (s->copy_stream) {
        cudaStreamSynchronize(s->copy_stream);
        cudaStreamDestroy(s->copy_stream);
    }
    if (s->ev_fork) cudaEventDestroy(s->ev_fork);
    if (s->ev_join) cudaEventDestroy(s->ev_join);
    for (int r = 0; r < SHARD_MAX_RANKS; ++r) {
        if (s->peer_stream[r]) {
            cudaStreamSynchronize(s->peer_stream[r]);
            cudaStreamDestroy(s->peer_stream[r]);
        }
        if (s->ev_peer[r]) cudaEventDestroy(s->ev_peer[r]);
    }
    if (s->nccl_comm && nccl_api().ok) nccl_api().CommDestroy(s->nccl_comm);
    for (int r = 0; r < s->world; ++r)
        if (r != s->rank && s->peer_ipc[r] && s->peer_base[r]) cudaIpcCloseMemHandle(s->peer_base[r]);
    if (s->base) cudaFree(s->base);
    delete s;
}

float *ullm_cuda_shard_y(const ullm_cuda_shard *s) { return s ? shard_y(s) : nullptr; }

int ullm_cuda_shard_read(ullm_cuda_shard *s, size_t offset, float *host, size_t n) {
    if (!s || (!host && n)) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    if (offset > s->y_floats || n > s->y_floats - offset) return ctx_fail(c, ULLM_ERR_FORMAT, "range outside the gather buffer");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ULLM_CUDA_TRY(c, cudaMemcpyAsync(host, shard_y(s) + offset, n * 4, cudaMemcpyDeviceToHost, c->stream));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_shard_export(const ullm_cuda_shard *s, void *handle) {
    if (!s || !handle) return ULLM_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) <= ULLM_SHARD_HANDLE_BYTES, "handle size");
    ULLM_CUDA_TRY(s->ctx, cudaSetDevice(s->ctx->device));
    cudaIpcMemHandle_t h;
    ULLM_CUDA_TRY(s->ctx, cudaIpcGetMemHandle(&h, s->base));
    memset(handle, 0, ULLM_SHARD_HANDLE_BYTES);
    memcpy(handle, &h, sizeof h);
    return ULLM_OK;
}

int ullm_cuda_shard_connect(ullm_cuda_shard *s, const void *handles) {
    if (!s || !handles) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    if (s->connected && s->world > 1) return ctx_fail(c, ULLM_ERR_INVALID, "this rank is already connected");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    for (int r = 0; r < s->world; ++r) {
        if (r == s->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)r * ULLM_SHARD_HANDLE_BYTES, sizeof h);
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return ctx_fail(c, ULLM_ERR_CUDA, "opening rank %d's gather buffer: %s (the ranks must be GPUs of one node with peer access)", r,
                            cudaGetErrorString(e));
        }
        s->peer_base[r] = p, s->peer_ipc[r] = true;
    }
    shard_wire(s);
    return ULLM_OK;
}

int ullm_cuda_shard_connect_local(ullm_cuda_shard *const *shards, int world) {
    if (!shards || world < 1 || world > SHARD_MAX_RANKS) return ULLM_ERR_INVALID;
    for (int r = 0; r < world; ++r)
        if (!shards[r] || shards[r]->world != world || shards[r]->rank != r) return ULLM_ERR_INVALID;
    for (int r = 0; r < world; ++r) {
        ullm_cuda_shard *s = shards[r];
        ullm_cuda_ctx *c = s->ctx;
        ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
        for (int q = 0; q < world; ++q) {
            const int qd = shards[q]->ctx->device;
            if (q != r && qd != c->device) {
                int can = 0;
                ULLM_CUDA_TRY(c, cudaDeviceCanAccessPeer(&can, c->device, qd));
                if (!can) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "GPU %d cannot address GPU %d's memory", c->device, qd);
                cudaError_t e = cudaDeviceEnablePeerAccess(qd, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    return ctx_fail(c, ULLM_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", qd, cudaGetErrorString(e));
                cudaGetLastError();
            }
            s->peer_base[q] = shards[q]->base;
        }
        shard_wire(s);
    }
    return ULLM_OK;
}

int ullm_cuda_shard_reset(ullm_cuda_shard *s) {
    if (!s) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    ULLM_CUDA_TRY(c, cudaMemset(s->base, 0, SHARD_CTL_BYTES));
    if (s->pair_bytes) ULLM_CUDA_TRY(c, cudaMemset((uint8_t *)s->base + SHARD_CTL_BYTES + shard_y_bytes(s), 0, s->pair_bytes)); // stale tags
    *c->h_status = DEV_OK;
    return ULLM_OK;
}

int ullm_cuda_shard_weight_create(ullm_cuda_shard *s, const ullm_gpu_weight *full, int mlx_table_dtype, ullm_cuda_weight **out) {
    if (!s || !full || !out || !full->bytes) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    *out = nullptr;
    size_t row0 = 0, rows = 0;
    if (ullm_cuda_shard_row_range(full->out, s->world, s->rank, &row0, &rows))
        return ctx_fail(c, ULLM_ERR_FORMAT, "%zu rows do not split evenly over %d ranks", full->out, s->world);
    size_t row_bytes;
    switch (full->dtype) {
    case ULLM_DTYPE_Q4_K: row_bytes = full->cols / QK_K * Q4K_BYTES; break;
    case ULLM_DTYPE_Q6_K: row_bytes = full->cols / QK_K * Q6K_BYTES; break;
    case ULLM_DTYPE_MLX_U32: row_bytes = full->cols / 2; break;
    default: return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "no CUDA forward kernel for dtype %d", full->dtype);
    }
    if (full->len < full->out * row_bytes) return ctx_fail(c, ULLM_ERR_FORMAT, "need %zu weight bytes, have %zu", full->out * row_bytes, full->len);
    ullm_gpu_weight part = *full;
    part.bytes = (const uint8_t *)full->bytes + row0 * row_bytes, part.len = rows * row_bytes, part.out = rows;
    if (full->dtype == ULLM_DTYPE_MLX_U32 && full->mlx_scales && full->mlx_biases && full->mlx_group && full->cols % full->mlx_group == 0) {
        const size_t tb = (full->cols / full->mlx_group) * (mlx_table_dtype == ULLM_DTYPE_BF16 ? 2 : 4);
        part.mlx_scales = (const float *)((const uint8_t *)full->mlx_scales + row0 * tb);
        part.mlx_biases = (const float *)((const uint8_t *)full->mlx_biases + row0 * tb);
    }
    int rc = ullm_cuda_weight_create(c, &part, mlx_table_dtype, out);
    if (rc) return rc;
    (*out)->row0 = row0, (*out)->out_total = full->out;
    return ULLM_OK;
}

static int shard_ready(ullm_cuda_shard *s) {
    if (!s->connected) return ctx_fail(s->ctx, ULLM_ERR_INVALID, "the group is not connected yet (ullm_cuda_shard_connect)");
    return ULLM_OK;
}

int ullm_cuda_shard_matvec_dev(ullm_cuda_shard *s, size_t n, const ullm_shard_op *ops, int flags, void *stream) {
    if (!s || (n && !ops)) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    int rc = shard_ready(s);
    if (rc) return rc;
    if (n == 0) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    ShardDev sh = s->dev;
    shard_timeout(s, sh);
    sh.wait = (flags & ULLM_SHARD_NO_WAIT) ? 0 : 1;
    std::vector<MatvecChainOp> v(n);
    bool fused = !c->force_generic && !c->no_chain;
    // The tagged exchange: one launch that waits for the other ranks itself, every op an even split by rank.
    bool tagged = sh.wait && s->pair_bytes && n <= 12 && !c->shard_no_tagged;
    for (size_t i = 0; i < n; ++i) {
        const ullm_shard_op &o = ops[i];
        if (!o.w || !o.d_x) return ULLM_ERR_INVALID;
        if ((uintptr_t)o.d_x % 16) return ctx_fail(c, ULLM_ERR_FORMAT, "device pointers must be 16-byte aligned");
        const size_t row0 = o.w->out_total ? o.w->row0 : o.row0;
        if (o.y_offset > s->y_floats || row0 > s->y_floats - o.y_offset || o.w->out > s->y_floats - o.y_offset - row0)
            return ctx_fail(c, ULLM_ERR_FORMAT, "op %zu: rows %zu..%zu at offset %zu lie outside the gather buffer of %zu floats", i, row0,
                            row0 + o.w->out, o.y_offset, s->y_floats);
        MatvecChainOp &m = v[i];
        m.fmt = o.w->fmt, m.w = o.w->w, m.x = o.d_x, m.y = shard_y(s) + o.y_offset + row0, m.out_dim = o.w->out, m.in_dim = o.w->cols;
        m.gather_off = o.y_offset, m.gather_len = o.w->out * (size_t)s->world;
        tagged = tagged && row0 == o.w->out * (size_t)s->rank && m.gather_len <= s->y_floats - o.y_offset;
        fused = fused && matvec_chain_supported(m.fmt, m.out_dim, m.in_dim, EPI_STORE) && ((uintptr_t)m.w % 16 == 0);
    }
    if (fused) {
        unsigned *d_sync = nullptr;
        if (!c->d_sync) {
            cudaError_t e = cudaMalloc((void **)&c->d_sync, 256);
            if (e == cudaSuccess) e = cudaMemset(c->d_sync, 0, 256);
            if (e != cudaSuccess) {
                cudaGetLastError();
                c->d_sync = nullptr;
                return ctx_fail(c, ULLM_ERR_OOM, "cudaMalloc for the chain barrier failed: %s", cudaGetErrorString(e));
            }
        }
        d_sync = c->d_sync;
        size_t i = 0;
        bool fell_back = false;
        while (i < n) {
            const size_t m = std::min<size_t>(12, n - i);
            ShardDev part = sh;
            part.signal = i + m == n ? 1 : 0; // the last launch of the step publishes for all of them
            part.tagged = tagged ? 1 : 0;
            cudaError_t e = launch_matvec_chain(c->dev, (int)m, v.data() + i, d_sync, c->d_status, st, c->use_pdl, &part);
            if (e == cudaErrorNotSupported && i == 0) {
                cudaGetLastError();
                fell_back = true;
                break;
            }
            if (e != cudaSuccess) {
                cudaGetLastError();
                return ctx_fail(c, ULLM_ERR_CUDA, "sharded matvec launch: %s", cudaGetErrorString(e));
            }
            i += m;
        }
        if (!fell_back) {
            c->last_plan = MatvecPlan();
            c->last_plan.streamed = true, c->last_plan.warps = 20, c->last_plan.grid = -3; // marks the sharded chain kernel
            return ULLM_OK;
        }
    }
    // ordinary kernels into this rank's buffer, then one copy of the new rows to the peers
    std::vector<ShardRegion> regs;
    for (size_t i = 0; i < n; ++i) {
        const ullm_shard_op &o = ops[i];
        rc = ullm_cuda_weight_matvec_dev(c, o.w, o.d_x, v[i].y, st);
        if (rc) return rc;
        regs.push_back(ShardRegion{v[i].y, (unsigned)o.w->out, 1u, o.w->out});
    }
    for (size_t i = 0; i < regs.size(); i += 16) {
        const size_t m = std::min<size_t>(16, regs.size() - i);
        ShardDev part = sh;
        part.signal = i + m == regs.size() ? 1 : 0;
        ULLM_CUDA_TRY(c, launch_shard_scatter(c->dev, part, (int)m, regs.data() + i, c->d_status, st));
    }
    return ULLM_OK;
}

int ullm_cuda_shard_matvec(ullm_cuda_shard *s, size_t n, const ullm_shard_op *ops, const float *const *x_host, float *y_host, size_t y_offset,
                           size_t y_count) {
    if (!s || (n && !ops) || (y_count && !y_host)) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    if (y_offset > s->y_floats || y_count > s->y_floats - y_offset) return ctx_fail(c, ULLM_ERR_FORMAT, "result range outside the gather buffer");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    // page-locked host vectors move in one small kernel per direction (no copy-engine hand-over); others by cudaMemcpyAsync
    if (x_host) {
        VecCopyList l{};
        int m = 0;
        bool mapped = !c->no_host_kernels;
        for (size_t i = 0; i < n && mapped; ++i) {
            if (!x_host[i] || !ops[i].w || !ops[i].d_x) continue;
            const float *v = device_view_of_host(x_host[i]);
            if (!v || m == VEC_COPY_MAX) mapped = false;
            else l.src[m] = v, l.dst[m] = (float *)ops[i].d_x, l.n[m] = (unsigned)ops[i].w->cols, ++m;
        }
        if (mapped && m) {
            ULLM_CUDA_TRY(c, vec_copy_multi(l, m, c->stream, c->use_pdl));
        } else if (!mapped) {
            for (size_t i = 0; i < n; ++i)
                if (x_host[i] && ops[i].w && ops[i].d_x)
                    ULLM_CUDA_TRY(c, cudaMemcpyAsync((void *)ops[i].d_x, x_host[i], ops[i].w->cols * 4, cudaMemcpyHostToDevice, c->stream));
        }
    }
    int rc = ullm_cuda_shard_matvec_dev(s, n, ops, 0, nullptr);
    if (rc) return rc;
    if (y_count) {
        float *yv = c->no_host_kernels ? nullptr : (float *)device_view_of_host(y_host);
        if (yv && y_count <= 0xffffffffull) {
            VecCopyList l{};
            l.src[0] = shard_y(s) + y_offset, l.dst[0] = yv, l.n[0] = (unsigned)y_count;
            ULLM_CUDA_TRY(c, vec_copy_multi(l, 1, c->stream, c->use_pdl));
        } else {
            ULLM_CUDA_TRY(c, cudaMemcpyAsync(y_host, shard_y(s) + y_offset, y_count * 4, cudaMemcpyDeviceToHost, c->stream));
        }
    }
    ULLM_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    return ctx_check_status(c);
}

int ullm_cuda_shard_wait_dev(ullm_cuda_shard *s, void *stream) {
    if (!s) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    int rc = shard_ready(s);
    if (rc) return rc;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    ShardDev sh = s->dev;
    shard_timeout(s, sh);
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    if (s->copies_pending) { // blocks still on their way to the peers: their publications come first
        ULLM_CUDA_TRY(c, cudaEventRecord(s->ev_join, s->copy_stream));
        ULLM_CUDA_TRY(c, cudaStreamWaitEvent(st, s->ev_join, 0));
        s->copies_pending = false;
    }
    ULLM_CUDA_TRY(c, launch_shard_wait(sh, c->d_status, st));
    return ULLM_OK;
}

int ullm_cuda_shard_matmul_dev(ullm_cuda_shard *s, const ullm_cuda_weight *w, const float *d_x, size_t tokens, size_t y_offset, size_t row0,
                               size_t out_total, int flags, void *stream) {
    if (!s || !w || !d_x) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    int rc = shard_ready(s);
    if (rc) return rc;
    if (tokens == 0) return ULLM_OK;
    if (w->out_total) row0 = w->row0, out_total = w->out_total;
    if (row0 + w->out > out_total) return ctx_fail(c, ULLM_ERR_FORMAT, "rows %zu..%zu lie outside a matrix of %zu rows", row0, row0 + w->out, out_total);
    if (y_offset > s->y_floats || tokens > (s->y_floats - y_offset) / out_total)
        return ctx_fail(c, ULLM_ERR_FORMAT, "[%zu, %zu] at offset %zu lies outside the gather buffer of %zu floats", tokens, out_total, y_offset, s->y_floats);
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    ShardDev sh = s->dev;
    shard_timeout(s, sh);
    sh.wait = (flags & ULLM_SHARD_NO_WAIT) ? 0 : 1;
    float *y = shard_y(s) + y_offset + row0;
    if (!c->force_generic && tokens >= (size_t)c->gemm_min_s && gemm_tc_supported(w->fmt, w->out, w->cols, tokens)) {
        void *xb = nullptr;
        if ((rc = ctx_scratch(c, 7, gemm_tc_scratch_bytes(w->out, w->cols, tokens, c->dev.sm_count), &xb))) return rc;
        const bool fused = (flags & ULLM_SHARD_FUSED_STORES) != 0 || s->world == 1;
        cudaError_t e = launch_gemm_tc(w->fmt, w->w, d_x, y, xb, w->out, w->cols, tokens, c->dev.sm_count, c->d_status, st, EPI_STORE, nullptr,
                                       out_total, fused ? &sh : nullptr);
        if (e == cudaSuccess && fused) e = launch_shard_signal(sh, c->d_status, st);
        if (e == cudaSuccess && !fused) {
            // The block is complete in this rank's buffer.  The copy engines push it to the peers on the copy stream
            // (strided: `tokens` rows of `rows` floats, out_total apart), the publication follows them there, and the
            // compute stream joins only when the caller wants the step to be complete.
            e = cudaEventRecord(s->ev_fork, st);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s->copy_stream, s->ev_fork, 0);
            // Narrow blocks, or many peers: one copy kernel (the block to every peer, then the publication) - strided
            // copies of rows of a few hundred floats to seven peers kept the engines busy for longer than the GEMMs
            // of a 1/8 slice take (70B block, 512 tokens, N = 8: 965 us through one copy stream, 835 with a stream
            // per peer, 574 with the kernel; N = 4: 615 against 619).  Otherwise the copy engines, which need no SM.
            const bool push = (flags & ULLM_SHARD_SM_PUSH) || c->shard_gemm_exchange == 2 ||
                              (c->shard_gemm_exchange == 0 && (s->world > 4 || w->out * 4 < 4096));
            if (push) {
                const ShardRegion reg{y, (unsigned)w->out, (unsigned)tokens, out_total};
                if (e == cudaSuccess) e = launch_shard_scatter(c->dev, sh, 1, &reg, c->d_status, s->copy_stream);
            } else {
                for (int r = 0; r < s->world && e == cudaSuccess; ++r) {
                    if (r == s->rank) continue;
                    if (!s->peer_stream[r]) {
                        e = cudaStreamCreateWithFlags(&s->peer_stream[r], cudaStreamNonBlocking);
                        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->ev_peer[r], cudaEventDisableTiming);
                        if (e != cudaSuccess) break;
                    }
                    e = cudaStreamWaitEvent(s->peer_stream[r], s->ev_fork, 0);
                    if (e == cudaSuccess)
                        e = cudaMemcpy2DAsync((char *)y + sh.delta[r], out_total * 4, y, out_total * 4, w->out * 4, tokens, cudaMemcpyDefault,
                                              s->peer_stream[r]);
                    if (e == cudaSuccess) e = cudaEventRecord(s->ev_peer[r], s->peer_stream[r]);
                    if (e == cudaSuccess) e = cudaStreamWaitEvent(s->copy_stream, s->ev_peer[r], 0);
                }
                if (e == cudaSuccess) e = launch_shard_signal(sh, c->d_status, s->copy_stream);
            }
            s->copies_pending = true;
            if (e == cudaSuccess && sh.wait) {
                e = cudaEventRecord(s->ev_join, s->copy_stream);
                if (e == cudaSuccess) e = cudaStreamWaitEvent(st, s->ev_join, 0);
                s->copies_pending = false;
            }
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return ctx_fail(c, ULLM_ERR_CUDA, "sharded GEMM launch: %s", cudaGetErrorString(e));
        }
        c->last_plan = MatvecPlan();
        c->last_plan.streamed = true, c->last_plan.grid = -1;
        return ULLM_OK;
    }
    // per-token matvecs into this rank's buffer, then one strided copy to the peers
    for (size_t t = 0; t < tokens; ++t)
        if ((rc = ullm_cuda_weight_matvec_dev(c, w, d_x + t * w->cols, y + t * out_total, st))) return rc;
    ShardRegion reg{y, (unsigned)w->out, (unsigned)tokens, out_total};
    ULLM_CUDA_TRY(c, launch_shard_scatter(c->dev, sh, 1, &reg, c->d_status, st));
    return ULLM_OK;
}

// ---- NCCL comparison arm ------------------------------------------------------
int ullm_cuda_shard_nccl_id(void *id) {
    if (!id) return ULLM_ERR_INVALID;
    const NcclApi &a = nccl_api();
    if (!a.ok) return ULLM_ERR_UNSUPPORTED;
    return a.GetUniqueId(id) == 0 ? ULLM_OK : ULLM_ERR_CUDA;
}
int ullm_cuda_shard_nccl_init(ullm_cuda_shard *s, const void *id) {
    if (!s || !id) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    const NcclApi &a = nccl_api();
    if (!a.ok) return ctx_fail(c, ULLM_ERR_UNSUPPORTED, "libnccl.so.2 is not available");
    if (s->nccl_comm) return ULLM_OK;
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    NcclId128 uid;
    memcpy(&uid, id, sizeof uid);
    const int r = a.CommInitRank(&s->nccl_comm, s->world, uid, s->rank);
    if (r != 0) {
        s->nccl_comm = nullptr;
        return ctx_fail(c, ULLM_ERR_CUDA, "ncclCommInitRank: %s", a.GetErrorString(r));
    }
    return ULLM_OK;
}
int ullm_cuda_shard_allgather_nccl_dev(ullm_cuda_shard *s, const float *d_send, float *d_recv, size_t count, void *stream) {
    if (!s || !d_send || !d_recv) return ULLM_ERR_INVALID;
    ullm_cuda_ctx *c = s->ctx;
    if (!s->nccl_comm) return ctx_fail(c, ULLM_ERR_INVALID, "ullm_cuda_shard_nccl_init has not been called");
    ULLM_CUDA_TRY(c, cudaSetDevice(c->device));
    const NcclApi &a = nccl_api();
    const int r = a.AllGather(d_send, d_recv, count, kNcclFloat, s->nccl_comm, stream ? (cudaStream_t)stream : c->stream);
    if (r != 0) return ctx_fail(c, ULLM_ERR_CUDA, "ncclAllGather: %s", a.GetErrorString(r));
    return ULLM_OK;
}
int ullm_cuda_shard_nccl_check(ullm_cuda_shard *s) {
    if (!s) return ULLM_ERR_INVALID;
    if (!s->nccl_comm) return ULLM_OK;
    const NcclApi &a = nccl_api();
    int async_err = 0;
    const int r = a.CommGetAsyncError(s->nccl_comm, &async_err);
    if (r != 0 || async_err != 0) return ctx_fail(s->ctx, ULLM_ERR_CUDA, "NCCL communicator error: %s", a.GetErrorString(r ? r : async_err));
    return ULLM_OK;
}
