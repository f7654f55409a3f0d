// ullm_cuda_moe_ffn_noalloc: the expert-gathered MoE FFN for callers that are not
// allowed to allocate device memory.
//
// Who that is: a host program that has handed the whole GPU to its own memory
// pool (a serving framework's caching allocator, for instance), so that a
// cudaMalloc made behind its back either fails or takes memory the pool thinks it
// owns; and a latency-critical decode loop that cannot afford the implicit
// device-wide synchronisation of cudaMalloc / cudaFree in the middle of a token.
// The regular entry points allocate: `ullm_cuda_experts_create` reserves the
// routing table and the per-pair intermediates, and the host-buffer calls grow
// staging areas.  This one takes every input and output as a device pointer the
// caller already owns and keeps the kernels' scratch (routing table, hidden[pair],
// down[pair], status word) in ONE fixed array that is part of the library image.
//
// What follows from that:
//  * The array is ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES (4 MiB) on every GPU that
//    loads this library, until the process exits.  A problem whose scratch does
//    not fit is rejected with ULLM_ERR_FORMAT and a message naming both sizes.
//  * All calls share the array and it keeps what the previous call left there.
//    Nothing in it has to start at zero except the status word, which each call
//    clears on the stream before its first kernel; everything else is rewritten
//    before it is read.  Two calls whose kernels overlap on the GPU (different
//    streams, or different threads) race on the array: serialise them.
//  * The first call on a device looks up the device address of the array (and
//    sets the kernels' shared-memory attribute).  Make that first call during
//    start-up, before any stream capture begins.
//  * The call blocks: it waits for its kernels on `stream` and reads the status
//    word back before it returns (only that stream is waited for, never the whole
//    device).  The calling thread's current device is the same after the call as
//    before it.
//  * No cudaMalloc, cudaFree or allocating library routine is called on any path
//    through this function.
#include "../../include/ullm_cuda.h"
#include "common.cuh"
#include "kernels.h"

#include <cstdarg>
#include <cstdio>
#include <mutex>

using namespace ullm;

// The scratch itself.  In host code this name is only a handle for the runtime,
// not a device address: the address is fetched with cudaGetSymbolAddress below
// and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_moe_noalloc_scratch[ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
struct PerDevice {
    bool ready = false;
    unsigned char *scratch = nullptr; // device address of g_moe_noalloc_scratch on this GPU
    DeviceInfo info;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

int fail(char *err, size_t cap, int code, const char *fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return code;
}
} // namespace

extern "C" int ullm_cuda_moe_ffn_noalloc(int device, const ullm_moe_experts_input *dev_experts, const float *d_x,
                                         const float *d_logits, size_t n_tok, size_t k, float *d_y, void *stream,
                                         char *err, size_t err_cap) {
    if (err && err_cap) err[0] = 0;
    if (!dev_experts || !d_x || !d_logits || !d_y) return fail(err, err_cap, ULLM_ERR_INVALID, "null argument");
    if ((uintptr_t)d_x % 16 || (uintptr_t)d_logits % 4 || (uintptr_t)d_y % 4)
        return fail(err, err_cap, ULLM_ERR_FORMAT, "d_x must be 16-byte aligned, d_logits and d_y 4-byte aligned");
    if (device < 0 || device >= kMaxDevices) return fail(err, err_cap, ULLM_ERR_INVALID, "device index out of range");
    const ullm_moe_experts_input &in = *dev_experts;
    const void *ptrs[9] = {in.gate_w, in.gate_scales, in.gate_biases, in.up_w,       in.up_scales,
                           in.up_biases, in.down_w,   in.down_scales, in.down_biases};
    for (const void *p : ptrs) {
        if (!p) return fail(err, err_cap, ULLM_ERR_INVALID, "null expert array");
        if ((uintptr_t)p % 16) return fail(err, err_cap, ULLM_ERR_FORMAT, "expert arrays must be 16-byte aligned device pointers");
    }
    if (in.table_dtype != ULLM_DTYPE_F32 && in.table_dtype != ULLM_DTYPE_BF16)
        return fail(err, err_cap, ULLM_ERR_UNSUPPORTED, "MLX tables must be f32 or bf16");
    MoeExperts e;
    e.gate_w = in.gate_w, e.gate_s = in.gate_scales, e.gate_b = in.gate_biases;
    e.up_w = in.up_w, e.up_s = in.up_scales, e.up_b = in.up_biases;
    e.down_w = in.down_w, e.down_s = in.down_scales, e.down_b = in.down_biases;
    e.table_bytes = in.table_dtype == ULLM_DTYPE_F32 ? 4 : 2;
    e.n_experts = in.n_experts, e.hidden = in.hidden, e.inter = in.inter, e.group = in.group;
    if (const char *m = moe_shape_error(e, n_tok, k)) return fail(err, err_cap, ULLM_ERR_FORMAT, "%s", m);
    // the first 256 bytes hold the status word, the kernels' scratch follows
    const size_t need = 256 + moe_scratch_bytes(e);
    if (need > ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES)
        return fail(err, err_cap, ULLM_ERR_FORMAT,
                    "this problem needs %zu bytes of scratch, the built-in array holds %u: use ullm_cuda_moe_ffn_dev", need,
                    (unsigned)ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES);

    // the caller's current device is put back on every way out
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() {
            if (prev >= 0) cudaSetDevice(prev);
        }
    } guard;
    if (cudaGetDevice(&guard.prev) != cudaSuccess) {
        cudaGetLastError();
        guard.prev = -1;
    }
    cudaError_t ce = cudaSetDevice(device);
    if (ce != cudaSuccess) return fail(err, err_cap, ULLM_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(ce));
    PerDevice &pd = g_dev[device];
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!pd.ready) { // once per device, with that device current
            void *p = nullptr;
            ce = cudaGetSymbolAddress(&p, g_moe_noalloc_scratch);
            if (ce != cudaSuccess || !p) {
                cudaGetLastError();
                return fail(err, err_cap, ULLM_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(ce));
            }
            cudaDeviceProp prop;
            ce = cudaGetDeviceProperties(&prop, device);
            if (ce != cudaSuccess) return fail(err, err_cap, ULLM_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(ce));
            if (prop.major != 10) return fail(err, err_cap, ULLM_ERR_UNSUPPORTED, "the kernels are built for sm_100a only");
            pd.scratch = (unsigned char *)p;
            pd.info.sm_count = prop.multiProcessorCount;
            pd.info.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
            pd.info.max_smem_sm = (int)prop.sharedMemPerMultiprocessor;
            pd.ready = true;
        }
    }
    cudaStream_t st = (cudaStream_t)stream;
    int *d_status = (int *)pd.scratch;
    ce = cudaMemsetAsync(d_status, 0, sizeof(int), st); // the one word that must start at zero
    if (ce != cudaSuccess) return fail(err, err_cap, ULLM_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(ce));
    ce = launch_moe_ffn(pd.info, e, d_x, d_logits, n_tok, k, d_y, nullptr, nullptr, pd.scratch + 256, d_status, st,
                        /*force_generic=*/false, /*pdl=*/false, nullptr);
    if (ce != cudaSuccess) {
        cudaGetLastError();
        return fail(err, err_cap, ULLM_ERR_CUDA, "launch: %s", cudaGetErrorString(ce));
    }
    // Blocks like the other host-facing calls, then reports a kernel that gave up on
    // a bounded wait.  The status word is copied on the same stream into a stack
    // variable (no allocation), so only this stream is waited for.
    int status = 0;
    ce = cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
    if (ce != cudaSuccess) return fail(err, err_cap, ULLM_ERR_CUDA, "synchronize: %s", cudaGetErrorString(ce));
    if (status != DEV_OK) return fail(err, err_cap, ULLM_ERR_TIMEOUT, "a device-side bounded wait expired");
    return ULLM_OK;
}
