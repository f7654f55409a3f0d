// Moving small host vectors without the copy engines (shared by the host-buffer entry points).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <algorithm>

// A batch-1 call from host vectors is a few KB in, a few KB out and a 10-20 us kernel: the copy engines' start-up
// and the hand-overs between them and the compute engine cost as much as the kernel.  When the caller's vectors
// are page-locked (and so addressable from the device), the vectors are therefore moved by two small kernels on
// the same stream instead: one stream of compute work, no engine switch.  Pageable vectors take cudaMemcpyAsync.
static __global__ void __launch_bounds__(256) host_vec_copy_kernel(const float *__restrict__ src, float *__restrict__ dst, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0 && i + 3 < n) {
        *(float4 *)(dst + i) = *(const float4 *)(src + i);
    } else {
        for (size_t j = i; j < n && j < i + 4; ++j) dst[j] = src[j];
    }
}
// Several vectors in one launch: segment i is n[i] floats from src[i] to dst[i]; blockIdx.y picks the segment.
constexpr int VEC_COPY_MAX = 16;
struct VecCopyList {
    const float *src[VEC_COPY_MAX];
    float *dst[VEC_COPY_MAX];
    unsigned n[VEC_COPY_MAX];
};
// Launched programmatically dependent on the kernel before it, and letting the kernel after it start at once:
// between the copy-in, the matvec launch and the copy-out of a host-vector call there is then no launch gap (the
// matvec kernel's producer warps stream weights while the inputs are still on their way; its consumers wait for
// this grid with griddepcontrol.wait before they read them).
static __global__ void __launch_bounds__(256) host_vec_copy_multi_kernel(const __grid_constant__ VecCopyList l) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory"); // the kernel before this one has written what is copied
    const float *src = l.src[blockIdx.y];
    float *dst = l.dst[blockIdx.y];
    const size_t n = l.n[blockIdx.y];
    const bool vec = ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        if (vec && i + 3 < n) *(float4 *)(dst + i) = *(const float4 *)(src + i);
        else
            for (size_t j = i; j < n && j < i + 4; ++j) dst[j] = src[j];
    }
}
static cudaError_t vec_copy_multi(const VecCopyList &l, int count, cudaStream_t st, bool pdl = false) {
    unsigned most = 0;
    for (int i = 0; i < count; ++i) most = std::max(most, l.n[i]);
    const unsigned gx = std::max(1u, std::min(32u, (most + 1023) / 1024));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(gx, (unsigned)count), cfg.blockDim = dim3(256), cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, host_vec_copy_multi_kernel, l);
}
static const float *device_view_of_host(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? (const float *)a.devicePointer : nullptr;
}
static cudaError_t vec_copy(const float *src, float *dst, size_t n, cudaStream_t st) {
    host_vec_copy_kernel<<<(unsigned)((n + 1023) / 1024), 256, 0, st>>>(src, dst, n);
    return cudaGetLastError();
}

