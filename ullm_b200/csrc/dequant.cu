// Bit-exact dequantization kernels (the check that the in-kernel unpack used by
// the matvec / GEMM kernels reads the formats exactly as ullm_core::dequant
// does).  Every product below is formed with an explicit round-to-nearest
// multiply and every sum with an explicit add so no FMA contraction can change
// a bit: Q4_K's `d*sc`, `(d*sc)*q` and `dmin*m` are exact in f32 and only the
// final subtraction rounds (crates/ullm-core/src/dequant.rs:203-210); Q6_K
// evaluates `(d*sc)*q` left to right (dequant.rs:275-278); MLX evaluates
// `q*scale` then `+ bias` (dequant.rs:313).
#include "common.cuh"
#include "kernels.h"

namespace ullm {

// One thread per qs byte: byte l of chunk c gives element 64c+l (low nibble)
// and 64c+32+l (high nibble)  (dequant.rs:188-217).
__global__ void dequant_q4k_kernel(const uint8_t *__restrict__ data, float *__restrict__ out, size_t nblocks,
                                   const uint32_t *__restrict__ row_sel, size_t row_bytes) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t b = gid >> 7;
    if (b >= nblocks) return;
    if (row_sel) data += (size_t)(*row_sel) * row_bytes;
    int t = (int)(gid & 127), c = t >> 5, l = t & 31;
    const uint8_t *blk = data + b * Q4K_BYTES;
    float d = f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    float dmin = f16_bits_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
    int s1, m1, s2, m2;
    scale_min_k4(2 * c, blk + 4, s1, m1);
    scale_min_k4(2 * c + 1, blk + 4, s2, m2);
    float d1 = __fmul_rn(d, (float)s1), mm1 = __fmul_rn(dmin, (float)m1);
    float d2 = __fmul_rn(d, (float)s2), mm2 = __fmul_rn(dmin, (float)m2);
    uint8_t q = blk[16 + 32 * c + l];
    float *o = out + b * QK_K + 64 * c;
    o[l] = __fsub_rn(__fmul_rn(d1, (float)(q & 0x0F)), mm1);
    o[32 + l] = __fsub_rn(__fmul_rn(d2, (float)(q >> 4)), mm2);
}

// One thread per (half nh, l): four elements l, l+32, l+64, l+96 of the half
// (dequant.rs:255-282).
__global__ void dequant_q6k_kernel(const uint8_t *__restrict__ data, float *__restrict__ out, size_t nblocks,
                                   const uint32_t *__restrict__ row_sel, size_t row_bytes) {
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t b = gid >> 6;
    if (b >= nblocks) return;
    if (row_sel) data += (size_t)(*row_sel) * row_bytes;
    int t = (int)(gid & 63), nh = t >> 5, l = t & 31, is = l >> 4;
    const uint8_t *blk = data + b * Q6K_BYTES;
    const uint8_t *ql = blk + 64 * nh, *qh = blk + 128 + 32 * nh;
    const int8_t *sc = (const int8_t *)(blk + 192) + 8 * nh;
    float d = f16_bits_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
    int h = qh[l];
    int q1 = ((ql[l] & 0x0F) | ((h & 3) << 4)) - 32;
    int q2 = ((ql[l + 32] & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
    int q3 = ((ql[l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
    int q4 = ((ql[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
    float *y = out + b * QK_K + 128 * nh;
    y[l] = __fmul_rn(__fmul_rn(d, (float)sc[is]), (float)q1);
    y[l + 32] = __fmul_rn(__fmul_rn(d, (float)sc[is + 2]), (float)q2);
    y[l + 64] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4]), (float)q3);
    y[l + 96] = __fmul_rn(__fmul_rn(d, (float)sc[is + 6]), (float)q4);
}

// One thread per packed word: eight elements, least-significant nibble first
// (dequant.rs:297-317).
__global__ void dequant_mlx4_kernel(const uint32_t *__restrict__ w, const float *__restrict__ scales,
                                    const float *__restrict__ biases, float *__restrict__ y, size_t out_dim,
                                    size_t in_dim, size_t group) {
    size_t words = in_dim / 8, groups = in_dim / group;
    size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= out_dim * words) return;
    size_t o = gid / words, wi = gid % words;
    uint32_t word = w[gid];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        size_t i = wi * 8 + n;
        size_t g = o * groups + i / group;
        float q = (float)((word >> (4 * n)) & 0xF);
        y[o * in_dim + i] = __fadd_rn(__fmul_rn(q, scales[g]), biases[g]);
    }
}

__global__ void widen_f16_kernel(const uint16_t *__restrict__ in, float *__restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f16_bits_to_f32(in[i]);
}
__global__ void widen_bf16_kernel(const uint16_t *__restrict__ in, float *__restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bf16_bits_to_f32(in[i]);
}

static inline unsigned nblk(size_t n, unsigned t) { return (unsigned)((n + t - 1) / t); }

cudaError_t launch_dequant(int dtype, const void *d_data, float *d_out, size_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    switch (dtype) {
    case 12: dequant_q4k_kernel<<<nblk(n / QK_K * 128, 256), 256, 0, st>>>((const uint8_t *)d_data, d_out, n / QK_K, nullptr, 0); break;
    case 14: dequant_q6k_kernel<<<nblk(n / QK_K * 64, 256), 256, 0, st>>>((const uint8_t *)d_data, d_out, n / QK_K, nullptr, 0); break;
    case 1: widen_f16_kernel<<<nblk(n, 256), 256, 0, st>>>((const uint16_t *)d_data, d_out, n); break;
    case 30: widen_bf16_kernel<<<nblk(n, 256), 256, 0, st>>>((const uint16_t *)d_data, d_out, n); break;
    case 0: return cudaMemcpyAsync(d_out, d_data, n * 4, cudaMemcpyDeviceToDevice, st);
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// Row `*d_row` of an MLX 4-bit table [rows, cols] -> cols f32, tables f32 or bf16 bits (dequant_mlx_row,
// crates/ullm-model/src/math.rs:68-79: q * scale + bias, product and sum rounded separately).
template <typename TBL>
__global__ void dequant_row_mlx4_kernel(const uint32_t *__restrict__ w, const TBL *__restrict__ scales, const TBL *__restrict__ biases,
                                        const uint32_t *__restrict__ d_row, size_t cols, size_t group, float *__restrict__ y) {
    const size_t words = cols / 8, wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= words) return;
    const size_t row = *d_row;
    const uint32_t word = w[row * words + wi];
    const size_t g = row * (cols / group) + wi * 8 / group; // a word never straddles a group (group % 8 == 0)
    float sc, bi;
    if (sizeof(TBL) == 2) sc = bf16_bits_to_f32((uint16_t)scales[g]), bi = bf16_bits_to_f32((uint16_t)biases[g]);
    else sc = (float)scales[g], bi = (float)biases[g];
#pragma unroll
    for (int n = 0; n < 8; ++n) y[wi * 8 + n] = __fadd_rn(__fmul_rn((float)((word >> (4 * n)) & 0xF), sc), bi);
}
cudaError_t launch_dequant_row_mlx4(const void *d_w, const void *d_scales, const void *d_biases, int tbl_bytes, size_t group,
                                    const uint32_t *d_row, size_t cols, float *d_out, cudaStream_t st) {
    if (cols % 8 || !group || group % 8 || cols % group) return cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((cols / 8 + 255) / 256);
    if (tbl_bytes == 2)
        dequant_row_mlx4_kernel<uint16_t><<<blocks, 256, 0, st>>>((const uint32_t *)d_w, (const uint16_t *)d_scales, (const uint16_t *)d_biases, d_row,
                                                                   cols, group, d_out);
    else
        dequant_row_mlx4_kernel<float><<<blocks, 256, 0, st>>>((const uint32_t *)d_w, (const float *)d_scales, (const float *)d_biases, d_row, cols,
                                                               group, d_out);
    return cudaGetLastError();
}

// Row `*d_row` of a [rows, cols] Q4_K / Q6_K table -> cols f32 (the embedding
// lookup of crates/ullm-model/src/lib.rs:692-710 with the token id on the device).
cudaError_t launch_dequant_row(int dtype, const void *d_table, const uint32_t *d_row, size_t cols, float *d_out,
                               cudaStream_t st) {
    if (cols % QK_K) return cudaErrorInvalidValue;
    size_t nb = cols / QK_K;
    static bool carved = false; // runs between streamed matvecs: keep their shared-memory carve-out
    if (!carved) {
        cudaFuncSetAttribute(dequant_q4k_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(dequant_q6k_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carved = true;
    }
    if (dtype == 12) dequant_q4k_kernel<<<nblk(nb * 128, 256), 256, 0, st>>>((const uint8_t *)d_table, d_out, nb, d_row, nb * Q4K_BYTES);
    else if (dtype == 14) dequant_q6k_kernel<<<nblk(nb * 64, 256), 256, 0, st>>>((const uint8_t *)d_table, d_out, nb, d_row, nb * Q6K_BYTES);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_dequant_mlx4(const uint32_t *d_w, const float *d_s, const float *d_b, float *d_y, size_t out_dim,
                                size_t in_dim, size_t group, cudaStream_t st) {
    size_t words = out_dim * (in_dim / 8);
    if (words == 0) return cudaSuccess;
    dequant_mlx4_kernel<<<nblk(words, 256), 256, 0, st>>>(d_w, d_s, d_b, d_y, out_dim, in_dim, group);
    return cudaGetLastError();
}

} // namespace ullm
