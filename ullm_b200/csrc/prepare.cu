// Resident-weight preparation: GGUF Q6_K rows re-ordered once, on the device, into
// a layout the streamed matvec reads with aligned 128-bit loads.
//
// A Q6_K super-block is 210 bytes (ql[128], qh[64], i8 scales[16], f16 d —
// crates/ullm-core/src/dequant.rs:255-282), so inside a row blocks are only
// 2-byte aligned, and every 6-bit value is split over a nibble of ql and two bits
// of qh.  The prepared row keeps exactly the same 210 bytes per block and exactly
// the same information (`unprepare` restores the original bytes, which the tests
// check), but per ROW of nb blocks it is three planes:
//
//   records  nb*4 x 48 B   one per (block, half nh, 16-run t'): the 16 positions
//                          l = 16t'..16t'+15 of half nh in all four groups, as
//                          three 16-byte vectors of bytes
//                             W1[l] = q_g0(l)            | hi2(g1, l) << 6
//                             W2[l] = lo4(g1, l)         | lo4(g2, l) << 4
//                             W3[l] = q_g3(l)            | hi2(g2, l) << 6
//                          (q = 6-bit value, lo4 / hi2 its low nibble / high bits;
//                          group g is the element range 128nh + 32g + l), so two of
//                          the four groups unpack with a single mask
//   scales   nb*4 x 4 B    the record's four int8 scales sc[8nh + t' + 2g], g = 0..3
//   d        nb   x 2 B    f16 super-block scale
//
// Rows stay `nb*210` bytes apart, so a matrix and any row slice of it keep their
// size and offsets.  Only defined for rows that are multiples of 16 bytes
// (in % 2048 == 0); other shapes keep the verbatim bytes and the verbatim kernel.
#include "common.cuh"
#include "kernels.h"

namespace ullm {

// one thread per record
__global__ void q6k_prepare_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t rows, uint32_t nb) {
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nrec = rows * nb * 4;
    if (gid >= nrec) return;
    const size_t row = gid / (nb * 4);
    const uint32_t ri = (uint32_t)(gid % (nb * 4)), b = ri >> 2, nh = (ri >> 1) & 1u, tp = ri & 1u;
    const uint8_t *blk = src + row * (size_t)nb * Q6K_BYTES + (size_t)b * Q6K_BYTES;
    uint8_t *orow = dst + row * (size_t)nb * Q6K_BYTES;
    const uint8_t *ql = blk + 64 * nh, *qh = blk + 128 + 32 * nh, *sc = blk + 192 + 8 * nh;
    uint8_t *rec = orow + (size_t)ri * 48;
    for (int i = 0; i < 16; ++i) {
        const int l = 16 * tp + i;
        const uint8_t a = ql[l], bb = ql[l + 32], h = qh[l];
        const uint8_t lo0 = a & 0x0F, lo1 = bb & 0x0F, lo2 = a >> 4, lo3 = bb >> 4;
        const uint8_t h0 = h & 3, h1 = (h >> 2) & 3, h2 = (h >> 4) & 3, h3 = (h >> 6) & 3;
        rec[i] = (uint8_t)(lo0 | (h0 << 4) | (h1 << 6));
        rec[16 + i] = (uint8_t)(lo1 | (lo2 << 4));
        rec[32 + i] = (uint8_t)(lo3 | (h3 << 4) | (h2 << 6));
    }
    uint8_t *scp = orow + (size_t)nb * 192 + (size_t)ri * 4;
    for (int g = 0; g < 4; ++g) scp[g] = sc[tp + 2 * g];
    if ((ri & 3u) == 0) {
        uint8_t *dp = orow + (size_t)nb * 208 + (size_t)b * 2;
        dp[0] = blk[208], dp[1] = blk[209];
    }
}

__global__ void q6k_unprepare_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t rows, uint32_t nb) {
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nrec = rows * nb * 4;
    if (gid >= nrec) return;
    const size_t row = gid / (nb * 4);
    const uint32_t ri = (uint32_t)(gid % (nb * 4)), b = ri >> 2, nh = (ri >> 1) & 1u, tp = ri & 1u;
    const uint8_t *irow = src + row * (size_t)nb * Q6K_BYTES;
    uint8_t *blk = dst + row * (size_t)nb * Q6K_BYTES + (size_t)b * Q6K_BYTES;
    const uint8_t *rec = irow + (size_t)ri * 48;
    uint8_t *ql = blk + 64 * nh, *qh = blk + 128 + 32 * nh, *sc = blk + 192 + 8 * nh;
    for (int i = 0; i < 16; ++i) {
        const int l = 16 * tp + i;
        const uint8_t w1 = rec[i], w2 = rec[16 + i], w3 = rec[32 + i];
        const uint8_t lo0 = w1 & 0x0F, h0 = (w1 >> 4) & 3, h1 = w1 >> 6;
        const uint8_t lo1 = w2 & 0x0F, lo2 = w2 >> 4;
        const uint8_t lo3 = w3 & 0x0F, h3 = (w3 >> 4) & 3, h2 = w3 >> 6;
        ql[l] = (uint8_t)(lo0 | (lo2 << 4));
        ql[l + 32] = (uint8_t)(lo1 | (lo3 << 4));
        qh[l] = (uint8_t)(h0 | (h1 << 2) | (h2 << 4) | (h3 << 6));
    }
    const uint8_t *scp = irow + (size_t)nb * 192 + (size_t)ri * 4;
    for (int g = 0; g < 4; ++g) sc[tp + 2 * g] = scp[g];
    if ((ri & 3u) == 0) {
        const uint8_t *dp = irow + (size_t)nb * 208 + (size_t)b * 2;
        blk[208] = dp[0], blk[209] = dp[1];
    }
}

bool q6k_can_prepare(size_t in_dim) { return in_dim % 2048 == 0; }

cudaError_t launch_q6k_prepare(const void *d_src, void *d_dst, size_t rows, size_t in_dim, bool inverse, cudaStream_t st) {
    if (!q6k_can_prepare(in_dim)) return cudaErrorInvalidValue;
    const uint32_t nb = (uint32_t)(in_dim / QK_K);
    const size_t nrec = rows * nb * 4;
    if (nrec == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((nrec + 255) / 256);
    if (inverse) q6k_unprepare_kernel<<<grid, 256, 0, st>>>((const uint8_t *)d_src, (uint8_t *)d_dst, rows, nb);
    else q6k_prepare_kernel<<<grid, 256, 0, st>>>((const uint8_t *)d_src, (uint8_t *)d_dst, rows, nb);
    return cudaGetLastError();
}

} // namespace ullm
