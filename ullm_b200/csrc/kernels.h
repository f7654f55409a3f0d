// Host-callable launchers of the CUDA kernels (internal C++ interface between
// the kernel translation units and the C ABI in api.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ullm {

struct DeviceInfo {
    int sm_count = 0;
    int max_smem_optin = 0; // bytes of dynamic shared memory a CTA may opt in to
    int max_smem_sm = 0;    // bytes of shared memory per SM
};

// Where the scale / bias tables of an MLX matrix live and how wide they are.
struct MlxTables {
    const void *scales = nullptr;
    const void *biases = nullptr;
    int elem_bytes = 4; // 4 = f32, 2 = bf16 bits
    size_t group = 0;
};

// dequant.cu
cudaError_t launch_dequant(int dtype, const void *d_data, float *d_out, size_t n, cudaStream_t st);
cudaError_t launch_dequant_row(int dtype, const void *d_table, const uint32_t *d_row, size_t cols, float *d_out,
                               cudaStream_t st);
// The same for an MLX 4-bit table (tables f32 or bf16 bits).
cudaError_t launch_dequant_row_mlx4(const void *d_w, const void *d_scales, const void *d_biases, int tbl_bytes, size_t group,
                                    const uint32_t *d_row, size_t cols, float *d_out, cudaStream_t st);
cudaError_t launch_dequant_mlx4(const uint32_t *d_w, const float *d_s, const float *d_b, float *d_y, size_t out_dim,
                                size_t in_dim, size_t group, cudaStream_t st);

// matvec.cu — y[o] = sum_i W[o,i] x[i].  fmt: 0 Q4_K, 1 Q6_K, 2 MLX4.
// `status` is a device int the kernels set to non-zero when a bounded wait
// expires.  `force_generic` selects the plain fallback kernel (tests).
struct MatvecPlan {
    bool streamed = false;
    int rows_per_tile = 0, warps = 0, stages = 0, smem_bytes = 0, grid = 0;
};
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };
struct MatvecOpts {
    bool force_generic = false;
    bool pdl = false; // launch with programmatic stream serialization
    MatvecPlan *plan_out = nullptr;
    int plan_wr = 0, plan_rw = 0, plan_stages = 0; // plan override (tests): row slices, rows per warp, ring depth; 0 = automatic
    // Fusions (streamed kernel only; cudaErrorNotSupported when the shape needs the
    // plain kernel):
    const float *norm_w = nullptr; // x <- rmsnorm(x, norm_w, eps) before the product
    float eps = 0.f;
    int epi = EPI_STORE;           // EPI_RESIDUAL: y = res + W x;  EPI_SWIGLU: rows are
                                   // interleaved (gate, up) pairs, y[j] = silu(Wx[2j]) * Wx[2j+1]
    const float *res = nullptr;
};
cudaError_t launch_matvec(const DeviceInfo &dev, int fmt, const void *d_w, const MlxTables &tb, const float *d_x,
                          float *d_y, size_t out_dim, size_t in_dim, int *d_status, cudaStream_t st,
                          const MatvecOpts &opts = MatvecOpts());
// Row-sharded output exchange (shard.cu).  Every rank of a group owns a gather buffer of the same
// layout; a rank's kernels store the rows they computed at the same offset into EVERY rank's buffer
// (plain stores through peer mappings over NVLink) and then publish a step number in every rank's
// control block; a bounded wait on the ranks' step numbers tells a rank that all rows have arrived.
constexpr int SHARD_MAX_RANKS = 8;
constexpr int SHARD_CTL_STRIDE = 32;                 // unsigned words between control words: one 128-byte line each
constexpr int SHARD_CTL_DONE = 8 * SHARD_CTL_STRIDE; // CTAs of the current launch that have stored all their rows
constexpr int SHARD_CTL_STEP = 9 * SHARD_CTL_STRIDE; // number of exchanges this rank has published
constexpr size_t SHARD_CTL_BYTES = 4096;             // control block in front of the gather buffer
struct ShardDev {
    int world = 0;                          // 0: not a sharded launch
    int rank = 0;
    long long delta[SHARD_MAX_RANKS] = {};  // bytes from an address in this rank's buffer to the same place in rank r's
    unsigned *ctl = nullptr;                // this rank's control block: word r * SHARD_CTL_STRIDE = rank r's published step
    unsigned *peer_flag[SHARD_MAX_RANKS] = {}; // this rank's word inside rank r's control block
    int signal = 1;                         // publish when the launch is done (0: a later launch of the same exchange does)
    int wait = 1;                           // ... and wait (bounded) for every rank's publication before the kernel ends
    unsigned long long timeout_ns = 2000000000ull;
    // Tagged exchange (matvec_chain_kernel, `tagged` != 0): rows travel as 8-byte {value, step} pairs into the
    // receivers' pair areas, and every rank's kernel polls the pairs it is owed and writes the values into its own
    // gather buffer - no fence, flag or second round trip between the last row and the end of the step.
    // pairs[(step & 1) * pair_floats + e] belongs to float e of the gather buffer `ybase`.
    int tagged = 0;
    float *ybase = nullptr;
    uint2 *pairs = nullptr;
    unsigned pair_floats = 0;
};
// Publishes the exchange whose rows earlier launches on `st` stored (and waits when sh.wait).
cudaError_t launch_shard_signal(const ShardDev &sh, int *d_status, cudaStream_t st);
// Waits (bounded) until every rank has published as many exchanges as this rank.
cudaError_t launch_shard_wait(const ShardDev &sh, int *d_status, cudaStream_t st);
// Copies `n` 2-D regions of this rank's buffer (first element, row length, rows, elements between rows; all in
// floats) to the same places in every other rank's buffer, then publishes (and waits when sh.wait).
struct ShardRegion {
    float *ptr;
    unsigned width, height;
    size_t stride;
};
cudaError_t launch_shard_scatter(const DeviceInfo &dev, const ShardDev &sh, int n, const ShardRegion *regions, int *d_status,
                                 cudaStream_t st);

// A list of matvecs in one persistent launch (matvec_chain.cu).  `dep` marks an op whose x or
// res was written by an earlier op of the same list.  d_sync: one zero-able unsigned in device memory.
struct MatvecChainOp {
    int fmt = 0; // FMT_Q4K or FMT_Q6KR
    const void *w = nullptr;
    const float *x = nullptr;
    float *y = nullptr;
    size_t out_dim = 0, in_dim = 0;
    const float *norm_w = nullptr;
    float eps = 0.f;
    int epi = EPI_STORE;
    const float *res = nullptr;
    bool dep = false;
    // sharded launch: [gather_off, gather_off + gather_len) is the whole vector in the gather buffer (floats), of
    // which y .. y + out_dim is this rank's part
    size_t gather_off = 0, gather_len = 0;
};
bool matvec_chain_supported(int fmt, size_t out_dim, size_t in_dim, int epi);
void matvec_chain_set_q6k_cost(double v);
void matvec_chain_deal(int n, const MatvecChainOp *ops, uint32_t grid, uint32_t *ncta); // CTAs per op of a list of independent ops
void matvec_chain_set_prefetch(int tiles);
void matvec_chain_set_chunk(int bytes);
void matvec_chain_set_overlap(int on);
void matvec_stream_set_chunk(int bytes);
// `shard` (optional): every op stores its rows into all ranks' gather buffers and the launch publishes the exchange.
cudaError_t launch_matvec_chain(const DeviceInfo &dev, int n, const MatvecChainOp *ops, unsigned *d_sync, int *d_status,
                                cudaStream_t st, bool pdl, const ShardDev *shard = nullptr);
// prepare.cu — Q6_K rows <-> the prepared layout (FMT_Q6KR)
bool q6k_can_prepare(size_t in_dim);
cudaError_t launch_q6k_prepare(const void *d_src, void *d_dst, size_t rows, size_t in_dim, bool inverse, cudaStream_t st);
// gemm.cu — tcgen05 / TMEM prefill GEMM on Q4_K (verbatim) rows, prepared Q6_K rows, or MLX 4-bit words (fmt FMT_MLX4 with `mlx`).
bool gemm_tc_supported(int fmt, size_t out_dim, size_t in_dim, size_t s);
bool gemm_tc_supported_mlx4(size_t out_dim, size_t in_dim, size_t s, const MlxTables &tb); // MLX 4-bit words, group 64, 16-byte aligned tables
size_t gemm_tc_scratch_bytes(size_t out_dim, size_t in_dim, size_t s, int sm_count); // bf16 activations + split-K partial sums
// epi / d_res: the matvec's epilogues on the [s, out] result (EPI_SWIGLU writes [s, out / 2]; d_res may alias d_y)
// ldy: elements between two tokens in d_y / d_res (0 = out_dim).  `shard` (optional, EPI_STORE only): every output element is
// stored into all ranks' gather buffers (d_y points into this rank's); the caller publishes afterwards (launch_shard_signal).
cudaError_t launch_gemm_tc(int fmt, const void *d_w, const float *d_x, float *d_y, void *d_scratch, size_t out_dim, size_t in_dim,
                           size_t s, int sm_count, int *d_status, cudaStream_t st, int epi = EPI_STORE, const float *d_res = nullptr,
                           size_t ldy = 0, const ShardDev *shard = nullptr, const MlxTables *mlx = nullptr);
bool matvec_is_streamed(const DeviceInfo &dev, int fmt, size_t out_dim, size_t in_dim, size_t group, int tbl_bytes,
                        int epi);
// Returns a static message when the shape cannot be computed at all.
const char *matvec_shape_error(int fmt, size_t out_dim, size_t in_dim, size_t group);

// moe.cu — stacked MLX 4-bit experts resident on the device.
struct MoeExperts {
    const void *gate_w = nullptr, *gate_s = nullptr, *gate_b = nullptr;
    const void *up_w = nullptr, *up_s = nullptr, *up_b = nullptr;
    const void *down_w = nullptr, *down_s = nullptr, *down_b = nullptr;
    int table_bytes = 4; // 4 = f32 tables, 2 = bf16 bits
    size_t n_experts = 0, hidden = 0, inter = 0, group = 0;
};
// Bytes of scratch (routing table + per-pair intermediates) one call needs.
size_t moe_scratch_bytes(const MoeExperts &e);
const char *moe_shape_error(const MoeExperts &e, size_t n_tok, size_t k);
// x [n_tok, hidden], logits [n_tok, n_experts] -> y [n_tok, hidden]; d_idx / d_wts
// ([n_tok, k]) may be null.  Everything is a device pointer.
cudaError_t launch_moe_ffn(const DeviceInfo &dev, const MoeExperts &e, const float *d_x, const float *d_logits,
                           size_t n_tok, size_t k, float *d_y, uint32_t *d_idx, float *d_wts, void *d_scratch,
                           int *d_status, cudaStream_t st, bool force_generic, bool pdl, int *streamed_out,
                           const float *d_res = nullptr, // [n_tok, hidden] added to the result (may alias d_y)
                           const float *d_norm_w = nullptr, float eps = 0.f); // RMSNorm of x inside the gate|up kernel (streamed path only:
                                                                               // cudaErrorNotSupported otherwise, nothing launched but the routing)

} // namespace ullm
