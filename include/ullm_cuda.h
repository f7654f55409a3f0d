/*
 * ullm_cuda.h — C ABI of the B200 (sm_100a) backend for uLLM's quantized
 * matrix-product path.
 *
 * The reference has no C ABI: its GPU backend is the Rust crate `ullm-metal`,
 * used concretely by `ullm-model`.  Every entry point below replaces one method
 * of that crate's public surface (cited as file:line inside the reference
 * project); the Rust crate `crates/ullm-cuda` binds them one to one.
 *
 * Conventions
 *  - All functions return an `ullm_status`; 0 is success.  A human-readable
 *    message for the last failure on a context is kept by the context
 *    (`ullm_cuda_last_error`).  UNSUPPORTED / FORMAT map onto
 *    `ullm_core::Error::{Unsupported, Format}` (crates/ullm-core/src/error.rs:11-20).
 *  - Host pointers are borrowed for the duration of the call only; the library
 *    copies what it keeps (as `GpuForward::new` does, forward.rs:247-268).
 *  - Calls taking host buffers are synchronous (the reference commits and waits,
 *    forward.rs:513-515).  `*_dev` calls take device pointers plus a
 *    `cudaStream_t` (as `void *`; NULL = the context's own stream), only enqueue,
 *    and are the resident / graph-capturable form.
 *  - A context is bound to one CUDA device and may be moved between threads but
 *    not used concurrently (the reference's `unsafe impl Send`, forward.rs:221-225).
 *  - There is no CPU fallback: without a CUDA device `ullm_cuda_ctx_create`
 *    fails with ULLM_ERR_UNSUPPORTED ("no CUDA device available"), like
 *    `MetalContext::new` (crates/ullm-metal/src/lib.rs:31-33).
 *  - Matrices are row-major `[out, in]` in their on-disk quantized form
 *    (`QWeight`, crates/ullm-model/src/lib.rs:49-61); activations are f32,
 *    token-major `[s, in]`, outputs `[s, out]` (forward.rs:675-676).
 */
#ifndef ULLM_CUDA_H
#define ULLM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ULLM_OK = 0,
    ULLM_ERR_UNSUPPORTED = 1, /* Error::Unsupported */
    ULLM_ERR_FORMAT = 2,      /* Error::Format      */
    ULLM_ERR_CUDA = 3,        /* a CUDA runtime call failed            */
    ULLM_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up     */
    ULLM_ERR_OOM = 5,
    ULLM_ERR_INVALID = 6      /* NULL pointer / bad handle              */
} ullm_status;

/* Weight element types: ggml tensor type ids (crates/ullm-gguf/src/types.rs:7-29)
 * plus a private id for MLX packed 4-bit words (`DType::U32`, dtype.rs:27). */
typedef enum {
    ULLM_DTYPE_F32 = 0,
    ULLM_DTYPE_F16 = 1,
    ULLM_DTYPE_Q4_K = 12,
    ULLM_DTYPE_Q6_K = 14,
    ULLM_DTYPE_BF16 = 30,
    ULLM_DTYPE_MLX_U32 = 1000
} ullm_dtype;

typedef struct ullm_cuda_ctx ullm_cuda_ctx;
typedef struct ullm_cuda_buf ullm_cuda_buf;
typedef struct ullm_cuda_fwd ullm_cuda_fwd;
typedef struct ullm_cuda_experts ullm_cuda_experts;
typedef struct ullm_cuda_weight ullm_cuda_weight;

/* ---- context: MetalContext::new / device_name (ullm-metal/src/lib.rs:31, :59) ---- */
int ullm_cuda_ctx_create(int device, ullm_cuda_ctx **out);
void ullm_cuda_ctx_destroy(ullm_cuda_ctx *ctx);
const char *ullm_cuda_last_error(const ullm_cuda_ctx *ctx);
/* Per-context switches (no counterpart in the reference, whose backend has none).
 *  ULLM_OPT_PDL (default 1): the library's kernels are launched "programmatically dependent" on
 *    their predecessor in the stream, so a kernel's weight stream starts while the previous kernel
 *    drains; results are the same either way.
 *  ULLM_OPT_SHARD_TIMEOUT_MS (default 2000): how long a rank of a row-sharded group waits for the
 *    other ranks' rows before the call fails with ULLM_ERR_TIMEOUT. */
enum { ULLM_OPT_PDL = 1, ULLM_OPT_SHARD_TIMEOUT_MS = 2 };
int ullm_cuda_ctx_set_option(ullm_cuda_ctx *ctx, int option, int value);
int ullm_cuda_device_name(const ullm_cuda_ctx *ctx, char *name, size_t cap);
int ullm_cuda_sm_count(const ullm_cuda_ctx *ctx);
/* Blocks until everything enqueued on the context's stream has finished and
 * reports a device-side status (ULLM_ERR_TIMEOUT if a kernel's bounded wait
 * expired). */
int ullm_cuda_synchronize(ullm_cuda_ctx *ctx);

/* ---- resident buffers: MetalContext::upload (lib.rs:64) ---- */
int ullm_cuda_upload(ullm_cuda_ctx *ctx, const void *bytes, size_t len, ullm_cuda_buf **out);
int ullm_cuda_alloc(ullm_cuda_ctx *ctx, size_t len, ullm_cuda_buf **out);
int ullm_cuda_download(ullm_cuda_ctx *ctx, const ullm_cuda_buf *buf, size_t offset, void *host, size_t len);
void *ullm_cuda_buf_ptr(const ullm_cuda_buf *buf);
size_t ullm_cuda_buf_len(const ullm_cuda_buf *buf);
void ullm_cuda_buf_free(ullm_cuda_ctx *ctx, ullm_cuda_buf *buf);

/* ---- dequantization (bit-exact against ullm_core::dequant) ----
 * `dequantize` (dequant.rs:52-110): n elements of dtype from `data` (host) into
 * `out` (host).  FORMAT when n is not a multiple of the block size or `data_len`
 * is short (dequant.rs:65-77); UNSUPPORTED for other dtypes. */
int ullm_cuda_dequantize(ullm_cuda_ctx *ctx, int dtype, const void *data, size_t data_len, float *out, size_t n);
/* `dequantize_mlx_q4` (dequant.rs:297-317): f32 scale/bias tables. */
int ullm_cuda_dequantize_mlx4(ullm_cuda_ctx *ctx, const uint32_t *weight, const float *scales, const float *biases,
                              size_t out_dim, size_t in_dim, size_t group, float *y);

/* ---- batch-1 matvec ----
 * MetalContext::matvec_quant (lib.rs:83-94): raw GGUF block bytes on the host. */
int ullm_cuda_matvec_quant(ullm_cuda_ctx *ctx, int dtype, const void *w_bytes, size_t w_len, const float *x, float *y,
                           size_t out_dim, size_t in_dim);
/* MetalContext::matvec_resident (lib.rs:97-107): weights already uploaded. */
int ullm_cuda_matvec_resident(ullm_cuda_ctx *ctx, int dtype, const ullm_cuda_buf *w, const float *x, float *y,
                              size_t out_dim, size_t in_dim);
/* MetalContext::matvec_mlx4 (lib.rs:112-158): packed words + f32 group tables. */
int ullm_cuda_matvec_mlx4(ullm_cuda_ctx *ctx, const void *w, const float *scales, const float *biases, const float *x,
                          float *y, size_t out_dim, size_t in_dim, size_t group);
/* GpuForward::matvec (forward.rs:639-673) on device pointers.  `d_w` must be
 * 16-byte aligned.  For ULLM_DTYPE_MLX_U32 pass the tables and their element
 * type (ULLM_DTYPE_F32, or ULLM_DTYPE_BF16 for the bits as stored on disk:
 * widening bf16 is exact, dequant.rs:286); otherwise NULL/0. */
int ullm_cuda_matvec_dev(ullm_cuda_ctx *ctx, int dtype, const void *d_w, const void *d_scales, const void *d_biases,
                         int table_dtype, size_t group, const float *d_x, float *d_y, size_t out_dim, size_t in_dim,
                         void *stream);

/* ---- resident weight matrices ----
 * A weight made resident for the kernels: the `WBuf` that `GpuForward::new` builds
 * from a `GpuWeight` (forward.rs:119-126, :253-268).  The bytes are copied; Q6_K
 * rows whose length is a multiple of 16 bytes are re-ordered on the device into an
 * aligned layout of the same size (`ullm_cuda_weight_export` returns the original
 * bytes, so nothing is lost).  `w` is a `ullm_gpu_weight` (declared below); for MLX
 * weights `mlx_table_dtype` says whether `mlx_scales` / `mlx_biases` point at f32
 * values (ULLM_DTYPE_F32, as the reference passes them) or at the bf16 bits stored
 * on disk (ULLM_DTYPE_BF16, kept as such). */
struct ullm_gpu_weight_s;
int ullm_cuda_weight_create(ullm_cuda_ctx *ctx, const struct ullm_gpu_weight_s *w, int mlx_table_dtype,
                            ullm_cuda_weight **out);
void ullm_cuda_weight_destroy(ullm_cuda_ctx *ctx, ullm_cuda_weight *w);
/* GpuForward::matvec (forward.rs:639-673): y = W x, host vectors, blocking. */
int ullm_cuda_weight_matvec(ullm_cuda_ctx *ctx, const ullm_cuda_weight *w, const float *x, float *y);
/* The same on device vectors, enqueued on `stream` (NULL = the context's). */
int ullm_cuda_weight_matvec_dev(ullm_cuda_ctx *ctx, const ullm_cuda_weight *w, const float *d_x, float *d_y, void *stream);
/* `n` independent matvecs enqueued by one call (the projections of one layer that
 * share no data: q/k/v, gate/up): y[i] = W[i] x[i], device vectors. */
int ullm_cuda_weight_matvec_batch_dev(ullm_cuda_ctx *ctx, size_t n, const ullm_cuda_weight *const *w,
                                      const float *const *d_x, float *const *d_y, void *stream);
/* The same from host vectors in ONE blocking call (a layer's independent projections): copies the
 * n input vectors in, runs the n matvecs, copies the n results out and waits once.  The reference
 * makes one submission per token (forward.rs:513-515); per-matrix calls of ullm_cuda_weight_matvec
 * pay one copy-in / launch / copy-out / wait round trip each. */
int ullm_cuda_weight_matvec_batch(ullm_cuda_ctx *ctx, size_t n, const ullm_cuda_weight *const *w, const float *const *x,
                                  float *const *y);
/* A list of matvecs on resident weights run as ONE persistent launch: the weight stream
 * of op i+1 follows that of op i without a gap, and the grid synchronises only where
 * `dep` says an op consumes what an earlier op of the list produced (x or res).  With the
 * optional prologue x <- rmsnorm(x, d_norm_w, eps) (math.rs:82-86) and the epilogues
 * y = W x | y = d_res + W x | y[j] = silu((W x)[2j]) * (W x)[2j+1] (rows stored as
 * interleaved gate/up pairs; math.rs:103-105) this is the dense FFN / attention-projection
 * chain of one decode step (lib.rs:807-969).  Q4_K and prepared Q6_K weights; other
 * weights, or `no_chain` contexts, run the same ops as separate launches.  No counterpart
 * in the reference (Metal encodes one compute pass per op, forward.rs:384-526). */
enum { ULLM_EPI_STORE = 0, ULLM_EPI_RESIDUAL = 1, ULLM_EPI_SWIGLU = 2 };
typedef struct ullm_chain_op {
    const ullm_cuda_weight *w;
    const float *d_x;      /* [in] device */
    float *d_y;            /* [out] device ([out/2] for ULLM_EPI_SWIGLU) */
    const float *d_norm_w; /* NULL = no RMSNorm prologue */
    float eps;
    int epi;
    const float *d_res;    /* ULLM_EPI_RESIDUAL only; may alias d_y */
    int dep;               /* non-zero: d_x / d_res were written by an earlier op of this list */
} ullm_chain_op;
int ullm_cuda_weight_matvec_chain_dev(ullm_cuda_ctx *ctx, size_t n, const ullm_chain_op *ops, void *stream);
/* GpuForward::matmul (forward.rs:679-725) on a resident weight: x [s, in] f32
 * token-major -> y [s, out].  Prefill-sized batches (32 tokens or more) run on the tensor
 * cores (activations and dequantized weights rounded to bf16, f32 accumulation): Q4_K,
 * Q6_K with in % 2048 == 0, and MLX 4-bit with group 64; other shapes form the product
 * one token at a time with the matvec kernels. */
int ullm_cuda_weight_matmul(ullm_cuda_ctx *ctx, const ullm_cuda_weight *w, const float *x, float *y, size_t s);
int ullm_cuda_weight_matmul_dev(ullm_cuda_ctx *ctx, const ullm_cuda_weight *w, const float *d_x, float *d_y, size_t s,
                                void *stream);
/* The weight's original on-disk bytes (`len` = ullm_cuda_weight_bytes). */
int ullm_cuda_weight_export(ullm_cuda_ctx *ctx, const ullm_cuda_weight *w, void *bytes, size_t len);
size_t ullm_cuda_weight_bytes(const ullm_cuda_weight *w);
/* A resident weight made from the MLX linear `<name>.weight / .scales / .biases` of an open
 * SafeTensors model (include/ullm_safetensors.h): what mlx_qweight (crates/ullm-model/src/mlx.rs:30-56)
 * followed by build_gpu's GpuWeight (lib.rs:739-749) produces, except that the tables stay the bf16 bits
 * of the file instead of being widened to f32 on the host (widening is exact, dequant.rs:286). */
struct ullm_st;
int ullm_cuda_weight_create_st(ullm_cuda_ctx *ctx, const struct ullm_st *st, const char *name, size_t group,
                               ullm_cuda_weight **out);

/* ---- batched matmul (prefill) ----
 * GpuForward::matmul (forward.rs:679-725; kernels matmul_q4k / matmul_q6k /
 * matmul_mlx4) and MetalContext::matmul_mlx4 (lib.rs:212-266).
 * x: [s, in] f32 token-major; y: [s, out] f32. */
int ullm_cuda_matmul_quant(ullm_cuda_ctx *ctx, int dtype, const void *w_bytes, size_t w_len, const float *x, float *y,
                           size_t out_dim, size_t in_dim, size_t s);
int ullm_cuda_matmul_mlx4(ullm_cuda_ctx *ctx, const void *w, const float *scales, const float *biases, const float *x,
                          float *y, size_t out_dim, size_t in_dim, size_t group, size_t s);
int ullm_cuda_matmul_dev(ullm_cuda_ctx *ctx, int dtype, const void *d_w, const void *d_scales, const void *d_biases,
                         int table_dtype, size_t group, const float *d_x, float *d_y, size_t out_dim, size_t in_dim,
                         size_t s, void *stream);

/* ---- row-sharded matrices over the GPUs of one node ----
 * No counterpart in the reference (multi-device scale-out is an open item of its roadmap,
 * docs/roadmap.md:83).  The split is the one its CPU path already uses: output rows are
 * independent (crates/ullm-model/src/math.rs:11-21), and a row of a quantized matrix is a
 * self-contained byte range (math.rs:29-31).  Rank r of N keeps rows [r*out/N, (r+1)*out/N) of a
 * matrix; every rank has the whole input vector; the one exchange of the path is that each rank's
 * output rows must reach every rank.
 *
 * A `ullm_cuda_shard` is one rank's end of such a group: a "gather buffer" of `y_floats` floats on
 * its GPU, laid out identically on every rank, in which the caller places the full-length result
 * vectors (by offset).  The kernels of rank r store the rows they computed at the same offset into
 * EVERY rank's gather buffer (plain stores over NVLink through peer mappings; nothing is read from
 * a peer), then publish a step number to every rank; the step is complete on a rank when it has
 * seen every rank's number.  A matvec step that waits for the other ranks itself (no
 * ULLM_SHARD_NO_WAIT) sends its rows as {value, step} pairs instead, which the receiving rank's
 * kernel polls and writes into its gather buffer: the same result without the publication round
 * trips (the shard then holds 16 more bytes per float of `y_floats`, for buffers up to 4 M floats).
 * No NCCL call is involved, so a step can be captured in a CUDA graph like any other kernel.
 *
 * Set-up, one process per GPU (rank = that process' index): ullm_cuda_shard_create, exchange the
 * ULLM_SHARD_HANDLE_BYTES handles of ullm_cuda_shard_export between the processes by any means
 * (they are plain bytes), ullm_cuda_shard_connect with all N handles in rank order.  One process
 * that owns several GPUs: create one context and one shard per GPU, then
 * ullm_cuda_shard_connect_local.  All ranks must be connected before any of them runs a step.
 *
 * Rules for the caller:
 *  - Every rank must run the same sequence of sharded calls with the same flags (steps are counted
 *    per rank, and the flags select how rows travel).
 *  - A rank waits at most ULLM_OPT_SHARD_TIMEOUT_MS for the others; then the call (or the next
 *    ullm_cuda_synchronize) reports ULLM_ERR_TIMEOUT instead of hanging — this is how a dead or
 *    stalled peer shows.  After a time-out the group is out of step: every rank calls
 *    ullm_cuda_shard_reset (with a host-side barrier of the caller's before the next step).
 *  - A region of the gather buffer that step s filled may be filled again by step s+2 at the
 *    earliest, and must have been read by then (a rank can run one step ahead of a peer, not
 *    two): alternate between two regions when consecutive steps produce the same vector. */
typedef struct ullm_cuda_shard ullm_cuda_shard;
#define ULLM_SHARD_HANDLE_BYTES 64
#define ULLM_SHARD_MAX_RANKS 8
int ullm_cuda_shard_create(ullm_cuda_ctx *ctx, int world, int rank, size_t y_floats, ullm_cuda_shard **out);
void ullm_cuda_shard_destroy(ullm_cuda_shard *s);
int ullm_cuda_shard_export(const ullm_cuda_shard *s, void *handle /* ULLM_SHARD_HANDLE_BYTES */);
int ullm_cuda_shard_connect(ullm_cuda_shard *s, const void *handles /* world x ULLM_SHARD_HANDLE_BYTES, rank order */);
int ullm_cuda_shard_connect_local(ullm_cuda_shard *const *shards, int world);
int ullm_cuda_shard_reset(ullm_cuda_shard *s);
/* Device address of this rank's gather buffer (y_floats floats). */
float *ullm_cuda_shard_y(const ullm_cuda_shard *s);
/* Copies `n` floats at `offset` of this rank's gather buffer to the host.  Waits for the context's
 * own stream; a caller that ran the step on another stream synchronises that stream first. */
int ullm_cuda_shard_read(ullm_cuda_shard *s, size_t offset, float *host, size_t n);
/* Rows [*row0, *row0 + *rows) of a matrix of `out` rows that `rank` of `world` keeps; FORMAT-style
 * failure (non-zero) when `out` does not divide evenly. */
int ullm_cuda_shard_row_range(size_t out, int world, int rank, size_t *row0, size_t *rows);
/* A resident weight holding only this rank's rows of `full` (a host description of the WHOLE
 * matrix, as ullm_cuda_weight_create takes it); MLX tables are sliced with the rows. */
int ullm_cuda_shard_weight_create(ullm_cuda_shard *s, const struct ullm_gpu_weight_s *full, int mlx_table_dtype,
                                  ullm_cuda_weight **out);
/* One step of `n` sharded matvecs: for every op, y[y_offset + row0 + i] = (W_rows x)[i] in every
 * rank's gather buffer, where W_rows is this rank's slice.  `w` is either a weight made by
 * ullm_cuda_shard_weight_create (row0 is known) or any resident weight holding the slice, with
 * `row0` given here.  Q4_K and prepared Q6_K slices run as one persistent launch whose epilogue
 * stores to all ranks; other weights run the ordinary kernels followed by a copy to the peers.
 * flags: ULLM_SHARD_NO_WAIT publishes without waiting (pair with ullm_cuda_shard_wait_dev). */
typedef struct ullm_shard_op {
    const ullm_cuda_weight *w;
    const float *d_x;  /* [in] device, this rank's copy of the full input vector */
    size_t y_offset;   /* where the full-length result starts in the gather buffer (floats) */
    size_t row0;       /* first row of the slice; ignored for weights made by ullm_cuda_shard_weight_create */
} ullm_shard_op;
enum { ULLM_SHARD_NO_WAIT = 1, ULLM_SHARD_FUSED_STORES = 2, ULLM_SHARD_SM_PUSH = 4 };
int ullm_cuda_shard_matvec_dev(ullm_cuda_shard *s, size_t n, const ullm_shard_op *ops, int flags, void *stream);
/* The same step from host vectors, blocking: x_host[i] (may be NULL: the op's d_x is already filled) is
 * copied into op i's d_x, the step runs with its wait, and floats [y_offset, y_offset + y_count) of
 * this rank's gather buffer — the gathered results — are copied to y_host. */
int ullm_cuda_shard_matvec(ullm_cuda_shard *s, size_t n, const ullm_shard_op *ops, const float *const *x_host, float *y_host,
                           size_t y_offset, size_t y_count);
/* Enqueues the bounded wait for every rank's latest step. */
int ullm_cuda_shard_wait_dev(ullm_cuda_shard *s, void *stream);
/* Prefill form: this rank's [tokens, rows] block of Y = X W^T goes to columns [row0, row0 + rows)
 * of the token-major [tokens, out_total] matrix at `y_offset` in every rank's gather buffer.
 * d_x: [tokens, in] f32 on this rank.  The tensor-core GEMM writes the block into this rank's
 * buffer and the copy engines push it to the peers on a stream of the group's own, followed there
 * by the publication; with ULLM_SHARD_NO_WAIT the call returns to the caller's stream at once, so
 * the next matrix' GEMM overlaps the transfer, and the last call of a step (without the flag) or
 * ullm_cuda_shard_wait_dev joins the transfers and waits for the other ranks.  Inside a stream
 * capture a step must therefore end with such a joining call.  ULLM_SHARD_FUSED_STORES makes the
 * GEMM's epilogue store every tile to all ranks itself instead (one kernel, no copy engine);
 * at prefill sizes that is the slower form, because a tile's stores over NVLink then run in series
 * with the tile's own arithmetic.  ULLM_SHARD_SM_PUSH moves the finished block with a copy kernel
 * (vector loads, stores to every peer) on the group's stream instead of the copy engines, which the
 * library also does by itself for narrow blocks (rows of less than 4 KB) and groups of more than
 * four ranks: the engines handle such strided copies poorly, and a small slice's GEMM leaves SMs idle. */
int ullm_cuda_shard_matmul_dev(ullm_cuda_shard *s, const ullm_cuda_weight *w, const float *d_x, size_t tokens, size_t y_offset,
                               size_t row0, size_t out_total, int flags, void *stream);
/* Comparison arm: the same exchange as an NCCL all-gather (libnccl.so.2 is loaded at run time;
 * UNSUPPORTED when it is absent).  Rank 0 makes the 128-byte id, the caller hands it to every rank,
 * every rank calls _nccl_init.  _allgather_nccl_dev gathers `count` floats per rank from d_send into
 * d_recv ([world][count]) on `stream`; _nccl_check reports an asynchronous communicator error
 * (ncclCommGetAsyncError) as ULLM_ERR_CUDA. */
#define ULLM_SHARD_NCCL_ID_BYTES 128
int ullm_cuda_shard_nccl_id(void *id /* ULLM_SHARD_NCCL_ID_BYTES */);
int ullm_cuda_shard_nccl_init(ullm_cuda_shard *s, const void *id);
int ullm_cuda_shard_allgather_nccl_dev(ullm_cuda_shard *s, const float *d_send, float *d_recv, size_t count, void *stream);
int ullm_cuda_shard_nccl_check(ullm_cuda_shard *s);

/* ---- mixture-of-experts FFN (MLX 4-bit stacked experts) ----
 * GpuExperts (forward.rs:67-75): `n_experts` matrices concatenated, gate/up
 * `[n_experts, inter, hidden/8]` words, down `[n_experts, hidden, inter/8]`,
 * tables `[n_experts, out, in/group]` of `table_dtype`. */
typedef struct {
    const void *gate_w, *gate_scales, *gate_biases;
    const void *up_w, *up_scales, *up_biases;
    const void *down_w, *down_scales, *down_biases;
    int table_dtype; /* ULLM_DTYPE_F32 or ULLM_DTYPE_BF16 */
    size_t n_experts, hidden, inter, group;
} ullm_moe_experts_input;
int ullm_cuda_experts_create(ullm_cuda_ctx *ctx, const ullm_moe_experts_input *in, ullm_cuda_experts **out);
/* The experts of one MoE layer from an open SafeTensors model: `<prefix>.gate_proj`, `.up_proj`,
 * `.down_proj`, each a stacked MLX linear [n_experts, out, in/8] (mlx_experts, mlx.rs:58-88, sliced
 * per expert there and concatenated again by build_gpu, lib.rs:751-771 — the on-disk stack already is
 * that concatenation, so the bytes go to the device as they lie in the file).  `prefix` is e.g.
 * "model.layers.3.mlp.switch_mlp". */
int ullm_cuda_experts_create_st(ullm_cuda_ctx *ctx, const struct ullm_st *st, const char *prefix, size_t n_experts,
                                size_t hidden, size_t inter, size_t group, ullm_cuda_experts **out);
void ullm_cuda_experts_destroy(ullm_cuda_ctx *ctx, ullm_cuda_experts *e);
/* moe_topk + moe_gate_up_all + moe_down_all + moe_combine (forward.rs:484-494,
 * shader.metal:301-444; CPU form crates/ullm-model/src/lib.rs:1453-1488) for
 * `n_tok` tokens at once: x [n_tok, hidden], router logits [n_tok, n_experts],
 * y [n_tok, hidden]; top-k by descending logit (ties: lower index first),
 * softmax over the k selected, accumulation in that order.  Optional outputs
 * `idx` [n_tok, k] (uint32) and `wts` [n_tok, k] may be NULL. */
int ullm_cuda_moe_ffn(ullm_cuda_ctx *ctx, const ullm_cuda_experts *e, const float *x, const float *logits, size_t n_tok,
                      size_t k, float *y, uint32_t *idx, float *wts);
/* The same on device pointers, enqueued on `stream` (NULL = the context's). */
int ullm_cuda_moe_ffn_dev(ullm_cuda_ctx *ctx, const ullm_cuda_experts *e, const float *d_x, const float *d_logits,
                          size_t n_tok, size_t k, float *d_y, uint32_t *d_idx, float *d_wts, void *stream);

/* No counterpart in the reference.  The same FFN for callers that must not
 * allocate device memory: programs whose own memory pool owns the whole GPU (a
 * cudaMalloc behind its back fails or steals from it) and latency-critical loops
 * that cannot take cudaMalloc's device-wide synchronisation.  Every array of
 * `dev_experts`, and `d_x` / `d_logits` / `d_y`, are device pointers the caller
 * owns (the expert arrays and `d_x` 16-byte aligned, else ULLM_ERR_FORMAT); the kernels' scratch lives in a fixed array inside the
 * library, ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES on every GPU that loads it.
 *  - Problems needing more scratch (roughly 128*(hidden+inter)*4 bytes + 16 KB)
 *    are rejected with ULLM_ERR_FORMAT.
 *  - The first call on a device performs a one-time address look-up: make it at
 *    start-up, before any stream capture.
 *  - The array is shared by all calls and keeps the previous call's contents;
 *    calls whose kernels overlap on the GPU race on it — serialise them.
 *  - Blocks until the result is in `d_y` (waits for `stream` only, not for the
 *    device), so it cannot be part of a stream capture.  Never calls cudaMalloc /
 *    cudaFree.  The calling thread's current device is restored before returning.
 * `err` (may be NULL) receives a message on failure. */
#define ULLM_CUDA_MOE_NOALLOC_SCRATCH_BYTES (4u << 20)
int ullm_cuda_moe_ffn_noalloc(int device, const ullm_moe_experts_input *dev_experts, const float *d_x,
                              const float *d_logits, size_t n_tok, size_t k, float *d_y, void *stream, char *err,
                              size_t err_cap);

/* ---- full decode step: GpuForward (forward.rs:162-757) ---- */
typedef struct { /* GpuParams, forward.rs:24-51 */
    size_t n_embd, n_layer, n_head, n_kv_head, head_dim, n_ff, n_ctx, vocab;
    float rope_theta, eps;
    int rope_neox, qk_norm, sandwich_norm, geglu;
    size_t n_experts, n_experts_used, moe_inter, sliding_window;
    /* Not in the reference (its KV cache is f32, forward.rs:355-356): store K/V
     * as IEEE half when non-zero. */
    int kv_f16;
} ullm_gpu_params;
typedef struct ullm_gpu_weight_s { /* GpuWeight, forward.rs:56-64 */
    int dtype;
    const void *bytes;
    size_t len, out, cols;
    const float *mlx_scales, *mlx_biases;
    size_t mlx_group;
} ullm_gpu_weight;
typedef struct { /* GpuLayerInput, forward.rs:78-100 (dense fields) */
    const float *attn_norm, *ffn_norm;
    ullm_gpu_weight wq, wk, wv, wo, w_gate, w_up, w_down;
    /* Option<&[f32]> of the reference, NULL = absent: projection biases [q_dim] / [kv_dim] / [kv_dim]
     * (Qwen2) and the per-head Q / K RMSNorm weights [head_dim] applied before RoPE (Qwen3; used when
     * params.qk_norm is set). */
    const float *q_bias, *k_bias, *v_bias, *q_norm, *k_norm;
    /* Mixture-of-experts layer (GpuLayerInput::moe_gate / experts_gate / experts_up / experts_down,
     * forward.rs:95-99): the router weight [n_experts, n_embd] and the stacked experts; `experts` NULL =
     * dense layer.  On an MoE layer w_gate / w_up / w_down are not read. */
    ullm_gpu_weight moe_gate;
    const ullm_moe_experts_input *experts;
} ullm_gpu_layer_input;
typedef struct { /* GpuModelInput, forward.rs:105-110 */
    ullm_gpu_params params;
    ullm_gpu_weight output;
    const float *final_norm;
    const ullm_gpu_layer_input *layers; /* params.n_layer entries */
    /* Element type of every `mlx_scales` / `mlx_biases` table above: ULLM_DTYPE_F32 (0, what the reference
     * passes) or ULLM_DTYPE_BF16 for the bits as stored on disk, kept as such on the device.  The experts'
     * tables carry their own `table_dtype`. */
    int mlx_table_dtype;
} ullm_gpu_model_input;

/* GpuForward::new (forward.rs:230).  rope_neox, qk_norm, the q/k/v biases, MLX 4-bit matrices and
 * mixture-of-experts layers (router matvec -> top-k -> routed experts, forward.rs:484-494) are built;
 * sandwich_norm, geglu and the sliding window return UNSUPPORTED instead of being silently ignored. */
int ullm_cuda_forward_create(ullm_cuda_ctx *ctx, const ullm_gpu_model_input *in, ullm_cuda_fwd **out);
/* The same from an open GGUF file (include/ullm_gguf.h): hyperparameters and tensor
 * names as LlamaModel::from_gguf reads them (crates/ullm-model/src/lib.rs:174-301:
 * <arch>.embedding_length ..., token_embd.weight, blk.N.attn_q.weight ..., output_norm.weight,
 * output.weight or the tied embeddings; optional blk.N.attn_{q,k,v}.bias and blk.N.attn_{q,k}_norm.weight),
 * then GpuForward::new as build_gpu calls it (lib.rs:712-805).  "llama" and "qwen2" architectures with
 * Q4_K / Q6_K matrices; files that carry sandwich-norm tensors are refused with UNSUPPORTED. */
struct ullm_gguf;
int ullm_cuda_forward_create_gguf(ullm_cuda_ctx *ctx, const struct ullm_gguf *g, int kv_f16, ullm_cuda_fwd **out);
/* The same from an open MLX model directory (include/ullm_safetensors.h): hyperparameters and tensor
 * names as LlamaModel::from_mlx reads them (crates/ullm-model/src/mlx.rs:103-232: config.json of a
 * Qwen3MoeForCausalLM, lm_head, model.norm.weight, model.layers.N.{input_layernorm, self_attn.{q,k,v,o}_proj,
 * self_attn.{q,k}_norm, post_attention_layernorm, mlp.gate, mlp.switch_mlp.{gate,up,down}_proj}), rotate-half
 * RoPE and per-head Q/K norms on, then GpuForward::new as build_gpu calls it (lib.rs:712-805).  Packed words
 * and bf16 tables go to the device as they lie in the mapped files. */
int ullm_cuda_forward_create_st(ullm_cuda_ctx *ctx, const struct ullm_st *st, int kv_f16, ullm_cuda_fwd **out);
void ullm_cuda_forward_destroy(ullm_cuda_fwd *f);
/* GpuForward::forward (forward.rs:384): one token at `pos`, returns vocab logits. */
int ullm_cuda_forward(ullm_cuda_fwd *f, const float *x_init, size_t pos, float *logits);
/* GpuForward::forward_debug (forward.rs:530-635; reached from `ULLM_GPU_DBG`, crates/ullm-cli/src/main.rs:387):
 * steps through layer 0 one op at a time, unfused, and reports for every intermediate the number of NaNs and
 * infinities and the largest finite magnitude, in the reference's order and under its labels: x_init, attn_norm,
 * wq, wk, [q_norm, k_norm,] rope_q, rope_k, attn_scores, attn_out, wo, ffn_norm, gate, up, glu, w_down.  As there,
 * the residual is not added between the two halves, projection biases are not applied, and K / V of `pos` are
 * written to the cache.  `out` has room for `cap` entries (32 is enough); `*n_out` receives the count.
 * UNSUPPORTED when layer 0 is a mixture-of-experts layer (the reference walks the dense FFN only). */
typedef struct ullm_debug_stat {
    char label[16];
    uint64_t nan, inf;
    float maxabs;
} ullm_debug_stat;
int ullm_cuda_forward_debug(ullm_cuda_fwd *f, const float *x_init, size_t pos, ullm_debug_stat *out, size_t cap, size_t *n_out);
/* Fills KV cache positions [pos0, pos0+n) of every layer from host f32 arrays
 * laid out [n_layer][n][kv_dim] (test / benchmark set-up: the reference fills
 * the cache by running tokens). */
int ullm_cuda_forward_set_kv(ullm_cuda_fwd *f, size_t pos0, size_t n, const float *k, const float *v);
/* GpuForward::supports_batched_prefill (forward.rs:744): 1 when every layer's matrices can go
 * through the tensor-core GEMM (Q4_K, or Q6_K with in % 2048 == 0). */
int ullm_cuda_forward_supports_batched_prefill(const ullm_cuda_fwd *f);
/* GpuForward::forward_batch (forward.rs:757-909): embeds [s, n_embd] f32 token-major for
 * positions 0..s-1 in one pass; fills the KV cache for those positions and returns the
 * LAST token's logits [vocab].  The projections run as bf16 tensor-core GEMMs, so logits
 * agree with s calls of ullm_cuda_forward to the bf16 tolerance (2e-2), not to 1e-3. */
int ullm_cuda_forward_batch(ullm_cuda_fwd *f, const float *embeds, size_t s, float *logits);
/* Greedy continuation kept on the device: runs `n` decode steps starting from
 * token embedding lookups of `embd_table` (dtype rows, resident) — argmax
 * (sample.rs:125-133, first index wins) feeds the next step without a host
 * round trip.  tokens_out[n]. */
int ullm_cuda_forward_greedy(ullm_cuda_fwd *f, const ullm_cuda_buf *embd_table, int embd_dtype, uint32_t first_token,
                             size_t pos, size_t n, uint32_t *tokens_out);
/* The same with the embedding matrix given as a resident weight (ullm_cuda_weight_create / _create_st), which
 * also covers MLX 4-bit tables (embedding row = dequant_mlx_row, crates/ullm-model/src/math.rs:68-79).  Q6_K
 * weights whose rows were re-ordered for the matvec kernels are refused: upload those bytes with
 * ullm_cuda_upload and use ullm_cuda_forward_greedy. */
int ullm_cuda_forward_greedy_weight(ullm_cuda_fwd *f, const ullm_cuda_weight *embd_table, uint32_t first_token, size_t pos,
                                    size_t n, uint32_t *tokens_out);

#ifdef __cplusplus
}
#endif
#endif /* ULLM_CUDA_H */
