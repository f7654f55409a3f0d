/*
 * CPU oracle for the quantized matrix-product path of uLLM.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * CPU algorithm (crates/ullm-core/src/dequant.rs, crates/ullm-model/src/math.rs,
 * crates/ullm-model/src/lib.rs, crates/ullm-model/src/sample.rs).  It is the
 * checker the CUDA kernels are compared against and the timed CPU baseline.
 * Nothing that ships (the CUDA library, its host wrappers) may call it.
 *
 * Parity pinning: the reference holds known answers only for the f16 widening,
 * the MLX 4-bit word (dequant.rs:324-334) and the Q8_0 / Q4_0 closed forms
 * (dequant.rs:345-367); the oracle is checked against all of them.  Q4_K and
 * Q6_K have NO known-answer vector in the reference ("parity unpinned" for those
 * two layouts): they are pinned instead by an independent second statement of
 * the same formats (the factored form the reference's GPU shader uses) kept in
 * the test-suite.
 *
 * Arithmetic rules restated from the reference: f32 everywhere, products and
 * sums evaluated left to right in index order, no fused multiply-add (build with
 * -ffp-contract=off), transcendental functions from the platform libm.
 */
#ifndef ULLM_ORACLE_H
#define ULLM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml tensor type ids (crates/ullm-gguf/src/types.rs:7-29); MLX packed words
 * have no ggml id, the reference calls them DType::U32 (dtype.rs:27). */
enum {
    UO_F32 = 0,
    UO_F16 = 1,
    UO_Q4_0 = 2,
    UO_Q8_0 = 8,
    UO_Q4_K = 12,
    UO_Q6_K = 14,
    UO_BF16 = 30,
    UO_MLX_U32 = 1000
};

/* Error convention of crates/ullm-core/src/error.rs:11-20. */
enum { UO_OK = 0, UO_ERR_FORMAT = 1, UO_ERR_UNSUPPORTED = 2 };

/* dtype.rs:55-82 */
size_t uo_block_size(int dtype);
size_t uo_type_size(int dtype);

/* dequant.rs:15-31, :286 */
float uo_f16_to_f32(uint16_t h);
float uo_bf16_to_f32(uint16_t h);

/* dequant.rs:41-49: (scale, min) pair j of the 12 packed bytes q. */
void uo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn);

/* dequant.rs:61-110: n = element count; returns UO_ERR_FORMAT when n is not a
 * multiple of the block size or data_len is short, UO_ERR_UNSUPPORTED for a
 * type without a dequantizer. */
int uo_dequantize_into(int dtype, const uint8_t *data, size_t data_len, float *out, size_t n);

/* dequant.rs:297-317 */
void uo_dequantize_mlx_q4(const uint32_t *weight, const float *scales, const float *biases,
                          size_t out, size_t in_dim, size_t group_size, float *y);

/* A weight kept quantized: crates/ullm-model/src/lib.rs:49-61 (QWeight) and
 * :39-43 (MlxQuant).  mlx_scales == NULL for GGUF block types. */
typedef struct {
    const uint8_t *data;
    int dtype;
    size_t out, cols;
    const float *mlx_scales, *mlx_biases;
    size_t mlx_group;
} uo_qweight;

/* math.rs:24-33, :68-79 */
void uo_dequant_row(const uo_qweight *w, size_t o, float *buf);
/* math.rs:9-22: y[o] = sum_i W[o,i]*x[i], sequential f32 sum, rows in parallel. */
void uo_matvec_q(const uo_qweight *w, const float *x, float *y);
/* math.rs:38-63: xs token-major [s_len, cols] -> y token-major [s_len, out]. */
void uo_matmul_q(const uo_qweight *w, const float *xs, size_t s_len, float *y);

/* math.rs:82-86, :89-100, :103-105, :116-136, :140-162 */
void uo_rope_neox(float *vec, size_t n_heads, size_t head_dim, size_t rotary_dim, size_t pos, float theta);
void uo_rmsnorm(const float *x, const float *weight, size_t n, float eps, float *y);
void uo_softmax(float *x, size_t n);
float uo_silu(float x);
void uo_rope(float *vec, size_t n_heads, size_t head_dim, size_t rotary_dim, size_t pos, float theta);

/* sample.rs:125-133: first index wins ties. */
size_t uo_argmax(const float *x, size_t n);

/* Routed part of lib.rs:1453-1488 for ONE token, given the router logits.
 * Experts are stacked [n_experts, out, ...] as mlx.rs:71-87 / lib.rs:751-771.
 * Top-k by descending logit (ties: lower index first), softmax over the k
 * selected, SwiGLU FFN per expert, accumulated in that order. */
typedef struct {
    const uint8_t *gate_w, *up_w, *down_w;           /* packed u32 words            */
    const float *gate_s, *gate_b, *up_s, *up_b, *down_s, *down_b; /* widened tables */
    size_t n_experts, hidden, inter, group;
} uo_moe_experts;
void uo_moe_topk(const float *logits, size_t n, size_t k, uint32_t *idx, float *wts);
void uo_moe_ffn(const uo_moe_experts *e, const float *logits, size_t k, const float *xb, float *out);

/* Dense Llama decode step: lib.rs:807-969 (non-gated, non-linear, non-MoE
 * branch), embed lib.rs:692-710.  kv_f16 != 0 rounds K and V through IEEE half
 * when they are written to the cache (the reference keeps f32: lib.rs:184). */
typedef struct {
    const float *attn_norm, *ffn_norm;
    uo_qweight wq, wk, wv, wo, w_gate, w_up, w_down;
    /* optional (NULL = absent): Qwen2 projection biases (lib.rs:877-885) and the per-head
     * Q/K RMSNorm weights [head_dim] applied before RoPE (lib.rs:887-901) */
    const float *q_bias, *k_bias, *v_bias, *q_norm, *k_norm;
    /* mixture-of-experts layer (lib.rs:953-955, 1453-1488): router weight [n_experts, n_embd], stacked
     * experts and experts per token; experts == NULL = dense layer (w_gate / w_up / w_down used) */
    uo_qweight moe_gate;
    const uo_moe_experts *experts;
    size_t n_experts_used;
} uo_layer;
typedef struct {
    size_t n_embd, n_layer, n_head, n_kv_head, head_dim, n_ff, n_ctx, vocab;
    float rope_theta, eps;
    uo_qweight tok_embeddings, output;
    const float *final_norm;
    const uo_layer *layers;
    float *key_cache, *val_cache; /* [n_layer][n_ctx][kv_dim] f32 */
    int kv_f16;
    int rope_neox; /* rotate-half pairs (x[i], x[i + d/2]) instead of interleaved ones (lib.rs:903-909) */
} uo_model;
void uo_embed(const uo_model *m, uint32_t token, float *x);
void uo_forward_llama(uo_model *m, uint32_t token, size_t pos, float *logits);
/* Same step but starting from a given embedding row (what the GPU surface gets:
 * crates/ullm-metal/src/forward.rs:384). */
void uo_forward_llama_embd(uo_model *m, const float *x_init, size_t pos, float *logits);

/* GpuForward::forward_debug (forward.rs:530-635) restated: largest finite |value| of every intermediate of layer 0. */
const char *uo_debug_label(int i);
int uo_forward_debug(uo_model *m, const float *x_init, size_t pos, int *label_idx, float *maxabs, int cap);

/* IEEE half round-trip used for the f16 KV cache (round to nearest even). */
float uo_round_f16(float v);

int uo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
