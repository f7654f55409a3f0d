/* SafeTensors / MLX model-directory reader: the second feed of the CUDA backend.
 *
 * Replaces, for that purpose, the reference's `SafeTensorsModel` (crates/ullm-safetensors/src/lib.rs:
 * open :35, open_file :45, open_dir :59, add_shard :108, config :170, text_config :177,
 * config_usize/f32/str :182-202, has_tensor :205, tensor_data :219) and the MLX loader's layout rules
 * (crates/ullm-model/src/mlx.rs: mlx_qweight :30, mlx_experts :58, the hyperparameters of from_mlx
 * :103-141).  Same rules:
 *   - a file is an 8-byte little-endian header length, a JSON object, then the tensor bytes; a
 *     tensor's bytes start at 8 + header length + data_offsets[0] (lib.rs:116-152);
 *   - the key "__metadata__" is not a tensor (lib.rs:131-133);
 *   - dtypes "F32", "F16", "BF16" and "U32" / "I32" (MLX packed 4-bit words) only; any other is
 *     ULLM_ST_ERR_UNSUPPORTED (lib.rs:229-241);
 *   - a shape entry that is not a non-negative integer counts as 0, a missing first offset as 0
 *     (lib.rs:144-151: `as_u64().unwrap_or(0)`);
 *   - a tensor's length is the product of its shape times the element size, the second data offset
 *     is not consulted (lib.rs:245-252); a tensor whose bytes reach past the end of its shard has no
 *     data (`tensor_data` -> None, lib.rs:224): `ullm_st_tensor.data` is NULL and nbytes 0;
 *   - a directory holds config.json (absent or unreadable = {} ; present but malformed = FORMAT) and
 *     either model.safetensors.index.json, whose "weight_map" values name the shards — opened in
 *     ascending file-name order, each once — or a single model.safetensors (lib.rs:59-104);
 *   - tensors are kept by name in ascending order; a name seen again in a later shard replaces the
 *     earlier entry (BTreeMap insert, lib.rs:154-163).
 * Every read is bounds-checked; shards are memory-mapped read-only and tensor pointers stay valid until
 * `ullm_st_close`.  Host code only: no GPU is touched.
 */
#ifndef ULLM_SAFETENSORS_H
#define ULLM_SAFETENSORS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ULLM_ST_OK = 0, ULLM_ST_ERR_UNSUPPORTED = 1, ULLM_ST_ERR_FORMAT = 2, ULLM_ST_ERR_IO = 6, ULLM_ST_ERR_INVALID = 7,
       ULLM_ST_ERR_MISSING = 8 };

typedef struct ullm_st ullm_st;

typedef struct ullm_st_tensor {
    const char *name;  /* NUL-terminated, owned by the model object */
    int dtype;         /* ULLM_DTYPE_* of ullm_cuda.h: F32 0, F16 1, BF16 30, MLX_U32 1000 */
    uint32_t n_dims;   /* <= 8 */
    uint64_t shape[8]; /* outermost first */
    uint32_t shard;    /* index of the file that holds the bytes */
    uint64_t offset;   /* absolute byte offset in that file */
    uint64_t nbytes;   /* product(shape) * element size; 0 when the bytes are not all in the file */
    const void *data;  /* NULL when the bytes are not all in the file */
} ullm_st_tensor;

/* SafeTensorsModel::open: a model directory or a single .safetensors file.  `from_bytes` parses one
 * file image held in memory (copied).  On failure *out is NULL and `err` (if given) holds the message. */
int ullm_st_open(const char *path, ullm_st **out, char *err, size_t err_cap);
int ullm_st_from_bytes(const void *bytes, size_t len, ullm_st **out, char *err, size_t err_cap);
void ullm_st_close(ullm_st *m);

size_t ullm_st_shard_count(const ullm_st *m);
/* tensor directory in ascending name order; by name (TensorBag::get + WeightSource::tensor_data) */
size_t ullm_st_tensor_count(const ullm_st *m);
int ullm_st_tensor_at(const ullm_st *m, size_t i, ullm_st_tensor *out);
int ullm_st_tensor_find(const ullm_st *m, const char *name, ullm_st_tensor *out); /* ULLM_ST_ERR_MISSING if absent */
int ullm_st_has_tensor(const ullm_st *m, const char *name);

/* config.json.  `path` is a dot-separated walk from the root: object keys, or decimal indices into
 * arrays ("quantization.group_size", "architectures.0", "text_config.hidden_size").
 * ULLM_ST_ERR_MISSING when the walk fails or the value has no such reading: u64 = a non-negative
 * integer (serde `as_u64`), f32 = any number (`as_f64` narrowed), str = a string. */
int ullm_st_config_u64(const ullm_st *m, const char *path, uint64_t *out);
int ullm_st_config_f32(const ullm_st *m, const char *path, float *out);
int ullm_st_config_str(const ullm_st *m, const char *path, const char **s, size_t *len);
/* 1 when the root config has a "text_config" member (text_config(), lib.rs:177-179) */
int ullm_st_has_text_config(const ullm_st *m);
/* 1 when the directory holds tokenizer.json (tokenizer_json_path, lib.rs:208-211) */
int ullm_st_has_tokenizer_json(const ullm_st *m);

/* ---- MLX 4-bit layout (crates/ullm-model/src/mlx.rs) ---- */

/* One MLX quantized linear, `<name>.weight` / `.scales` / `.biases` (mlx_qweight, mlx.rs:30-56):
 * weight [out, in/8] packed words, in = 8 * shape[1]; tables [out, in/group] as the bf16 bits stored
 * on disk (the reference widens them to f32 at load, mlx.rs:17-26; widening is exact).
 * ULLM_ST_ERR_FORMAT when a tensor is missing, is not of the expected type or its size does not fit. */
typedef struct ullm_st_mlx_weight {
    const uint32_t *weight;
    const uint16_t *scales, *biases; /* bf16 bits */
    uint64_t out, in, group;
} ullm_st_mlx_weight;
int ullm_st_mlx_weight_get(const ullm_st *m, const char *name, uint64_t group, ullm_st_mlx_weight *out, char *err, size_t err_cap);

/* Stacked experts `<name>.weight` [n_experts, out, in/8] with tables [n_experts, out, in/group]
 * (mlx_experts, mlx.rs:58-88): expert e is words e*out*(in/8) .. and table entries e*out*(in/group) ..
 * `expert` selects one slice; pass n_experts to get the whole stack (out = n_experts * out rows). */
int ullm_st_mlx_experts_get(const ullm_st *m, const char *name, uint64_t n_experts, uint64_t out_dim, uint64_t in_dim,
                            uint64_t group, uint64_t expert, ullm_st_mlx_weight *out, char *err, size_t err_cap);

/* The hyperparameters LlamaModel::from_mlx reads from config.json (mlx.rs:103-141) with its defaults:
 * architectures[0] must be "Qwen3MoeForCausalLM" (else ULLM_ST_ERR_UNSUPPORTED); quantization.group_size
 * 64; num_key_value_heads = num_attention_heads; head_dim = hidden_size / num_attention_heads;
 * max_position_embeddings 8192, capped at 8192; rope_theta 1e6; rms_norm_eps 1e-6.  A missing required
 * key (hidden_size, num_attention_heads, num_hidden_layers, num_experts, num_experts_per_tok,
 * moe_intermediate_size, vocab_size) is ULLM_ST_ERR_FORMAT. */
typedef struct ullm_st_mlx_params {
    uint64_t n_embd, n_layer, n_head, n_kv_head, head_dim, n_experts, n_experts_used, moe_inter, n_ctx, vocab, group;
    float rope_theta, eps;
} ullm_st_mlx_params;
int ullm_st_mlx_params_get(const ullm_st *m, ullm_st_mlx_params *out, char *err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif
