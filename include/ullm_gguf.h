/* GGUF model-file reader: the feed of the CUDA backend (weights by name, hyperparameters by key).
 *
 * Replaces, for that purpose, the reference's `GgufModel` (crates/ullm-gguf/src/lib.rs:45-169:
 * open / from_bytes / parse, metadata_get, architecture, tensor_data) and its `WeightSource`
 * face (crates/ullm-core/src/ir.rs:63-69: tensor_bag / tensor_data).  Same rules:
 *   - magic "GGUF" (0x46554747 LE), versions 2 and 3 only (lib.rs:76-87), little-endian;
 *   - metadata values of the 13 GGUF types, arrays not nested (value.rs:65-112);
 *   - tensor shapes stored fastest-dimension-first, reported outermost-first (lib.rs:135-138);
 *   - tensor data starts at the end of the tensor directory rounded up to
 *     `general.alignment` (default 32, at least 1; lib.rs:123-131), each tensor at its
 *     relative offset from there, and must lie inside the file (lib.rs:140-150);
 *   - ggml type ids as crates/ullm-gguf/src/types.rs:7-29, block geometry as
 *     crates/ullm-core/src/dtype.rs:55-82.
 * Every read is bounds-checked: a truncated or malformed file is ULLM_GGUF_ERR_FORMAT, never a crash.
 * The file is memory-mapped read-only (or copied, for `from_bytes`); tensor pointers stay valid
 * until `ullm_gguf_close`.  Host code only: no GPU is touched.
 */
#ifndef ULLM_GGUF_H
#define ULLM_GGUF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ULLM_GGUF_OK = 0, ULLM_GGUF_ERR_UNSUPPORTED = 1, ULLM_GGUF_ERR_FORMAT = 2, ULLM_GGUF_ERR_IO = 6, ULLM_GGUF_ERR_INVALID = 7,
       ULLM_GGUF_ERR_MISSING = 8 };

typedef struct ullm_gguf ullm_gguf;

typedef struct ullm_gguf_tensor {
    const char *name;   /* NUL-terminated, owned by the file object */
    int dtype;          /* ggml type id (F32 0, F16 1, Q4_K 12, Q6_K 14, BF16 30, ...) */
    uint32_t n_dims;    /* <= 8 */
    uint64_t shape[8];  /* outermost first: a weight matrix is {out, in} */
    uint64_t offset;    /* absolute byte offset in the file */
    uint64_t nbytes;
    const void *data;   /* the bytes themselves */
} ullm_gguf_tensor;

/* GgufModel::open / from_bytes.  On failure *out is NULL and `err` (if given) holds the message. */
int ullm_gguf_open(const char *path, ullm_gguf **out, char *err, size_t err_cap);
int ullm_gguf_from_bytes(const void *bytes, size_t len, ullm_gguf **out, char *err, size_t err_cap);
void ullm_gguf_close(ullm_gguf *g);

uint32_t ullm_gguf_version(const ullm_gguf *g);
/* general.architecture, or "" (GgufModel::architecture, lib.rs:176-180) */
const char *ullm_gguf_architecture(const ullm_gguf *g);
uint64_t ullm_gguf_alignment(const ullm_gguf *g);
uint64_t ullm_gguf_data_start(const ullm_gguf *g);

/* tensor directory, in file order; by name (TensorBag::get) */
size_t ullm_gguf_tensor_count(const ullm_gguf *g);
int ullm_gguf_tensor_at(const ullm_gguf *g, size_t i, ullm_gguf_tensor *out);
int ullm_gguf_tensor_find(const ullm_gguf *g, const char *name, ullm_gguf_tensor *out); /* ULLM_GGUF_ERR_MISSING if absent */

/* metadata (metadata_get + Value::{to_u64, to_f32, as_str, as_array}); ULLM_GGUF_ERR_MISSING when the
 * key is absent or its value has no such reading */
size_t ullm_gguf_meta_count(const ullm_gguf *g);
const char *ullm_gguf_meta_key_at(const ullm_gguf *g, size_t i); /* keys in ascending order */
int ullm_gguf_meta_type(const ullm_gguf *g, const char *key, int *type_id, int *elem_type_id, uint64_t *array_len);
int ullm_gguf_meta_u64(const ullm_gguf *g, const char *key, uint64_t *out);  /* any integer or bool */
int ullm_gguf_meta_f32(const ullm_gguf *g, const char *key, float *out);     /* f32 or f64 */
int ullm_gguf_meta_str(const ullm_gguf *g, const char *key, const char **s, size_t *len);
int ullm_gguf_meta_array_u64(const ullm_gguf *g, const char *key, size_t i, uint64_t *out);
int ullm_gguf_meta_array_f32(const ullm_gguf *g, const char *key, size_t i, float *out);
int ullm_gguf_meta_array_str(const ullm_gguf *g, const char *key, size_t i, const char **s, size_t *len);

/* The hyperparameters LlamaModel::from_gguf reads (crates/ullm-model/src/lib.rs:174-225), with its
 * defaults: head_count_kv = head_count, context_length 2048 capped at 8192, key_length =
 * embedding_length / head_count, rope.freq_base 10000, layer_norm_rms_epsilon 1e-5, vocab =
 * <arch>.vocab_size or the length of tokenizer.ggml.tokens (lib.rs:207-215).  ULLM_GGUF_ERR_FORMAT
 * when a required key is missing, ULLM_GGUF_ERR_UNSUPPORTED for architectures other than "llama" and "qwen2"
 * (the reference also loads "gemma3", whose sandwich norms, GeGLU and sliding window this backend does not build). */
typedef struct ullm_gguf_llama_params {
    uint64_t n_embd, n_layer, n_head, n_kv_head, head_dim, n_ff, n_ctx, vocab;
    float rope_theta, eps;
} ullm_gguf_llama_params;
int ullm_gguf_llama_params_get(const ullm_gguf *g, ullm_gguf_llama_params *out, char *err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif
