/*
 * CPU oracle for uLLM's quantized matrix-product path.  TEST INFRASTRUCTURE ONLY
 * (see ullm_oracle.h).  Each function cites the reference lines it restates;
 * paths are relative to the reference project root.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp (the reference is
 * Rust, which never contracts a*b+c into an FMA and sums f32 iterators in index
 * order; rayon's row parallelism becomes an OpenMP loop over output rows).
 */
#include "ullm_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- crates/ullm-core/src/dtype.rs:55-82 ---- */
size_t uo_block_size(int dtype) {
    switch (dtype) {
    case UO_F32: case UO_F16: case UO_BF16: case UO_MLX_U32: return 1;
    case UO_Q4_0: case UO_Q8_0: return 32;
    case UO_Q4_K: case UO_Q6_K: return 256;
    default: return 0;
    }
}
size_t uo_type_size(int dtype) {
    switch (dtype) {
    case UO_F32: case UO_MLX_U32: return 4;
    case UO_F16: case UO_BF16: return 2;
    case UO_Q4_0: return 18;
    case UO_Q8_0: return 34;
    case UO_Q4_K: return 144;
    case UO_Q6_K: return 210;
    default: return 0;
    }
}

/* ---- crates/ullm-core/src/dequant.rs:15-31 ---- */
float uo_f16_to_f32(uint16_t h) {
    unsigned sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, mant = h & 0x3ffu;
    float v;
    if (exp == 0) {
        v = (float)mant * 5.9604644775390625e-08f; /* 2^-24: zero or subnormal */
    } else if (exp == 0x1f) {
        v = mant == 0 ? INFINITY : NAN;
    } else {
        v = (1.0f + (float)mant / 1024.0f) * ldexpf(1.0f, (int)exp - 15);
    }
    return sign ? -v : v;
}
/* dequant.rs:35-37 */
static inline float rd_f16(const uint8_t *b, size_t off) {
    return uo_f16_to_f32((uint16_t)(b[off] | ((uint16_t)b[off + 1] << 8)));
}
/* dequant.rs:286-288 */
float uo_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---- dequant.rs:41-49 ---- */
void uo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* dequant.rs:112-122 */
static void q8_0(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * 34;
        float d = rd_f16(blk, 0);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = d * (float)(int8_t)blk[2 + j];
    }
}
/* dequant.rs:124-136 */
static void q4_0(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * 18;
        float d = rd_f16(blk, 0);
        const uint8_t *qs = blk + 2;
        for (int j = 0; j < 16; j++) {
            out[b * 32 + j] = d * (float)((int)(qs[j] & 0x0F) - 8);
            out[b * 32 + j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
        }
    }
}
/* dequant.rs:188-217 */
static void q4_k(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * 144;
        float d = rd_f16(blk, 0), dmin = rd_f16(blk, 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        float *o = out + b * 256;
        int is = 0;
        for (int c = 0; c < 4; c++) {
            uint8_t s1, m1, s2, m2;
            uo_scale_min_k4(is, scales, &s1, &m1);
            uo_scale_min_k4(is + 1, scales, &s2, &m2);
            float d1 = d * (float)s1, mm1 = dmin * (float)m1;
            float d2 = d * (float)s2, mm2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) *o++ = d1 * (float)(qs[l] & 0x0F) - mm1;
            for (int l = 0; l < 32; l++) *o++ = d2 * (float)(qs[l] >> 4) - mm2;
            qs += 32;
            is += 2;
        }
    }
}
/* dequant.rs:255-282 */
static void q6_k(const uint8_t *data, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = data + b * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d = rd_f16(blk, 208);
        for (int nh = 0; nh < 2; nh++) {
            const uint8_t *l4 = ql + nh * 64, *h2 = qh + nh * 32;
            const int8_t *s = sc + nh * 8;
            float *y = out + b * 256 + nh * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = ((l4[l] & 0x0F) | ((h2[l] & 3) << 4)) - 32;
                int q2 = ((l4[l + 32] & 0x0F) | (((h2[l] >> 2) & 3) << 4)) - 32;
                int q3 = ((l4[l] >> 4) | (((h2[l] >> 4) & 3) << 4)) - 32;
                int q4 = ((l4[l + 32] >> 4) | (((h2[l] >> 6) & 3) << 4)) - 32;
                y[l] = d * (float)s[is] * (float)q1;
                y[l + 32] = d * (float)s[is + 2] * (float)q2;
                y[l + 64] = d * (float)s[is + 4] * (float)q3;
                y[l + 96] = d * (float)s[is + 6] * (float)q4;
            }
        }
    }
}

/* ---- dequant.rs:61-110 ---- */
int uo_dequantize_into(int dtype, const uint8_t *data, size_t data_len, float *out, size_t n) {
    size_t block = uo_block_size(dtype), ts = uo_type_size(dtype);
    if (block == 0) return UO_ERR_UNSUPPORTED; /* a type the enum does not carry */
    if (n % block != 0) return UO_ERR_FORMAT;
    size_t nblocks = n / block;
    if (data_len < nblocks * ts) return UO_ERR_FORMAT;
    switch (dtype) {
    case UO_F32:
        memcpy(out, data, n * 4);
        break;
    case UO_F16:
        for (size_t i = 0; i < n; i++) out[i] = rd_f16(data, 2 * i);
        break;
    case UO_BF16:
        for (size_t i = 0; i < n; i++)
            out[i] = uo_bf16_to_f32((uint16_t)(data[2 * i] | ((uint16_t)data[2 * i + 1] << 8)));
        break;
    case UO_Q8_0: q8_0(data, nblocks, out); break;
    case UO_Q4_0: q4_0(data, nblocks, out); break;
    case UO_Q4_K: q4_k(data, nblocks, out); break;
    case UO_Q6_K: q6_k(data, nblocks, out); break;
    default: return UO_ERR_UNSUPPORTED; /* dequant.rs:103-107 (U32 lands here too) */
    }
    return UO_OK;
}

/* ---- dequant.rs:297-317 ---- */
void uo_dequantize_mlx_q4(const uint32_t *weight, const float *scales, const float *biases,
                          size_t out, size_t in_dim, size_t group_size, float *y) {
    size_t words = in_dim / 8, groups = in_dim / group_size;
    for (size_t o = 0; o < out; o++)
        for (size_t i = 0; i < in_dim; i++) {
            uint32_t word = weight[o * words + i / 8];
            uint32_t q = (word >> ((i % 8) * 4)) & 0xF;
            size_t g = o * groups + i / group_size;
            y[o * in_dim + i] = (float)q * scales[g] + biases[g];
        }
}

/* ---- crates/ullm-model/src/math.rs:68-79 ---- */
static void dequant_mlx_row(const uo_qweight *w, size_t o, float *buf) {
    size_t cols = w->cols, words = cols / 8, groups = cols / w->mlx_group;
    size_t base = o * words * 4;
    for (size_t i = 0; i < cols; i++) {
        const uint8_t *p = w->data + base + (i / 8) * 4;
        uint32_t word = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
        uint32_t q = (word >> ((i % 8) * 4)) & 0xF;
        size_t g = o * groups + i / w->mlx_group;
        buf[i] = (float)q * w->mlx_scales[g] + w->mlx_biases[g];
    }
}
/* lib.rs:57-61 */
static inline size_t row_bytes(const uo_qweight *w) {
    return (w->cols / uo_block_size(w->dtype)) * uo_type_size(w->dtype);
}
/* math.rs:24-33 */
void uo_dequant_row(const uo_qweight *w, size_t o, float *buf) {
    if (w->mlx_scales) {
        dequant_mlx_row(w, o, buf);
    } else {
        size_t rb = row_bytes(w);
        uo_dequantize_into(w->dtype, w->data + o * rb, rb, buf, w->cols);
    }
}
/* math.rs:17: buf.iter().zip(x).map(|(a,b)| a*b).sum() */
static inline float dot_seq(const float *a, const float *b, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s += a[i] * b[i];
    return s;
}

/* ---- math.rs:9-22 ---- */
void uo_matvec_q(const uo_qweight *w, const float *x, float *y) {
    size_t cols = w->cols, out = w->out;
#pragma omp parallel
    {
        float *buf = (float *)malloc(cols * sizeof(float));
#pragma omp for schedule(static)
        for (long o = 0; o < (long)out; o++) {
            uo_dequant_row(w, (size_t)o, buf);
            y[o] = dot_seq(buf, x, cols);
        }
        free(buf);
    }
}

/* ---- math.rs:38-63 ---- */
void uo_matmul_q(const uo_qweight *w, const float *xs, size_t s_len, float *y) {
    size_t cols = w->cols, out = w->out;
#pragma omp parallel
    {
        float *buf = (float *)malloc(cols * sizeof(float));
#pragma omp for schedule(static)
        for (long o = 0; o < (long)out; o++) {
            uo_dequant_row(w, (size_t)o, buf);
            for (size_t s = 0; s < s_len; s++) y[s * out + (size_t)o] = dot_seq(buf, xs + s * cols, cols);
        }
        free(buf);
    }
}

/* ---- math.rs:82-86 ---- */
void uo_rmsnorm(const float *x, const float *weight, size_t n, float eps, float *y) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
    float ms = ss / (float)n + eps;
    float inv = 1.0f / sqrtf(ms);
    for (size_t i = 0; i < n; i++) y[i] = x[i] * inv * weight[i];
}
/* ---- math.rs:89-100 ---- */
void uo_softmax(float *x, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; i++) max = fmaxf(max, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - max);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (size_t i = 0; i < n; i++) x[i] *= inv;
}
/* ---- math.rs:103-105 ---- */
float uo_silu(float x) { return x / (1.0f + expf(-x)); }
/* ---- math.rs:116-136 ---- */
void uo_rope(float *vec, size_t n_heads, size_t head_dim, size_t rotary_dim, size_t pos, float theta) {
    for (size_t h = 0; h < n_heads; h++) {
        size_t off = h * head_dim;
        for (size_t i = 0; i + 1 < rotary_dim; i += 2) {
            float freq = 1.0f / powf(theta, (float)i / (float)rotary_dim);
            float ang = (float)pos * freq;
            float sn = sinf(ang), cs = cosf(ang);
            float a = vec[off + i], b = vec[off + i + 1];
            vec[off + i] = a * cs - b * sn;
            vec[off + i + 1] = a * sn + b * cs;
        }
    }
}
/* math.rs:140-162: rotate-half pairs; only the first rotary_dim of a head turns */
void uo_rope_neox(float *vec, size_t n_heads, size_t head_dim, size_t rotary_dim, size_t pos, float theta) {
    size_t half = rotary_dim / 2;
    for (size_t h = 0; h < n_heads; h++) {
        size_t off = h * head_dim;
        for (size_t i = 0; i < half; i++) {
            float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)rotary_dim);
            float ang = (float)pos * freq;
            float sn = sinf(ang), cs = cosf(ang);
            float a = vec[off + i], b = vec[off + i + half];
            vec[off + i] = a * cs - b * sn;
            vec[off + i + half] = a * sn + b * cs;
        }
    }
}
/* ---- crates/ullm-model/src/sample.rs:125-133 ---- */
size_t uo_argmax(const float *x, size_t n) {
    size_t best = 0;
    for (size_t i = 0; i < n; i++)
        if (x[i] > x[best]) best = i;
    return best;
}

/* ---- lib.rs:1455-1475 ---- */
void uo_moe_topk(const float *logits, size_t n, size_t k, uint32_t *idx, float *wts) {
    /* Descending selection; the reference sorts with an unstable sort, so equal
     * logits have no defined order there: lower index first here. */
    uint8_t *taken = (uint8_t *)calloc(n, 1);
    for (size_t j = 0; j < k; j++) {
        size_t best = n;
        for (size_t i = 0; i < n; i++)
            if (!taken[i] && (best == n || logits[i] > logits[best])) best = i;
        taken[best] = 1;
        idx[j] = (uint32_t)best;
    }
    free(taken);
    float max = -INFINITY;
    for (size_t j = 0; j < k; j++) max = fmaxf(max, logits[idx[j]]);
    float wsum = 0.0f;
    for (size_t j = 0; j < k; j++) {
        float e = expf(logits[idx[j]] - max);
        wsum += e;
        wts[j] = e;
    }
    for (size_t j = 0; j < k; j++) wts[j] /= wsum;
}

/* ---- lib.rs:1476-1488 ---- */
void uo_moe_ffn(const uo_moe_experts *e, const float *logits, size_t k, const float *xb, float *out) {
    uint32_t idx[64];
    float wts[64];
    if (k > 64) k = 64;
    uo_moe_topk(logits, e->n_experts, k, idx, wts);
    size_t hid = e->hidden, inter = e->inter, gs = e->group;
    size_t gu_words = inter * hid / 8, gu_groups = inter * hid / gs;
    size_t dn_words = hid * inter / 8, dn_groups = hid * inter / gs;
    float *gate = (float *)malloc(inter * sizeof(float));
    float *up = (float *)malloc(inter * sizeof(float));
    float *down = (float *)malloc(hid * sizeof(float));
    for (size_t o = 0; o < hid; o++) out[o] = 0.0f;
    for (size_t j = 0; j < k; j++) {
        size_t ex = idx[j];
        uo_qweight wg = {e->gate_w + ex * gu_words * 4, UO_MLX_U32, inter, hid,
                         e->gate_s + ex * gu_groups, e->gate_b + ex * gu_groups, gs};
        uo_qweight wu = {e->up_w + ex * gu_words * 4, UO_MLX_U32, inter, hid,
                         e->up_s + ex * gu_groups, e->up_b + ex * gu_groups, gs};
        uo_qweight wd = {e->down_w + ex * dn_words * 4, UO_MLX_U32, hid, inter,
                         e->down_s + ex * dn_groups, e->down_b + ex * dn_groups, gs};
        uo_matvec_q(&wg, xb, gate);
        uo_matvec_q(&wu, xb, up);
        for (size_t i = 0; i < inter; i++) gate[i] = uo_silu(gate[i]) * up[i];
        uo_matvec_q(&wd, gate, down);
        float wk = wts[j];
        for (size_t o = 0; o < hid; o++) out[o] += wk * down[o];
    }
    free(gate);
    free(up);
    free(down);
}

/* IEEE half round-trip (round to nearest even) for the f16 KV cache. */
float uo_round_f16(float v) {
    _Float16 h = (_Float16)v;
    return (float)h;
}

/* ---- lib.rs:692-710 ---- */
void uo_embed(const uo_model *m, uint32_t token, float *x) { uo_dequant_row(&m->tok_embeddings, token, x); }

/* ---- lib.rs:832-968 (dense softmax-attention branch) ---- */
void uo_forward_llama_embd(uo_model *m, const float *x_init, size_t pos, float *logits) {
    size_t n_embd = m->n_embd, hd = m->head_dim;
    size_t kv_dim = m->n_kv_head * hd, q_dim = m->n_head * hd, kv_mul = m->n_head / m->n_kv_head;
    float scale = 1.0f / sqrtf((float)hd); /* lib.rs:821 */
    float *x = (float *)malloc(n_embd * 4), *xb = (float *)malloc(n_embd * 4);
    float *q = (float *)malloc(q_dim * 4), *k = (float *)malloc(kv_dim * 4), *v = (float *)malloc(kv_dim * 4);
    float *att = (float *)malloc(q_dim * 4), *proj = (float *)malloc(n_embd * 4);
    float *gate = (float *)malloc((m->n_ff + 1) * 4), *up = (float *)malloc((m->n_ff + 1) * 4);
    float *scores = (float *)malloc((pos + 1) * 4);
    memcpy(x, x_init, n_embd * 4);
    for (size_t l = 0; l < m->n_layer; l++) {
        const uo_layer *lw = &m->layers[l];
        uo_rmsnorm(x, lw->attn_norm, n_embd, m->eps, xb);
        uo_matvec_q(&lw->wq, xb, q);
        uo_matvec_q(&lw->wk, xb, k);
        uo_matvec_q(&lw->wv, xb, v);
        if (lw->q_bias) for (size_t i = 0; i < q_dim; i++) q[i] += lw->q_bias[i];   /* lib.rs:877-885 */
        if (lw->k_bias) for (size_t i = 0; i < kv_dim; i++) k[i] += lw->k_bias[i];
        if (lw->v_bias) for (size_t i = 0; i < kv_dim; i++) v[i] += lw->v_bias[i];
        if (lw->q_norm) { /* lib.rs:887-901: per-head RMSNorm before RoPE */
            float tmp[512];
            for (size_t h = 0; h < m->n_head; h++) {
                uo_rmsnorm(q + h * hd, lw->q_norm, hd, m->eps, tmp);
                memcpy(q + h * hd, tmp, hd * 4);
            }
        }
        if (lw->k_norm) {
            float tmp[512];
            for (size_t h = 0; h < m->n_kv_head; h++) {
                uo_rmsnorm(k + h * hd, lw->k_norm, hd, m->eps, tmp);
                memcpy(k + h * hd, tmp, hd * 4);
            }
        }
        if (m->rope_neox) {
            uo_rope_neox(q, m->n_head, hd, hd, pos, m->rope_theta);
            uo_rope_neox(k, m->n_kv_head, hd, hd, pos, m->rope_theta);
        } else {
            uo_rope(q, m->n_head, hd, hd, pos, m->rope_theta);
            uo_rope(k, m->n_kv_head, hd, hd, pos, m->rope_theta);
        }
        size_t kv_base = l * m->n_ctx * kv_dim, off = kv_base + pos * kv_dim;
        for (size_t i = 0; i < kv_dim; i++) {
            m->key_cache[off + i] = m->kv_f16 ? uo_round_f16(k[i]) : k[i];
            m->val_cache[off + i] = m->kv_f16 ? uo_round_f16(v[i]) : v[i];
        }
        for (size_t i = 0; i < q_dim; i++) att[i] = 0.0f;
        for (size_t h = 0; h < m->n_head; h++) {
            size_t kvh = h / kv_mul;
            const float *qh = q + h * hd;
            for (size_t t = 0; t <= pos; t++)
                scores[t] = dot_seq(qh, m->key_cache + kv_base + t * kv_dim + kvh * hd, hd) * scale;
            uo_softmax(scores, pos + 1);
            float *ao = att + h * hd;
            for (size_t t = 0; t <= pos; t++) {
                const float *vt = m->val_cache + kv_base + t * kv_dim + kvh * hd;
                float a = scores[t];
                for (size_t d = 0; d < hd; d++) ao[d] += a * vt[d];
            }
        }
        uo_matvec_q(&lw->wo, att, proj);
        for (size_t i = 0; i < n_embd; i++) x[i] += proj[i];
        uo_rmsnorm(x, lw->ffn_norm, n_embd, m->eps, xb);
        if (lw->experts) { /* lib.rs:953-955: router logits, then the routed experts (lib.rs:1453-1488) */
            float *rl = (float *)malloc(lw->experts->n_experts * 4);
            uo_matvec_q(&lw->moe_gate, xb, rl);
            uo_moe_ffn(lw->experts, rl, lw->n_experts_used, xb, proj);
            free(rl);
        } else {
            uo_matvec_q(&lw->w_gate, xb, gate);
            uo_matvec_q(&lw->w_up, xb, up);
            for (size_t i = 0; i < m->n_ff; i++) gate[i] = uo_silu(gate[i]) * up[i];
            uo_matvec_q(&lw->w_down, gate, proj);
        }
        for (size_t i = 0; i < n_embd; i++) x[i] += proj[i];
    }
    uo_rmsnorm(x, m->final_norm, n_embd, m->eps, xb);
    uo_matvec_q(&m->output, xb, logits);
    free(x); free(xb); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up); free(scores);
}
/* GpuForward::forward_debug (crates/ullm-metal/src/forward.rs:530-635) on the CPU: layer 0 one op at a time, the
 * largest finite magnitude of every intermediate in the order the reference prints them.  As there, the residual is
 * not added between the attention and the FFN half (ffn_norm normalises x_init), projection biases are not applied,
 * and K / V of `pos` go into the cache.  Returns the number of entries (labels: uo_debug_label). */
static const char *const UO_DEBUG_LABELS[] = {"x_init", "attn_norm", "wq", "wk", "q_norm", "k_norm", "rope_q", "rope_k", "attn_scores",
                                              "attn_out", "wo", "ffn_norm", "gate", "up", "glu", "w_down"};
const char *uo_debug_label(int i) { return i >= 0 && i < 16 ? UO_DEBUG_LABELS[i] : ""; }
static float maxabs_finite(const float *v, size_t n) {
    float mx = 0.0f;
    for (size_t i = 0; i < n; i++)
        if (isfinite(v[i]) && fabsf(v[i]) > mx) mx = fabsf(v[i]);
    return mx;
}
int uo_forward_debug(uo_model *m, const float *x_init, size_t pos, int *label_idx, float *maxabs, int cap) {
    size_t n_embd = m->n_embd, hd = m->head_dim, n_ff = m->n_ff;
    size_t kv_dim = m->n_kv_head * hd, q_dim = m->n_head * hd, kv_mul = m->n_head / m->n_kv_head;
    float scale = 1.0f / sqrtf((float)hd);
    const uo_layer *lw = &m->layers[0];
    if (lw->experts || cap < 16) return -1;
    float *xb = (float *)malloc(n_embd * 4), *q = (float *)malloc(q_dim * 4), *k = (float *)malloc(kv_dim * 4), *v = (float *)malloc(kv_dim * 4);
    float *att = (float *)malloc(q_dim * 4), *proj = (float *)malloc(n_embd * 4);
    float *gate = (float *)malloc((n_ff + 1) * 4), *up = (float *)malloc((n_ff + 1) * 4);
    float *scores = (float *)malloc(m->n_head * (pos + 1) * 4);
    int n = 0;
#define UO_PUT(idx, ptr, cnt) (label_idx[n] = (idx), maxabs[n] = maxabs_finite((ptr), (cnt)), n++)
    UO_PUT(0, x_init, n_embd);
    uo_rmsnorm(x_init, lw->attn_norm, n_embd, m->eps, xb);
    UO_PUT(1, xb, n_embd);
    uo_matvec_q(&lw->wq, xb, q);
    UO_PUT(2, q, q_dim);
    uo_matvec_q(&lw->wk, xb, k);
    UO_PUT(3, k, kv_dim);
    uo_matvec_q(&lw->wv, xb, v);
    float tmp[512];
    if (lw->q_norm) {
        for (size_t h = 0; h < m->n_head; h++) {
            uo_rmsnorm(q + h * hd, lw->q_norm, hd, m->eps, tmp);
            memcpy(q + h * hd, tmp, hd * 4);
        }
        UO_PUT(4, q, q_dim);
    }
    if (lw->k_norm) {
        for (size_t h = 0; h < m->n_kv_head; h++) {
            uo_rmsnorm(k + h * hd, lw->k_norm, hd, m->eps, tmp);
            memcpy(k + h * hd, tmp, hd * 4);
        }
        UO_PUT(5, k, kv_dim);
    }
    if (m->rope_neox) {
        uo_rope_neox(q, m->n_head, hd, hd, pos, m->rope_theta);
        uo_rope_neox(k, m->n_kv_head, hd, hd, pos, m->rope_theta);
    } else {
        uo_rope(q, m->n_head, hd, hd, pos, m->rope_theta);
        uo_rope(k, m->n_kv_head, hd, hd, pos, m->rope_theta);
    }
    UO_PUT(6, q, q_dim);
    UO_PUT(7, k, kv_dim);
    size_t off = pos * kv_dim;
    for (size_t i = 0; i < kv_dim; i++) {
        m->key_cache[off + i] = m->kv_f16 ? uo_round_f16(k[i]) : k[i];
        m->val_cache[off + i] = m->kv_f16 ? uo_round_f16(v[i]) : v[i];
    }
    for (size_t h = 0; h < m->n_head; h++)
        for (size_t t = 0; t <= pos; t++)
            scores[h * (pos + 1) + t] = dot_seq(q + h * hd, m->key_cache + t * kv_dim + (h / kv_mul) * hd, hd) * scale;
    UO_PUT(8, scores, m->n_head * (pos + 1));
    for (size_t i = 0; i < q_dim; i++) att[i] = 0.0f;
    for (size_t h = 0; h < m->n_head; h++) {
        float *sc = scores + h * (pos + 1), *ao = att + h * hd;
        uo_softmax(sc, pos + 1);
        for (size_t t = 0; t <= pos; t++) {
            const float *vt = m->val_cache + t * kv_dim + (h / kv_mul) * hd;
            for (size_t d = 0; d < hd; d++) ao[d] += sc[t] * vt[d];
        }
    }
    UO_PUT(9, att, q_dim);
    uo_matvec_q(&lw->wo, att, proj);
    UO_PUT(10, proj, n_embd);
    uo_rmsnorm(x_init, lw->ffn_norm, n_embd, m->eps, xb);
    UO_PUT(11, xb, n_embd);
    uo_matvec_q(&lw->w_gate, xb, gate);
    UO_PUT(12, gate, n_ff);
    uo_matvec_q(&lw->w_up, xb, up);
    UO_PUT(13, up, n_ff);
    for (size_t i = 0; i < n_ff; i++) gate[i] = uo_silu(gate[i]) * up[i];
    UO_PUT(14, gate, n_ff);
    uo_matvec_q(&lw->w_down, gate, proj);
    UO_PUT(15, proj, n_embd);
#undef UO_PUT
    free(xb); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up); free(scores);
    return n;
}
void uo_forward_llama(uo_model *m, uint32_t token, size_t pos, float *logits) {
    float *x = (float *)malloc(m->n_embd * 4);
    uo_embed(m, token, x);
    uo_forward_llama_embd(m, x, pos, logits);
    free(x);
}

int uo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
