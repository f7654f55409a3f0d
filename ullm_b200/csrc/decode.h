// Resident dense-Llama decode engine (see decode.cu).
#pragma once

#include "common.cuh"
#include "kernels.h"

#include <vector>

namespace ullm {

struct ForwardParams { // GpuParams, crates/ullm-metal/src/forward.rs:24-51 (dense subset)
    size_t n_embd = 0, n_layer = 0, n_head = 0, n_kv_head = 0, head_dim = 0, n_ff = 0, n_ctx = 0, vocab = 0;
    float rope_theta = 10000.f, eps = 1e-5f;
    int kv_f16 = 0;
    int rope_neox = 0, qk_norm = 0;
    size_t n_experts = 0, n_experts_used = 0, moe_inter = 0; // mixture-of-experts layers (n_ff may then be 0)
};
struct HostWeight { // GpuWeight, forward.rs:56-64
    int dtype = 0;
    const void *bytes = nullptr;
    size_t out = 0, cols = 0;
    const void *scales = nullptr, *biases = nullptr; // MLX 4-bit: per-group tables (element type: HostModel::mlx_table_bytes)
    size_t group = 0;
};
struct HostLayer {
    const float *attn_norm = nullptr, *ffn_norm = nullptr;
    HostWeight wq, wk, wv, wo, w_gate, w_up, w_down;
    const float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    // mixture-of-experts layer (GpuLayerInput::moe_gate / experts_*, forward.rs:95-99): router [n_experts, n_embd] and the
    // stacked experts as host pointers; `experts` null = dense layer
    HostWeight moe_gate;
    const MoeExperts *experts = nullptr;
};
struct HostModel {
    int mlx_table_bytes = 4; // 4 = f32 tables (as the reference passes them), 2 = bf16 bits as stored on disk
    HostWeight output;
    const float *final_norm = nullptr;
    std::vector<HostLayer> layers;
};

// One line of GpuForward::forward_debug's report (crates/ullm-metal/src/forward.rs:566-580).
struct DebugStat {
    char label[16];
    unsigned long long nan, inf;
    float maxabs; // largest finite magnitude
};

struct Forward {
    static constexpr size_t MAX_GREEDY = 4096; // tokens kept on the device between host reads
    struct Mat {
        int fmt = 0;
        void *w = nullptr;
        size_t out = 0, cols = 0;
        void *scales = nullptr, *biases = nullptr; // MLX 4-bit tables
        int tbl_bytes = 4;
        size_t group = 0;
    };
    struct Layer {
        float *attn_norm = nullptr, *ffn_norm = nullptr;
        float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr; // optional
        bool qk_fused = false, gu_fused = false, qkv_fused = false; // qkv_fused: MLX q | k | v rows and tables stacked (wqk holds them)
        Mat wqk, wq, wk, wv, wo, wgu, wg, wu, wd;
        bool moe = false; // router + routed experts instead of the dense FFN
        Mat moe_gate;
        MoeExperts experts;
    };

    DeviceInfo dev;
    int device = 0;
    ForwardParams P;
    cudaStream_t stream = nullptr;
    std::vector<Layer> layers;
    Mat output;
    float *final_norm = nullptr;
    float2 *rope = nullptr;
    void *kcache = nullptr, *vcache = nullptr;
    int n_split = 0;
    float *x = nullptr, *xb = nullptr, *qk = nullptr, *vbuf = nullptr, *attn = nullptr, *hidden = nullptr, *gate = nullptr,
          *up = nullptr, *logits = nullptr, *partial = nullptr;
    unsigned *counters = nullptr;
    void *argmax_part = nullptr; // per-CTA candidates of the greedy argmax
    void *state = nullptr; // device ints: [0] pos, [1] token, [2] step
    uint32_t *tokens_out = nullptr;
    void *h_pin = nullptr;
    float *h_x = nullptr, *h_logits = nullptr; // page-locked staging of forward()'s input row and logits
    volatile int *h_status = nullptr;
    int *d_status = nullptr;
    bool owned_host = false;
    std::vector<void *> owned;
    bool use_graph = true, use_pdl = false, use_chain = false; // use_chain: q|k and v of a layer in one persistent launch
    unsigned *chain_sync = nullptr; // grid-barrier words of the chain kernel
    cudaGraphExec_t graph_exec[2] = {nullptr, nullptr};
    const void *graph_table = nullptr;
    int graph_dtype = 0;
    int launches = 0, graph_launches = 0;

    ~Forward();
    static const char *check_params(const ForwardParams &p);
    cudaError_t init(const DeviceInfo &devinfo, int device, const ForwardParams &params, const HostModel &m);
    cudaError_t forward(const float *x_init, size_t pos, float *logits_host);
    cudaError_t greedy(const void *embd_table, int embd_dtype, uint32_t first_token, size_t pos, size_t n,
                       uint32_t *tokens_host);
    cudaError_t set_kv(size_t pos0, size_t n, const float *k, const float *v);
    // GpuForward::forward_debug (forward.rs:530-635): layer 0 one op at a time, unfused, with the non-finite counts and
    // the largest magnitude of every intermediate.  cudaErrorNotSupported when layer 0 is a mixture-of-experts layer.
    cudaError_t debug_layer0(const float *x_init, size_t pos, DebugStat *out, size_t cap, size_t *n_out);
    float *dbg = nullptr; // scratch of debug_layer0, allocated on first use
    // batched prefill (prefill.cu): all s prompt tokens in one pass, KV cache filled for 0..s-1,
    // logits of the last token
    bool batch_supported() const;
    cudaError_t forward_batch(const float *embeds_host, size_t s, float *logits_host);
    float *bx = nullptr, *bxn = nullptr, *bqk = nullptr, *bv = nullptr, *bh = nullptr;
    void *bscratch = nullptr;
    // mixture-of-experts step: router logits, experts' output, routing scratch; tmpn / tmpo serve the
    // unfused fallback of mv() (normalised input, un-added output)
    float *moe_logits = nullptr, *moe_out = nullptr, *tmpn = nullptr, *tmpo = nullptr;
    void *moe_scratch = nullptr;
    int mlx_table_bytes = 4;
    MlxTables embd_mlx; // tables of the embedding matrix when greedy() is given an MLX 4-bit one (embd_dtype 1000)

  private:
    cudaError_t dev_alloc(void **out, size_t bytes);
    cudaError_t upload(const void *host, size_t bytes, void **out);
    cudaError_t upload_rows(const void *bytes, int fmt, size_t out_dim, size_t cols, Mat *out);
    cudaError_t upload_pair(const HostWeight &a, const HostWeight &b, bool interleave, Mat *out);
    cudaError_t upload_one(const HostWeight &a, Mat *out);
    cudaError_t upload_mlx_stack(const HostWeight *const *ws, int n, Mat *out);
    cudaError_t upload_experts(const MoeExperts &h, MoeExperts *out);
    cudaError_t mv(const Mat &m, const float *in, float *out, const float *norm_w, int epi, const float *res);
    cudaError_t enqueue_step(int mode, const void *embd_table, int embd_dtype);
    cudaError_t run_step(int mode, const void *embd_table, int embd_dtype);
};

} // namespace ullm
