"""Seeded synthetic weights and activations in the on-disk formats of the path.

Real GGUF / MLX model files are not available, so every workload is generated:
GGUF ``block_q4_K`` / ``block_q6_K`` super-blocks and MLX 4-bit affine groups
with the value distributions the benchmark configurations name.  Random numbers
come from a counter-based SplitMix64 (constants as in the reference's sampler,
crates/ullm-model/src/sample.rs:136-142), so any slice of a stream can be
produced independently and the same seed gives the same bytes everywhere.
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

Q4K_BLOCK_BYTES = 144
Q6K_BLOCK_BYTES = 210
QK_K = 256


def seed_for(config: int, stream: int) -> int:
    return 0x5EED0000 + 16 * config + stream


def splitmix64(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """Outputs ``offset .. offset+n`` of the SplitMix64 stream started at ``seed``."""
    with np.errstate(over="ignore"):
        i = np.arange(offset + 1, offset + n + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int) -> np.ndarray:
    """f64 uniform in [0, 1) from the top 53 bits."""
    return (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def uniform_range(seed: int, n: int, lo: float, hi: float) -> np.ndarray:
    return lo + (hi - lo) * uniform(seed, n)


def normal(seed: int, n: int) -> np.ndarray:
    """N(0,1) as f32 (Box-Muller in f64)."""
    m = (n + 1) // 2
    u = uniform(seed, 2 * m)
    u1 = 1.0 - u[:m]  # (0, 1]
    u2 = u[m:]
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])[:n]
    return out.astype(np.float32)


def rand_bytes(seed: int, n: int) -> np.ndarray:
    m = (n + 7) // 8
    return splitmix64(seed, m).view(np.uint8)[:n].copy()


def rand_ints(seed: int, n: int, lo: int, hi_incl: int) -> np.ndarray:
    span = hi_incl - lo + 1
    return (lo + (splitmix64(seed, n) >> np.uint64(33)).astype(np.int64) % span).astype(np.int64)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    """Exact widening (crates/ullm-core/src/dequant.rs:286)."""
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of ``scale_min_k4`` (dequant.rs:41-49): eight 6-bit (scale, min)
    pairs per block -> the 12 packed bytes.  ``sc``/``mn``: [..., 8] in 0..63."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    q = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    for j in range(4):
        q[..., j] = sc[..., j] | ((sc[..., j + 4] >> 4) << 6)
        q[..., j + 4] = mn[..., j] | ((mn[..., j + 4] >> 4) << 6)
        q[..., j + 8] = (sc[..., j + 4] & 15) | ((mn[..., j + 4] & 15) << 4)
    return q


def gen_q4k(rows: int, cols: int, seed: int) -> np.ndarray:
    """``[rows, cols/256*144]`` bytes: f16 d, dmin ~ U(0.001, 0.05); 6-bit scales
    and mins uniform in 0..63; 128 uniform random quant bytes."""
    assert cols % QK_K == 0
    nb = rows * (cols // QK_K)
    blk = np.empty((nb, Q4K_BLOCK_BYTES), np.uint8)
    dd = uniform_range(seed, 2 * nb, 0.001, 0.05).astype(np.float16).view(np.uint8).reshape(nb, 4)
    blk[:, 0:4] = dd
    sm = rand_ints(seed + 0x1000, 16 * nb, 0, 63).reshape(nb, 16)
    blk[:, 4:16] = pack_scales_k4(sm[:, :8], sm[:, 8:])
    blk[:, 16:144] = rand_bytes(seed + 0x2000, 128 * nb).reshape(nb, 128)
    return blk.reshape(rows, -1)


def gen_q6k(rows: int, cols: int, seed: int) -> np.ndarray:
    """``[rows, cols/256*210]`` bytes: 128 B low nibbles + 64 B high bits uniform,
    16 int8 scales uniform in -128..127, f16 d ~ U(0.0005, 0.01)."""
    assert cols % QK_K == 0
    nb = rows * (cols // QK_K)
    blk = np.empty((nb, Q6K_BLOCK_BYTES), np.uint8)
    blk[:, 0:192] = rand_bytes(seed + 0x2000, 192 * nb).reshape(nb, 192)
    blk[:, 192:208] = rand_ints(seed + 0x1000, 16 * nb, -128, 127).astype(np.int8).view(np.uint8).reshape(nb, 16)
    blk[:, 208:210] = uniform_range(seed, nb, 0.0005, 0.01).astype(np.float16).view(np.uint8).reshape(nb, 2)
    return blk.reshape(rows, -1)


def gen_mlx4(out: int, cols: int, group: int, seed: int):
    """MLX 4-bit affine: words u32 ``[out, cols/8]`` uniform, bf16 scale ~
    U(0.005, 0.03) and bias ~ U(-0.1, 0.1) per group (returned as bf16 bits)."""
    assert cols % 8 == 0 and cols % group == 0
    words = splitmix64(seed + 0x2000, (out * (cols // 8) + 1) // 2).view(np.uint32)[: out * (cols // 8)].copy()
    ng = out * (cols // group)
    scales = f32_to_bf16(uniform_range(seed, ng, 0.005, 0.03).astype(np.float32))
    biases = f32_to_bf16(uniform_range(seed + 0x1000, ng, -0.1, 0.1).astype(np.float32))
    return words.reshape(out, cols // 8), scales.reshape(out, -1), biases.reshape(out, -1)


def router_logits(n_tok: int, n_experts: int, k: int, seed: int) -> np.ndarray:
    """Seeded N(0,1) router logits with no tie among each token's top ``k+1``."""
    lg = normal(seed, n_tok * n_experts).reshape(n_tok, n_experts)
    top = -np.sort(-lg, axis=1)[:, : k + 1]
    assert (np.diff(top, axis=1) < 0).all(), "tie in the router's top-k"
    return lg


# The reference's own GPU-vs-CPU unit-test generators
# (crates/ullm-metal/src/lib.rs:358-391 and :395-412).
def check_quant_weights(dtype_block_bytes: int, d_offsets, out: int = 256, cols: int = 512) -> np.ndarray:
    total = out * (cols // QK_K) * dtype_block_bytes
    k = np.arange(total, dtype=np.uint64)
    w = ((k * np.uint64(131) + np.uint64(7)) % np.uint64(251)).astype(np.uint8).reshape(-1, dtype_block_bytes)
    for off in d_offsets:  # f16 0x3000 = 0.125, little-endian
        w[:, off] = 0x00
        w[:, off + 1] = 0x30
    return w.reshape(out, -1)


def check_quant_x(cols: int = 512) -> np.ndarray:
    return ((np.arange(cols) % 13).astype(np.float32) - np.float32(6.0)) * np.float32(0.1)


def check_mlx4(out: int = 96, cols: int = 256, group: int = 64):
    words = cols // 8
    k = np.arange(out * words * 4, dtype=np.uint64)
    w = ((k * np.uint64(131) + np.uint64(7)) % np.uint64(251)).astype(np.uint8).view(np.uint32).reshape(out, words)
    g = np.arange(out * (cols // group))
    scales = ((g % 7).astype(np.float32) - np.float32(3.0)) * np.float32(0.01)
    biases = ((g % 5).astype(np.float32) - np.float32(2.0)) * np.float32(0.02)
    return w, scales.reshape(out, -1), biases.reshape(out, -1)


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """The reference's own metric (crates/ullm-metal/src/lib.rs:336-343):
    max|got-ref| / max(max|ref|, 1e-6)."""
    got = np.asarray(got, np.float32).reshape(-1)
    ref = np.asarray(ref, np.float32).reshape(-1)
    scale = max(float(np.max(np.abs(ref))) if ref.size else 0.0, 1e-6)
    return (float(np.max(np.abs(got - ref))) if ref.size else 0.0) / scale


# ---- synthetic Llama-shaped model (GGUF Q4_K_M mix) -------------------------
Q4_K, Q6_K = 12, 14  # ggml type ids

LLAMA_1B = dict(n_embd=2048, n_layer=16, n_head=32, n_kv_head=8, head_dim=64, n_ff=8192, n_ctx=1280, vocab=128256,
                rope_theta=500000.0, eps=1e-5)
LLAMA_TINY = dict(n_embd=256, n_layer=2, n_head=4, n_kv_head=2, head_dim=64, n_ff=512, n_ctx=64, vocab=512,
                  rope_theta=500000.0, eps=1e-5)


def gen_weight(dtype: int, out: int, cols: int, seed: int) -> np.ndarray:
    return gen_q4k(out, cols, seed) if dtype == Q4_K else gen_q6k(out, cols, seed)


def gen_llama_model(p: dict, seed: int) -> dict:
    """Random weights in the Q4_K_M mix: Q6_K for attn_v / ffn_down / output,
    Q4_K elsewhere (token_embd included); norms f32 = 1 + 0.1 N(0,1).  Tensor
    shapes as the GGUF loader builds them (crates/ullm-model/src/lib.rs:270-301).
    Returns ``{"params", "tok_embd": (dtype, bytes), "output": ..., "final_norm",
    "layers": [{"attn_norm", "ffn_norm", "wq": (dtype, bytes, out, cols), ...}]}``."""
    e, hd = p["n_embd"], p["head_dim"]
    qd, kvd, ff = p["n_head"] * hd, p["n_kv_head"] * hd, p["n_ff"]
    s = [seed * 1000]

    def nxt():
        s[0] += 7
        return s[0]

    def w(dtype, out, cols):
        return (dtype, gen_weight(dtype, out, cols, nxt()), out, cols)

    def norm(n):
        return (np.float32(1.0) + np.float32(0.1) * normal(nxt(), n)).astype(np.float32)

    layers = []
    for _ in range(p["n_layer"]):
        layers.append(dict(
            attn_norm=norm(e), ffn_norm=norm(e),
            wq=w(Q4_K, qd, e), wk=w(Q4_K, kvd, e), wv=w(Q6_K, kvd, e), wo=w(Q4_K, e, qd),
            w_gate=w(Q4_K, ff, e), w_up=w(Q4_K, ff, e), w_down=w(Q6_K, e, ff),
        ))
    return dict(params=dict(p), tok_embd=w(Q4_K, p["vocab"], e), output=w(Q6_K, p["vocab"], e), final_norm=norm(e),
                layers=layers)


def gen_kv_prefill(p: dict, n_pos: int, seed: int):
    """K and V for positions 0..n_pos of every layer ~ N(0,1) rounded to f16,
    as f32 arrays [n_layer, n_pos, kv_dim]."""
    kvd = p["n_kv_head"] * p["head_dim"]
    n = p["n_layer"] * n_pos * kvd
    k = normal(seed, n).astype(np.float16).astype(np.float32).reshape(p["n_layer"], n_pos, kvd)
    v = normal(seed + 1, n).astype(np.float16).astype(np.float32).reshape(p["n_layer"], n_pos, kvd)
    return k, v


QWEN3MOE_TINY = dict(n_embd=256, n_layer=2, n_head=4, n_kv_head=2, head_dim=64, n_ff=0, n_ctx=64, vocab=512, rope_theta=1000000.0,
                     eps=1e-6, n_experts=8, n_experts_used=2, moe_inter=128, group=64)
# Qwen3-30B-A3B's shape (crates/ullm-model/src/mlx.rs:117-141 reads it from config.json), with fewer layers by default
QWEN3MOE_30B = dict(n_embd=2048, n_layer=48, n_head=32, n_kv_head=4, head_dim=128, n_ff=0, n_ctx=1280, vocab=151936,
                    rope_theta=1000000.0, eps=1e-6, n_experts=128, n_experts_used=8, moe_inter=768, group=64)


def gen_qwen3moe_model(p: dict, seed: int) -> dict:
    """Random MLX 4-bit Qwen3-MoE weights laid out as ``LlamaModel::from_mlx`` builds them
    (crates/ullm-model/src/mlx.rs:143-213): every linear ``(MLX_U32, words, out, cols, scales, biases, group)``
    with bf16 tables as bits, norms = bf16-exact 1 + 0.1 N(0,1), per layer a router ``moe_gate`` and the
    stacked experts ``{"gate", "up", "down": (words, scales, biases), n_experts, hidden, inter, group}``."""
    e, hd, g = p["n_embd"], p["head_dim"], p["group"]
    qd, kvd, ne, mi = p["n_head"] * hd, p["n_kv_head"] * hd, p["n_experts"], p["moe_inter"]
    s = [seed * 1000 + 0x77000]

    def nxt():
        s[0] += 7
        return s[0]

    def mlx(out, cols):
        # biases near -7.5 * scale centre the 4-bit values: with the all-positive weights of gen_mlx4 every
        # activation would be dominated by one common component and the logits would not depend on the position
        words, sc, bi = gen_mlx4(out, cols, g, nxt())
        bi = f32_to_bf16((np.float32(-7.5) * bf16_to_f32(sc) + np.float32(0.1) * bf16_to_f32(bi)).astype(np.float32))
        return words, sc, bi

    def w(out, cols):
        words, sc, bi = mlx(out, cols)
        return (1000, words, out, cols, sc, bi, g)

    def norm(n):
        return bf16_to_f32(f32_to_bf16((np.float32(1.0) + np.float32(0.1) * normal(nxt(), n)).astype(np.float32)))

    layers = []
    for _ in range(p["n_layer"]):
        layers.append(dict(
            attn_norm=norm(e), ffn_norm=norm(e), q_norm=norm(hd), k_norm=norm(hd),
            wq=w(qd, e), wk=w(kvd, e), wv=w(kvd, e), wo=w(e, qd), moe_gate=w(ne, e),
            experts=dict(gate=mlx(ne * mi, e), up=mlx(ne * mi, e), down=mlx(ne * e, mi),
                         n_experts=ne, hidden=e, inter=mi, group=g),
        ))
    return dict(params=dict(p), tok_embd=w(p["vocab"], e), output=w(p["vocab"], e), final_norm=norm(e), layers=layers)
