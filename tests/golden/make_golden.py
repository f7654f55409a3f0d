"""Regenerates the committed golden fixtures of this directory.

Two kinds of fixture:

* ``reference_kats.json`` — the known answers the reference's own unit tests
  hold for this path, transcribed from its test code (the reference is Rust and
  cannot be executed here): f16 widening (crates/ullm-core/src/dequant.rs:337-342),
  the MLX 4-bit word captured from mlx.dequantize (:324-334), the Q8_0 and Q4_0
  closed forms (:345-367), the short-buffer error (:370-373), the F32 matvec
  identity and the matmul == stacked-matvec case
  (crates/ullm-model/src/math.rs:192-233).  Hand-written, not produced by a run.
* ``oracle_small.npz`` — outputs of the C oracle (oracle/ullm_oracle.c) on small
  seeded inputs, so that the GPU tests also have fixed vectors that do not depend
  on building the oracle.  Produced by running this script:
      python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from ullm_b200 import synth  # noqa: E402

KATS = {
    "f16": [[0x0000, 0.0], [0x3C00, 1.0], [0x4000, 2.0], [0xC000, -2.0]],
    "mlx_q4": {
        "word": 2569837433, "scale": 0.004425049, "bias": -0.039794922, "group": 64,
        "expect": [3e-5, -0.00882, 0.00888, 3e-5, 0.01331, -0.03094, 3e-5, 3e-5], "abs_tol": 1e-4,
    },
    "q8_0": {"d_bits": 0x4000, "qs": list(range(32)), "expect_scale": 2.0, "abs_tol": 1e-4},
    "q4_0": {"d_bits": 0x3C00, "qs_byte": 0x80, "expect_first16": -8.0, "expect_last16": 0.0, "abs_tol": 1e-4},
    "short_buffer": {"dtype": "Q8_0", "len": 10, "n": 32, "error": "Format"},
    "matvec_identity": {"w": [1.0, 0.0, 0.0, 1.0], "x": [3.0, 5.0], "y": [3.0, 5.0]},
    "matmul_stacked": {"w": [[1.0, 2.0], [3.0, 4.0], [-1.0, 0.5]], "xs": [1.0, 0.0, 0.5, -2.0, 3.0, 3.0], "s_len": 3},
}


def main():
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(KATS, f, indent=1)

    out = {}
    # dequantization + matvec on small seeded matrices, incl. a ragged row count
    for name, dt, gen, rows, cols in (("q4k", oracle.Q4_K, synth.gen_q4k, 24, 1024), ("q6k", oracle.Q6_K, synth.gen_q6k, 24, 1024)):
        w = gen(rows, cols, synth.seed_for(9, 0))
        x = synth.normal(synth.seed_for(9, 1), cols)
        out[f"{name}_w"] = w
        out[f"{name}_x"] = x
        out[f"{name}_deq"] = oracle.dequantize(dt, w, rows * cols)
        W = oracle.Weight(dt, w, rows, cols)
        out[f"{name}_y"] = oracle.matvec_q(W, x)
        xs = synth.normal(synth.seed_for(9, 2), 5 * cols).reshape(5, cols)
        out[f"{name}_xs"] = xs
        out[f"{name}_ys"] = oracle.matmul_q(W, xs, 5)
    words, sc, bi = synth.gen_mlx4(24, 512, 64, synth.seed_for(9, 3))
    s32, b32 = synth.bf16_to_f32(sc), synth.bf16_to_f32(bi)
    x = synth.normal(synth.seed_for(9, 4), 512)
    out["mlx_w"], out["mlx_s"], out["mlx_b"], out["mlx_x"] = words, sc, bi, x
    out["mlx_deq"] = oracle.dequantize_mlx_q4(words, s32, b32, 24, 512, 64)
    out["mlx_y"] = oracle.matvec_q(oracle.Weight(oracle.MLX_U32, words, 24, 512, s32, b32, 64), x)

    # MoE: 4 experts of [64, 128] / [128, 64], group 64, 3 tokens, top-2
    ne, hid, inter, gs, ntok, k = 4, 128, 64, 64, 3, 2
    g = synth.gen_mlx4(ne * inter, hid, gs, synth.seed_for(9, 5))
    u = synth.gen_mlx4(ne * inter, hid, gs, synth.seed_for(9, 6))
    d = synth.gen_mlx4(ne * hid, inter, gs, synth.seed_for(9, 7))
    ex = oracle.Experts(*[(t[0], synth.bf16_to_f32(t[1]), synth.bf16_to_f32(t[2])) for t in (g, u, d)], ne, hid, inter, gs)
    xt = synth.normal(synth.seed_for(9, 8), ntok * hid).reshape(ntok, hid)
    lg = synth.router_logits(ntok, ne, k, synth.seed_for(9, 9))
    for i, t in enumerate((g, u, d)):
        out[f"moe_w{i}"], out[f"moe_s{i}"], out[f"moe_b{i}"] = t
    out["moe_x"], out["moe_logits"] = xt, lg
    out["moe_y"] = np.stack([oracle.moe_ffn(ex, lg[t], k, xt[t]) for t in range(ntok)])

    # rmsnorm / rope / softmax / silu vectors
    v = synth.normal(synth.seed_for(9, 10), 256)
    wn = (1 + 0.1 * synth.normal(synth.seed_for(9, 11), 256)).astype(np.float32)
    out["norm_x"], out["norm_w"], out["norm_y"] = v, wn, oracle.rmsnorm(v, wn, 1e-5)
    out["rope_y"] = oracle.rope(v, 4, 64, 64, 1031, 500000.0)
    out["softmax_y"] = oracle.softmax(v[:37])
    out["silu_y"] = np.array([oracle.silu(float(t)) for t in v[:16]], np.float32)
    np.savez_compressed(os.path.join(HERE, "oracle_small.npz"), **out)
    print("wrote", sorted(out))


if __name__ == "__main__":
    main()
