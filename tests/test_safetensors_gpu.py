"""GPU tests of the SafeTensors / MLX feed: resident weights and stacked experts made straight from an
open model directory (``ullm_cuda_weight_create_st`` / ``ullm_cuda_experts_create_st``) against the same
objects made from arrays and against the oracle (mlx_qweight / mlx_experts, crates/ullm-model/src/mlx.rs:30-88;
moe_ffn, crates/ullm-model/src/lib.rs:1453-1488)."""
import os

import numpy as np
import pytest

import oracle
from ullm_b200 import backend, safetensors as stm, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3

CFG = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 1024, "num_attention_heads": 8, "num_hidden_layers": 2,
       "num_key_value_heads": 2, "head_dim": 128, "num_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 96,
       "vocab_size": 512, "quantization": {"group_size": 32, "bits": 4}}


def widen(t):
    return (t[0], synth.bf16_to_f32(t[1]), synth.bf16_to_f32(t[2]))


def build_dir(path):
    """Two MoE layers in two shards plus one attention projection, laid out like an MLX Qwen3-MoE directory."""
    p = CFG
    ne, hid, inter, gs = p["num_experts"], p["hidden_size"], p["moe_intermediate_size"], p["quantization"]["group_size"]
    arrays, shards = {}, {}
    for layer in range(2):
        ts = []
        for j, (name, o, i) in enumerate((("gate_proj", inter, hid), ("up_proj", inter, hid), ("down_proj", hid, inter))):
            w, s, b = synth.gen_mlx4(ne * o, i, gs, synth.seed_for(2, 40 + 10 * layer + j))
            arrays[(layer, name)] = (w, s, b)
            ts += stm.mlx_linear_tensors(f"model.layers.{layer}.mlp.switch_mlp.{name}", w.reshape(ne, o, i // 8), s.reshape(ne, o, -1), b.reshape(ne, o, -1))
        shards[f"model-0000{layer + 1}-of-00002.safetensors"] = ts
    q = synth.gen_mlx4(p["num_attention_heads"] * p["head_dim"], hid, gs, synth.seed_for(2, 70))
    arrays["q"] = q
    shards["model-00001-of-00002.safetensors"] += stm.mlx_linear_tensors("model.layers.0.self_attn.q_proj", *q)
    stm.write_model_dir(path, CFG, shards)
    return arrays


def test_experts_and_weights_from_a_model_directory(ctx, tmp_path):
    d = os.path.join(tmp_path, "qwen3moe")
    arrays = build_dir(d)
    st = stm.SafeTensors(d)
    p = st.mlx_params()
    ne, hid, inter, gs, k = p["n_experts"], p["n_embd"], p["moe_inter"], p["group"], p["n_experts_used"]
    assert (ne, hid, inter, gs, k) == (16, 1024, 96, 32, 4)
    ntok = 5
    x = synth.normal(synth.seed_for(2, 80), ntok * hid).reshape(ntok, hid)
    lg = synth.router_logits(ntok, ne, k, synth.seed_for(2, 81))
    for layer in range(2):
        g, u, dn = (arrays[(layer, n)] for n in ("gate_proj", "up_proj", "down_proj"))
        from_file = backend.Experts.from_safetensors(ctx, st, f"model.layers.{layer}.mlp.switch_mlp", ne, hid, inter, gs)
        from_arrays = backend.Experts(ctx, g, u, dn, ne, hid, inter, gs)
        ya, yb = from_file.moe_ffn(x, lg, k), from_arrays.moe_ffn(x, lg, k)
        assert np.array_equal(ya, yb), layer  # same bytes on the device -> the same bits out
        ex = oracle.Experts(widen(g), widen(u), widen(dn), ne, hid, inter, gs)
        ref = np.stack([oracle.moe_ffn(ex, lg[t], k, x[t]) for t in range(ntok)])
        assert synth.rel_err(ya, ref) < TOL
        from_file.free(), from_arrays.free()
    qw, qs, qb = arrays["q"]
    w = backend.Weight.from_safetensors(ctx, st, "model.layers.0.self_attn.q_proj", gs)
    assert (w.out, w.cols) == (1024, 1024)
    w2 = backend.Weight(ctx, backend.MLX_U32, qw, 1024, 1024, qs, qb, gs)
    y, y2 = w.matvec(x[0]), w2.matvec(x[0])
    assert np.array_equal(y, y2)
    ow = oracle.Weight(backend.MLX_U32, qw, 1024, 1024, synth.bf16_to_f32(qs), synth.bf16_to_f32(qb), gs)
    assert synth.rel_err(y, oracle.matvec_q(ow, x[0])) < TOL
    w.free(), w2.free()
    # errors surface as FormatError with the reader's message, nothing half-built is left behind
    with pytest.raises(backend.FormatError) as e:
        backend.Experts.from_safetensors(ctx, st, "model.layers.7.mlp.switch_mlp", ne, hid, inter, gs)
    assert "missing tensor" in str(e.value)
    with pytest.raises(backend.FormatError):
        backend.Experts.from_safetensors(ctx, st, "model.layers.0.mlp.switch_mlp", ne + 1, hid, inter, gs)
    with pytest.raises(backend.FormatError):
        backend.Weight.from_safetensors(ctx, st, "model.layers.0.self_attn.k_proj", gs)
