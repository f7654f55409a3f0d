"""GPU parity tests for the decode step with mixture-of-experts layers and MLX 4-bit matrices (the Qwen3-MoE
path: GpuForward with moe_gate / experts, crates/ullm-metal/src/forward.rs:484-494) against the oracle's
restatement of ``forward_llama`` + ``moe_ffn`` (crates/ullm-model/src/lib.rs:807-969, 1453-1488), and for the
engine built straight from an MLX model directory (``LlamaModel::from_mlx``, crates/ullm-model/src/mlx.rs:103-232)."""
import os

import numpy as np
import pytest

import oracle
from ullm_b200 import backend, safetensors as stm, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3


def oracle_model(m, kv_f16):
    """The same weights for the oracle: tables widened to f32 as the reference does at load (mlx.rs:17-26)."""
    def mk(t):
        return oracle.Weight(t[0], t[1], t[2], t[3], synth.bf16_to_f32(t[4]), synth.bf16_to_f32(t[5]), t[6])

    def wide(t):
        return (t[0], synth.bf16_to_f32(t[1]), synth.bf16_to_f32(t[2]))

    layers = []
    for l in m["layers"]:
        x = l["experts"]
        d = {k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items() if k != "experts"}
        d["experts"] = oracle.Experts(wide(x["gate"]), wide(x["up"]), wide(x["down"]), x["n_experts"], x["hidden"], x["inter"], x["group"])
        d["n_experts_used"] = m["params"]["n_experts_used"]
        layers.append(d)
    return oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16, rope_neox=True)


@pytest.mark.parametrize("kv_f16", [False, True])
def test_tiny_qwen3moe_decode_matches_oracle(ctx, kv_f16):
    p = dict(synth.QWEN3MOE_TINY)
    m = synth.gen_qwen3moe_model(p, 3)
    om = oracle_model(m, kv_f16)
    gf = backend.GpuForward(ctx, m, kv_f16=kv_f16, rope_neox=1, qk_norm=1)
    assert not gf.supports_batched_prefill()
    tok = 7
    for pos in range(6):
        ref = om.forward(tok, pos)
        got = gf.forward(om.embed(tok), pos)
        assert synth.rel_err(got, ref) < TOL, pos
        assert int(np.argmax(got)) == oracle.argmax(ref)
        tok = oracle.argmax(ref)
    gf.free()


def test_qwen3moe_greedy_tokens_on_the_device(ctx, tmp_path):
    """A greedy continuation with the MLX embedding lookup, the argmax and the bookkeeping on the device; the
    embedding matrix comes from the model directory.  Teacher-forced check of every step beside it."""
    p = dict(synth.QWEN3MOE_TINY)
    m = synth.gen_qwen3moe_model(p, 3)
    d = os.path.join(tmp_path, "qwen3moe")
    stm.qwen3moe_to_dir(d, m)
    st = stm.SafeTensors(d)
    om = oracle_model(m, True)
    gf = backend.GpuForward.from_safetensors(ctx, st, kv_f16=True)
    embd = backend.Weight.from_safetensors(ctx, st, "model.embed_tokens", p["group"])
    n_gen, first = 20, 11
    ref_tokens, margins, tok = [], [], first
    for i in range(n_gen):
        lg = om.forward(tok, i)
        srt = np.sort(lg)
        margins.append(float(srt[-1] - srt[-2]))
        tok = oracle.argmax(lg)
        ref_tokens.append(tok)
    got = gf.greedy_weight(embd, first, 0, n_gen)
    assert got.tolist() == ref_tokens, (got.tolist(), ref_tokens, margins)
    gf.free(), embd.free()


def test_engine_built_from_an_mlx_directory(ctx, tmp_path):
    p = dict(synth.QWEN3MOE_TINY)
    m = synth.gen_qwen3moe_model(p, 5)
    d = os.path.join(tmp_path, "qwen3moe")
    stm.qwen3moe_to_dir(d, m)
    st = stm.SafeTensors(d)
    assert st.n_shards == 2
    a = backend.GpuForward(ctx, m, kv_f16=True, rope_neox=1, qk_norm=1)
    b = backend.GpuForward.from_safetensors(ctx, st, kv_f16=True)
    om = oracle_model(m, True)
    tok = 3
    for pos in range(4):
        x = om.embed(tok)
        la, lb = a.forward(x, pos), b.forward(x, pos)
        assert np.array_equal(la, lb), pos  # the same bytes on the device -> the same bits out
        assert synth.rel_err(lb, om.forward(tok, pos)) < TOL
        tok = int(np.argmax(lb))
    a.free(), b.free()
    # a directory of another architecture, and one with a tensor missing
    import json

    cfg = json.load(open(os.path.join(d, "config.json")))
    json.dump(dict(cfg, architectures=["LlamaForCausalLM"]), open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(backend.Unsupported):
        backend.GpuForward.from_safetensors(ctx, stm.SafeTensors(d))
    json.dump(dict(cfg, num_hidden_layers=3), open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(backend.FormatError) as e:
        backend.GpuForward.from_safetensors(ctx, stm.SafeTensors(d))
    assert "model.layers.2" in str(e.value)


def test_moe_forward_argument_checks(ctx):
    p = dict(synth.QWEN3MOE_TINY)
    m = synth.gen_qwen3moe_model(p, 3)
    with pytest.raises(backend.FormatError):  # experts given, params say none
        backend.GpuForward(ctx, dict(m, params=dict(p, n_experts=0, n_experts_used=0, moe_inter=0, n_ff=512)), rope_neox=1, qk_norm=1)
    with pytest.raises(backend.Unsupported):  # more experts per token than experts
        backend.GpuForward(ctx, dict(m, params=dict(p, n_experts_used=9)), rope_neox=1, qk_norm=1)
    bad = dict(m, layers=[dict(l) for l in m["layers"]])
    bad["layers"][1]["experts"] = dict(bad["layers"][1]["experts"], inter=64)
    with pytest.raises(backend.FormatError):
        backend.GpuForward(ctx, bad, rope_neox=1, qk_norm=1)
