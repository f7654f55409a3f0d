"""GPU parity tests for the resident decode step against the oracle's restatement
of ``forward_llama`` (crates/ullm-model/src/lib.rs:807-969)."""
import numpy as np
import pytest

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu


def oracle_model(m, kv_f16):
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    return oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16)


@pytest.mark.parametrize("kv_f16", [False, True])
def test_tiny_decode_logits_match_oracle(ctx, kv_f16):
    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 3)
    om = oracle_model(m, kv_f16)
    gf = backend.GpuForward(ctx, m, kv_f16=kv_f16)
    assert not gf.supports_batched_prefill()
    tok = 7
    for pos in range(6):
        ref = om.forward(tok, pos)
        got = gf.forward(om.embed(tok), pos)
        assert synth.rel_err(got, ref) < 1e-3, pos
        assert int(np.argmax(got)) == oracle.argmax(ref)
        tok = oracle.argmax(ref)
    gf.free()


def test_tiny_decode_with_prefilled_cache_and_greedy(ctx):
    """Prefilled f16 cache, then a greedy continuation kept on the device; every
    step is also checked teacher-forced so a near-tie cannot hide later steps."""
    p = dict(synth.LLAMA_TINY)
    p["n_ctx"] = 256
    m = synth.gen_llama_model(p, 5)
    n_pre, n_gen = 100, 24
    k, v = synth.gen_kv_prefill(p, n_pre, 77)
    om = oracle_model(m, True)
    om.key_cache[:, :n_pre] = k
    om.val_cache[:, :n_pre] = v
    gf = backend.GpuForward(ctx, m, kv_f16=True)
    gf.set_kv(0, k, v)
    embd = ctx.upload(m["tok_embd"][1])
    first = 11
    ref_tokens, margins = [], []
    tok = first
    for i in range(n_gen):
        lg = om.forward(tok, n_pre + i)
        s = np.sort(lg)
        margins.append(float(s[-1] - s[-2]))
        tok = oracle.argmax(lg)
        ref_tokens.append(tok)
    got = gf.greedy(embd, m["tok_embd"][0], first, n_pre, n_gen)
    assert got.tolist() == ref_tokens, (got.tolist(), ref_tokens, margins)
    gf.free()


def test_decode_rejects_unbuilt_variants(ctx):
    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 3)
    for flag in ("sandwich_norm", "geglu", "sliding_window", "n_experts"):
        with pytest.raises(backend.Unsupported):
            backend.GpuForward(ctx, m, **{flag: 1})
    with pytest.raises(backend.FormatError):  # qk_norm without the norm vectors
        backend.GpuForward(ctx, m, qk_norm=1)
    bad = dict(m)
    bad["output"] = (backend.F32, m["output"][1], m["output"][2], m["output"][3])
    with pytest.raises(backend.Unsupported):  # forward.rs:376-378
        backend.GpuForward(ctx, bad)
    gf = backend.GpuForward(ctx, m)
    with pytest.raises(backend.FormatError):
        gf.forward(np.zeros(p["n_embd"], np.float32), p["n_ctx"])
    gf.free()


def test_llama_1b_shape_greedy_sequence(ctx):
    """Benchmark configuration 3 at its stated length: Llama-3.2-1B-shaped, Q4_K_M mix, f16 KV prefilled
    with 1024 positions, a 16-token prompt processed token by token, then 128 greedy tokens.

    The oracle's 128 tokens, each step's runner-up and the gap between their logits (relative to the
    largest |logit|, the unit of the 1e-3 logit bar) are a committed fixture
    (tests/golden/c3_decode_128.npz, made by tests/golden/make_c3_decode.py).  Two comparisons:
    the sequence the device generates on its own, and a teacher-forced pass that feeds the oracle's
    tokens so that all 128 steps are compared even if the free-running sequence leaves the oracle's
    at a near-tie.  A step may differ from the oracle only where the oracle's own gap is inside the
    logit tolerance, and then only by picking the runner-up."""
    import os

    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "c3_decode_128.npz"))
    p = dict(synth.LLAMA_1B)
    m = synth.gen_llama_model(p, synth.seed_for(3, 0))
    n_pre, n_prompt, n_gen = 1024, 16, 128
    k, v = synth.gen_kv_prefill(p, n_pre, synth.seed_for(3, 1))
    prompt = synth.rand_ints(synth.seed_for(3, 2), n_prompt, 0, p["vocab"] - 1)
    assert prompt.tolist() == gold["prompt"].tolist()
    om = oracle_model(m, True)
    om.key_cache[:, :n_pre] = k
    om.val_cache[:, :n_pre] = v
    gf = backend.GpuForward(ctx, m, kv_f16=True)
    gf.set_kv(0, k, v)
    for i, t in enumerate(prompt):
        got = gf.forward(om.embed(int(t)), n_pre + i)
        if i < 3:  # logits against the oracle's forward at the first prompt positions (about a second of CPU each)
            assert synth.rel_err(got, om.forward(int(t), n_pre + i)) < 1e-3, i
    first = int(np.argmax(got))
    assert first == int(gold["first"])
    tokens, second, gap = gold["tokens"].tolist(), gold["second"].tolist(), gold["rel_gap"]
    tie = 2e-3  # a GPU logit may be off by 1e-3 of the largest |logit| on either candidate

    embd = ctx.upload(m["tok_embd"][1])
    free = gf.greedy(embd, m["tok_embd"][0], first, n_pre + n_prompt, n_gen).tolist()
    same = next((i for i in range(n_gen) if free[i] != tokens[i]), n_gen)
    if same < n_gen:
        assert gap[same] < tie and free[same] == second[same], (same, free[same], tokens[same], second[same], float(gap[same]))

    prev, swaps = first, []
    for i in range(n_gen):  # teacher-forced: the oracle's token goes in, whatever the device would have picked
        lg = gf.forward(om.embed(prev), n_pre + n_prompt + i)
        a = int(np.argmax(lg))
        if a != tokens[i]:
            assert gap[i] < tie and a == second[i], (i, a, tokens[i], second[i], float(gap[i]))
            swaps.append(i)
        prev = tokens[i]
    assert len(swaps) <= int(np.sum(gap < tie))
    gf.free()


def test_engine_built_from_a_gguf_file_equals_the_one_built_from_arrays(ctx, tmp_path):
    """The GGUF feed (include/ullm_gguf.h -> ullm_cuda_forward_create_gguf): same weights through a
    .gguf file on disk must give bit-identical logits, and a file with tied embeddings or with a
    tensor of an unbuilt variant behaves as LlamaModel::from_gguf says (lib.rs:270-304)."""
    import os

    from ullm_b200 import gguf

    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 11)
    path = os.path.join(tmp_path, "tiny.gguf")
    with open(path, "wb") as f:
        f.write(gguf.llama_to_gguf(m, alignment=64))
    g = gguf.Gguf(path)
    a, b = backend.GpuForward(ctx, m, kv_f16=True), backend.GpuForward.from_gguf(ctx, g, kv_f16=True)
    om = oracle_model(m, True)
    tok = 3
    for pos in range(4):
        x = om.embed(tok)
        la, lb = a.forward(x, pos), b.forward(x, pos)
        assert np.array_equal(la, lb), pos
        assert synth.rel_err(lb, om.forward(tok, pos)) < 1e-3
        tok = int(np.argmax(lb))
    # greedy continuation with the embedding table taken from the file
    t = g.tensor("token_embd.weight")
    embd = ctx.upload(t["data"])
    assert np.array_equal(a.greedy(embd, t["dtype"], tok, 4, 6), b.greedy(embd, t["dtype"], tok, 4, 6))
    a.free(), b.free()
    # a sandwich-norm tensor (Gemma): that variant is not built -> Unsupported, not ignored
    blob = gguf.llama_to_gguf(m)
    g2 = gguf.Gguf(blob)
    ts = [(x["name"], x["dtype"], x["shape"], x["data"].copy()) for x in g2.tensors()]
    ts.append(("blk.0.post_attention_norm.weight", 0, (p["n_embd"],), np.ones(p["n_embd"], np.float32)))
    keys = [(k, gguf.T_STRING if isinstance(g2.get(k), str) else (gguf.T_F32 if isinstance(g2.get(k), float) else gguf.T_U32), g2.get(k)) for k in g2.keys()]
    with pytest.raises(backend.Unsupported):
        backend.GpuForward.from_gguf(ctx, gguf.Gguf(gguf.write_gguf(keys, ts)))
    # tied embeddings: no output.weight -> the embedding matrix is the output projection
    ts_tied = [x for x in ts[:-1] if x[0] != "output.weight"]
    tied = backend.GpuForward.from_gguf(ctx, gguf.Gguf(gguf.write_gguf(keys, ts_tied)))
    m_tied = dict(m, output=m["tok_embd"])
    ref = backend.GpuForward(ctx, m_tied)
    x = om.embed(5)
    assert np.array_equal(tied.forward(x, 0), ref.forward(x, 0))
    tied.free(), ref.free()


def test_gguf_qwen2_biases_and_qk_norms(ctx):
    """LlamaModel::from_gguf reads "qwen2" files and the optional bias / Q-K-norm tensors of any architecture
    (lib.rs:200-209, 277-281); build_gpu turns qk_norm on when layer 0 has the weights (lib.rs:714)."""
    from ullm_b200 import gguf

    p = dict(synth.LLAMA_TINY)
    m = variant_model(p, 31, True, True)
    # the values a file holds: K bias stored as F16, K norm as BF16
    for l in m["layers"]:
        l["k_bias"] = l["k_bias"].astype(np.float16).astype(np.float32)
        l["k_norm"] = synth.bf16_to_f32(synth.f32_to_bf16(l["k_norm"]))
    g = gguf.Gguf(gguf.llama_to_gguf(m, arch="qwen2"))
    assert g.architecture == "qwen2" and g.llama_params()["n_ff"] == p["n_ff"]
    a, b = backend.GpuForward(ctx, m, kv_f16=True, qk_norm=1), backend.GpuForward.from_gguf(ctx, g, kv_f16=True)
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    om = oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, True)
    tok = 11
    for pos in range(4):
        x = om.embed(tok)
        la, lb = a.forward(x, pos), b.forward(x, pos)
        assert np.array_equal(la, lb), pos
        assert synth.rel_err(lb, om.forward(tok, pos)) < 1e-3
        tok = int(np.argmax(lb))
    a.free(), b.free()
    # a file with the Q norm only, or with norms in some layers only, is malformed
    ts = [(x["name"], x["dtype"], x["shape"], x["data"].copy()) for x in g.tensors()]
    keys = [(k, gguf.T_STRING if isinstance(g.get(k), str) else (gguf.T_F32 if isinstance(g.get(k), float) else gguf.T_U32), g.get(k)) for k in g.keys()]
    for dropped in (("blk.0.attn_k_norm.weight",), ("blk.1.attn_q_norm.weight", "blk.1.attn_k_norm.weight")):
        with pytest.raises(backend.FormatError):
            backend.GpuForward.from_gguf(ctx, gguf.Gguf(gguf.write_gguf(keys, [t for t in ts if t[0] not in dropped])))


def variant_model(p, seed, bias, qk_norm):
    m = synth.gen_llama_model(p, seed)
    qd, kvd, hd = p["n_head"] * p["head_dim"], p["n_kv_head"] * p["head_dim"], p["head_dim"]
    for i, l in enumerate(m["layers"]):
        if bias:  # Qwen2-style projection biases (lib.rs:877-885)
            l["q_bias"], l["k_bias"], l["v_bias"] = (synth.normal(900 + 10 * i + j, n) * np.float32(20.0) for j, n in enumerate((qd, kvd, kvd)))
        if qk_norm:  # Qwen3-style per-head Q/K RMSNorm weights (lib.rs:887-901)
            l["q_norm"] = (1.0 + 0.1 * synth.normal(950 + i, hd)).astype(np.float32)
            l["k_norm"] = (1.0 + 0.1 * synth.normal(970 + i, hd)).astype(np.float32)
    return m


@pytest.mark.parametrize("bias,qk_norm,neox,kv_f16", [(True, False, False, True), (False, True, False, False), (False, False, True, True),
                                                      (True, True, True, False)])
def test_decode_variants_bias_qknorm_neox(ctx, bias, qk_norm, neox, kv_f16):
    """The GpuParams / GpuLayerInput options of forward.rs:35-50,86-90 that the dense step carries:
    q/k/v biases, per-head Q/K RMSNorm before RoPE, rotate-half RoPE — each against the oracle."""
    p = dict(synth.LLAMA_TINY)
    m = variant_model(p, 31, bias, qk_norm)
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    om = oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16, rope_neox=neox)
    gf = backend.GpuForward(ctx, m, kv_f16=kv_f16, rope_neox=1 if neox else 0, qk_norm=1 if qk_norm else 0)
    base = backend.GpuForward(ctx, synth.gen_llama_model(p, 31), kv_f16=kv_f16)
    tok, differs = 11, False
    for pos in range(6):
        ref = om.forward(tok, pos)
        got = gf.forward(om.embed(tok), pos)
        assert synth.rel_err(got, ref) < 1e-3, pos
        differs = differs or synth.rel_err(base.forward(om.embed(tok), pos), ref) > 1e-2  # the option is not a no-op
        tok = oracle.argmax(ref)
    assert differs
    gf.free(), base.free()


@pytest.mark.parametrize("hd,n_head,n_kv_head,variant", [(128, 8, 1, False), (128, 2, 2, False), (64, 4, 4, False), (64, 8, 1, False),
                                                         (128, 4, 1, True), (128, 8, 1, True)])
def test_attention_head_shapes_with_a_multi_split_context(ctx, hd, n_head, n_kv_head, variant):
    """Every head geometry the attention kernel is instantiated for (head_dim 64 / 128, 1 to 8 query heads per
    KV head), on a context that spans several 32-position splits, so that the split merge runs; ``variant`` adds
    the per-head Q/K norm and rotate-half RoPE (the Qwen3 path)."""
    p = dict(synth.LLAMA_TINY, head_dim=hd, n_head=n_head, n_kv_head=n_kv_head, n_ctx=160)
    m = variant_model(p, 41, False, variant)
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    n_pre = 70
    k, v = synth.gen_kv_prefill(p, n_pre, 77)
    for kv_f16 in (True, False):
        om = oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16, rope_neox=variant)
        om.key_cache[:, :n_pre], om.val_cache[:, :n_pre] = k, v  # values that are exact in f16
        gf = backend.GpuForward(ctx, m, kv_f16=kv_f16, rope_neox=1 if variant else 0, qk_norm=1 if variant else 0)
        gf.set_kv(0, k, v)
        tok = 5
        for pos in range(n_pre, n_pre + 5):
            ref = om.forward(tok, pos)
            got = gf.forward(om.embed(tok), pos)
            assert synth.rel_err(got, ref) < 1e-3, (kv_f16, pos)
            tok = oracle.argmax(ref)
        gf.free()


@pytest.mark.parametrize("variant", ["llama", "qk_norm_neox"])
def test_forward_debug_walks_layer_0_like_the_reference(ctx, variant):
    """``GpuForward::forward_debug`` (crates/ullm-metal/src/forward.rs:530-635): layer 0 op by op.  Labels and order are
    the reference's; every intermediate's largest magnitude must agree with the oracle's walk of the same ops, and a
    NaN planted in the input must show up in the counts instead of disappearing."""
    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 13)
    flags = {}
    if variant == "qk_norm_neox":
        for i, l in enumerate(m["layers"]):
            l["q_norm"] = 1.0 + 0.1 * synth.normal(900 + i, p["head_dim"])
            l["k_norm"] = 1.0 + 0.1 * synth.normal(950 + i, p["head_dim"])
        flags = dict(rope_neox=1, qk_norm=1)
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    om = oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, True, rope_neox=bool(flags))
    gf = backend.GpuForward(ctx, m, kv_f16=True, **flags)
    x = om.embed(5)
    for pos in (0, 1, 2):  # each walk writes K / V of its position, so later positions attend to earlier ones
        ref = om.forward_debug(x, pos)
        got = gf.forward_debug(x, pos)
        assert [g[0] for g in got] == [r[0] for r in ref]
        for (label, nan, inf, mx), (_, rmx) in zip(got, ref):
            assert nan == 0 and inf == 0, label
            assert abs(mx - rmx) <= 1e-3 * max(rmx, 1e-6), (pos, label, mx, rmx)
    bad = x.copy()
    bad[3] = np.nan
    got = dict((g[0], g) for g in gf.forward_debug(bad, 3))
    assert got["x_init"][1] == 1 and got["attn_norm"][1] == p["n_embd"] and got["w_down"][1] > 0
    gf.free()
