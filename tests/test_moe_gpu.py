"""GPU parity tests for the expert-gathered MoE FFN (MLX 4-bit experts) against
the oracle's restatement of ``moe_ffn`` (crates/ullm-model/src/lib.rs:1453-1488)."""
import os

import numpy as np
import pytest

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_small.npz"))


def make(ne, hid, inter, gs, seed):
    g = synth.gen_mlx4(ne * inter, hid, gs, seed)
    u = synth.gen_mlx4(ne * inter, hid, gs, seed + 1)
    d = synth.gen_mlx4(ne * hid, inter, gs, seed + 2)
    return g, u, d


def widen(t):
    return (t[0], synth.bf16_to_f32(t[1]), synth.bf16_to_f32(t[2]))


def oracle_moe(g, u, d, ne, hid, inter, gs, x, lg, k):
    ex = oracle.Experts(widen(g), widen(u), widen(d), ne, hid, inter, gs)
    return np.stack([oracle.moe_ffn(ex, lg[t], k, x[t]) for t in range(x.shape[0])])


def test_moe_golden_fixture(ctx):
    g, u, d = [(GOLD[f"moe_w{i}"], GOLD[f"moe_s{i}"], GOLD[f"moe_b{i}"]) for i in range(3)]
    ex = backend.Experts(ctx, g, u, d, 4, 128, 64, 64)  # bf16 tables as stored
    y, idx, wts = ex.moe_ffn(GOLD["moe_x"], GOLD["moe_logits"], 2, want_routing=True)
    assert synth.rel_err(y, GOLD["moe_y"]) < TOL
    for t in range(3):
        oi, ow = oracle.moe_topk(GOLD["moe_logits"][t], 2)
        assert idx[t].tolist() == oi.tolist()
        assert np.allclose(wts[t], ow, rtol=1e-5, atol=1e-7)
    ex.free()


@pytest.mark.parametrize("generic", [0, 1])
@pytest.mark.parametrize("f32_tables", [0, 1])
@pytest.mark.parametrize("ne,hid,inter,gs,ntok,k", [
    (8, 256, 128, 64, 3, 2),     # small
    (16, 1024, 96, 32, 8, 4),    # inter not a multiple of the row tile; group 32
    (6, 2048, 128, 128, 11, 3),  # more than 8 tokens: two launch groups; two column groups
    (5, 64, 64, 64, 1, 5),       # every expert chosen by the one token
])
def test_moe_matches_oracle(ctx, ne, hid, inter, gs, ntok, k, f32_tables, generic):
    g, u, d = make(ne, hid, inter, gs, synth.seed_for(2, 3))
    x = synth.normal(synth.seed_for(2, 6), ntok * hid).reshape(ntok, hid)
    lg = synth.router_logits(ntok, ne, min(k, ne - 1), synth.seed_for(2, 7))
    ref = oracle_moe(g, u, d, ne, hid, inter, gs, x, lg, k)
    ex = backend.Experts(ctx, *([widen(t) for t in (g, u, d)] if f32_tables else (g, u, d)), ne, hid, inter, gs)
    ctx.debug_set("force_generic", generic)
    try:
        y = ex.moe_ffn(x, lg, k)
        streamed = ctx.last_plan()["streamed"]
    finally:
        ctx.debug_set("force_generic", 0)
    assert streamed == (0 if generic else 1)
    assert synth.rel_err(y, ref) < TOL
    ex.free()


def test_moe_config2_shape(ctx):
    """128 experts, gate/up [768, 2048], down [2048, 768], group 64, 8 tokens, top-8."""
    ne, hid, inter, gs, ntok, k = 128, 2048, 768, 64, 8, 8
    g, u, d = make(ne, hid, inter, gs, synth.seed_for(2, 0))
    x = synth.normal(synth.seed_for(2, 4), ntok * hid).reshape(ntok, hid)
    lg = synth.router_logits(ntok, ne, k, synth.seed_for(2, 5))
    ex = backend.Experts(ctx, g, u, d, ne, hid, inter, gs)
    y, idx, wts = ex.moe_ffn(x, lg, k, want_routing=True)
    assert ctx.last_plan()["streamed"] == 1
    ref = oracle_moe(g, u, d, ne, hid, inter, gs, x, lg, k)
    assert synth.rel_err(y, ref) < TOL
    assert np.array_equal(idx, np.argsort(-lg, axis=1, kind="stable")[:, :k].astype(np.uint32))
    assert np.allclose(wts.sum(1), 1, atol=1e-5)
    y2 = ex.moe_ffn(x, lg, k)
    assert np.array_equal(y, y2)  # deterministic: slots combined in descending-logit order
    ex.free()


def test_moe_errors(ctx):
    g, u, d = make(4, 128, 64, 64, 1)
    ex = backend.Experts(ctx, g, u, d, 4, 128, 64, 64)
    x, lg = np.zeros((1, 128), np.float32), np.zeros((1, 4), np.float32)
    with pytest.raises(backend.FormatError):
        ex.moe_ffn(x, lg, 5)  # k > n_experts
    with pytest.raises(backend.FormatError):
        ex.moe_ffn(x, lg, 0)
    with pytest.raises(backend.FormatError):
        backend.Experts(ctx, g, u, d, 4, 128, 64, 48)  # hidden not a multiple of the group
    ex.free()
