"""CPU tests: the oracle against the reference's own known answers, against an
independent second statement of the formats, and against the committed fixtures."""
import json
import os

import numpy as np
import pytest

import np_formats as nf
import oracle
from ullm_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden")
KATS = json.load(open(os.path.join(GOLD, "reference_kats.json")))


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLD, "oracle_small.npz"))


# ---- known answers transcribed from the reference's unit tests -----------------
def test_f16_widening_kat():  # dequant.rs:337-342
    for bits, val in KATS["f16"]:
        assert oracle.f16_to_f32(bits) == val


def test_f16_widening_is_ieee_for_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    ours = oracle.dequantize(oracle.F16, bits, 65536)
    ieee = bits.view(np.float16).astype(np.float32)
    assert np.array_equal(np.isnan(ours), np.isnan(ieee))
    ok = ~np.isnan(ieee)
    assert np.array_equal(ours[ok].view(np.uint32), ieee[ok].view(np.uint32))


def test_mlx_q4_kat():  # dequant.rs:324-334 (captured from mlx.dequantize)
    k = KATS["mlx_q4"]
    y = oracle.dequantize_mlx_q4([k["word"]], [k["scale"]], [k["bias"]], 1, 8, k["group"])[0]
    assert np.all(np.abs(y - np.array(k["expect"], np.float32)) < k["abs_tol"])


def test_q8_0_kat():  # dequant.rs:345-353
    k = KATS["q8_0"]
    data = bytes([k["d_bits"] & 0xFF, k["d_bits"] >> 8] + k["qs"])
    out = oracle.dequantize(oracle.Q8_0, np.frombuffer(data, np.uint8), 32)
    assert np.all(np.abs(out - k["expect_scale"] * np.arange(32)) < k["abs_tol"])


def test_q4_0_kat():  # dequant.rs:355-367
    k = KATS["q4_0"]
    data = bytes([k["d_bits"] & 0xFF, k["d_bits"] >> 8] + [k["qs_byte"]] * 16)
    out = oracle.dequantize(oracle.Q4_0, np.frombuffer(data, np.uint8), 32)
    assert np.all(np.abs(out[:16] - k["expect_first16"]) < k["abs_tol"])
    assert np.all(np.abs(out[16:] - k["expect_last16"]) < k["abs_tol"])


def test_short_buffer_and_ragged_count_are_format_errors():  # dequant.rs:65-77, :370-373
    with pytest.raises(oracle.OracleError) as e:
        oracle.dequantize(oracle.Q8_0, np.zeros(10, np.uint8), 32)
    assert e.value.code == oracle.ERR_FORMAT
    with pytest.raises(oracle.OracleError) as e:
        oracle.dequantize(oracle.Q4_K, np.zeros(144, np.uint8), 255)
    assert e.value.code == oracle.ERR_FORMAT
    with pytest.raises(oracle.OracleError) as e:  # U32 has no block dequantizer: dequant.rs:103-107
        oracle.dequantize(oracle.MLX_U32, np.zeros(16, np.uint8), 4)
    assert e.value.code == oracle.ERR_UNSUPPORTED
    assert oracle.dequantize(oracle.Q4_K, np.zeros(0, np.uint8), 0).size == 0  # empty input


def test_matvec_identity_kat():  # math.rs:192-205
    k = KATS["matvec_identity"]
    w = oracle.Weight(oracle.F32, np.array(k["w"], np.float32), 2, 2)
    assert oracle.matvec_q(w, k["x"]).tolist() == k["y"]


def test_matmul_equals_stacked_matvec_kat():  # math.rs:207-233 (exact equality)
    k = KATS["matmul_stacked"]
    w = oracle.Weight(oracle.F32, np.array(k["w"], np.float32), 3, 2)
    xs = np.array(k["xs"], np.float32).reshape(k["s_len"], 2)
    batched = oracle.matmul_q(w, xs, k["s_len"])
    stacked = np.stack([oracle.matvec_q(w, xs[s]) for s in range(k["s_len"])])
    assert np.array_equal(batched, stacked)


# ---- the two statements of each layout agree bit for bit ---------------------
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_q4k_two_statements_agree(seed):
    w = synth.gen_q4k(32, 1024, seed)
    assert np.array_equal(oracle.dequantize(oracle.Q4_K, w, 32 * 1024), nf.dequant_q4k(w, 32 * 1024))


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_q6k_two_statements_agree(seed):
    w = synth.gen_q6k(32, 1024, seed)
    assert np.array_equal(oracle.dequantize(oracle.Q6_K, w, 32 * 1024), nf.dequant_q6k(w, 32 * 1024))


def test_q4k_q6k_arbitrary_bytes_agree():
    """Uniform random bytes everywhere (scales, mins, d included; NaN/Inf d masked out)."""
    for blk, dt, fn, doffs in ((144, oracle.Q4_K, nf.dequant_q4k, (0, 2)), (210, oracle.Q6_K, nf.dequant_q6k, (208,))):
        w = synth.rand_bytes(77, 64 * blk).reshape(64, blk).copy()
        for off in doffs:  # keep the f16 exponent below 31
            w[:, off + 1] &= 0xBB
        a, b = oracle.dequantize(dt, w, 64 * 256), fn(w, 64 * 256)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q4k_subnormal_and_zero_d():  # dequant.rs:20
    w = synth.gen_q4k(4, 256, 5).reshape(4, 144).copy()
    w[0, 0:2] = (0x01, 0x00)  # smallest subnormal d
    w[1, 0:4] = 0  # d = dmin = 0
    w[2, 2:4] = (0xFF, 0x03)  # largest subnormal dmin
    a = oracle.dequantize(oracle.Q4_K, w, 1024)
    assert np.array_equal(a, nf.dequant_q4k(w, 1024))
    assert np.all(a[256:512] == 0)


def test_mlx_two_statements_agree():
    w, s, b = synth.gen_mlx4(24, 768, 64, 4)
    s32, b32 = synth.bf16_to_f32(s), synth.bf16_to_f32(b)
    assert np.array_equal(oracle.dequantize_mlx_q4(w, s32, b32, 24, 768, 64), nf.dequant_mlx4(w, s32, b32, 64))


def test_scale_min_k4_inverts_the_generator_packing():
    sc = synth.rand_ints(1, 8, 0, 63)
    mn = synth.rand_ints(2, 8, 0, 63)
    q = synth.pack_scales_k4(sc[None], mn[None])[0]
    for j in range(8):
        assert oracle.scale_min_k4(j, q) == (sc[j], mn[j])


# ---- matvec / matmul / MoE semantics ---------------------------------------
def test_matvec_is_sequential_f32_sum():  # math.rs:17
    w = synth.gen_q4k(3, 512, 9)
    x = synth.normal(10, 512)
    wf = oracle.dequantize(oracle.Q4_K, w, 3 * 512).reshape(3, 512)
    ref = np.zeros(3, np.float32)
    for o in range(3):
        acc = np.float32(0)
        for i in range(512):
            acc = np.float32(acc + np.float32(wf[o, i] * x[i]))
        ref[o] = acc
    assert np.array_equal(oracle.matvec_q(oracle.Weight(oracle.Q4_K, w, 3, 512), x), ref)


def test_matmul_q_equals_stacked_matvec_quantized():
    for dt, gen in ((oracle.Q4_K, synth.gen_q4k), (oracle.Q6_K, synth.gen_q6k)):
        w = oracle.Weight(dt, gen(16, 512, 3), 16, 512)
        xs = synth.normal(4, 7 * 512).reshape(7, 512)
        assert np.array_equal(oracle.matmul_q(w, xs, 7), np.stack([oracle.matvec_q(w, xs[s]) for s in range(7)]))


def test_moe_topk_matches_sorted_softmax():  # lib.rs:1455-1475
    lg = synth.router_logits(1, 128, 8, 11)[0]
    idx, wts = oracle.moe_topk(lg, 8)
    order = np.argsort(-lg, kind="stable")[:8]
    assert idx.tolist() == order.tolist()
    e = np.exp(lg[order] - lg[order].max())
    assert np.allclose(wts, e / e.sum(), rtol=1e-6)
    assert abs(wts.sum() - 1) < 1e-6


def test_rmsnorm_softmax_rope_basics():  # math.rs:175-189
    y = oracle.rmsnorm([1, 2, 3, 4], [1, 1, 1, 1], 0.0)
    assert abs(np.sqrt(np.mean(y * y)) - 1) < 1e-5
    p = oracle.softmax([1, 2, 3])
    assert abs(p.sum() - 1) < 1e-6 and p[2] > p[1] > p[0]
    v = synth.normal(5, 128)
    r = oracle.rope(v, 2, 64, 64, 17, 500000.0)
    assert np.allclose(np.hypot(r[0::2], r[1::2]), np.hypot(v[0::2], v[1::2]), rtol=1e-5)  # rotations keep norms
    assert np.array_equal(oracle.rope(v, 2, 64, 64, 0, 500000.0), v)
    assert oracle.argmax([1.0, 3.0, 3.0, 2.0]) == 1  # first index wins ties (sample.rs:125-133)


# ---- committed fixtures -----------------------------------------------------
def test_oracle_reproduces_committed_fixtures(small):
    for name, dt in (("q4k", oracle.Q4_K), ("q6k", oracle.Q6_K)):
        w, x = small[f"{name}_w"], small[f"{name}_x"]
        rows, cols = w.shape[0], x.size
        assert np.array_equal(oracle.dequantize(dt, w, rows * cols), small[f"{name}_deq"])
        W = oracle.Weight(dt, w, rows, cols)
        assert np.array_equal(oracle.matvec_q(W, x), small[f"{name}_y"])
        assert np.array_equal(oracle.matmul_q(W, small[f"{name}_xs"], 5), small[f"{name}_ys"])
    s32, b32 = synth.bf16_to_f32(small["mlx_s"]), synth.bf16_to_f32(small["mlx_b"])
    assert np.array_equal(oracle.dequantize_mlx_q4(small["mlx_w"], s32, b32, 24, 512, 64), small["mlx_deq"])
    assert np.array_equal(oracle.rmsnorm(small["norm_x"], small["norm_w"], 1e-5), small["norm_y"])
    assert np.array_equal(oracle.rope(small["norm_x"], 4, 64, 64, 1031, 500000.0), small["rope_y"])


def test_tiny_llama_decode_runs_and_kv_f16_matters_little():
    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 3)

    def build(kv_f16):
        mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
        layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
        return oracle.LlamaModel(p, mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16)

    a, b = build(False), build(True)
    tok = 5
    for pos in range(4):
        la, lb = a.forward(tok, pos), b.forward(tok, pos)
        assert np.isfinite(la).all()
        assert synth.rel_err(lb, la) < 2e-2
        tok = oracle.argmax(la)


# ---- third-party pin: ggml's own numpy dequantizer ------------------------------
def test_q4k_q6k_equal_ggmls_reference_dequantizer_bit_for_bit():
    """The reference's k-quant routines are a port of ggml's (crates/ullm-core/src/dequant.rs:3-5) and hold no
    known-answer vector for Q4_K / Q6_K.  The `gguf` Python package ships ggml's own numpy dequantizer: an
    implementation independent of this repository.  The oracle must reproduce it bit for bit on the benchmark's
    block distribution and on arbitrary random bytes (with a finite f16 scale)."""
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T
    from gguf import quants

    for dt, qt, gen, bb, d_off in ((oracle.Q4_K, T.Q4_K, synth.gen_q4k, 144, (0, 2)), (oracle.Q6_K, T.Q6_K, synth.gen_q6k, 210, (208,))):
        cases = [np.asarray(gen(64, 4096, 77)).reshape(-1).view(np.uint8)]
        rnd = synth.rand_bytes(78, 512 * bb).reshape(512, bb).copy()
        for o in d_off:  # keep the f16 scale fields finite: clear the top exponent bit of their high byte
            rnd[:, o + 1] &= 0xBF
        cases.append(rnd.reshape(-1))
        for blob in cases:
            n = blob.size // bb * 256
            ours = oracle.dequantize(dt, blob, n)
            theirs = quants.dequantize(blob.reshape(-1, bb), qt).astype(np.float32).reshape(-1)
            assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32)), (dt, "oracle differs from ggml's dequantizer")
