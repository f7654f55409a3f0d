"""CPU tests of the SafeTensors / MLX reader in ``libullm_cuda.so`` (``include/ullm_safetensors.h``).

The first case is the reference's own loader test (crates/ullm-safetensors/src/lib.rs:259-292: one F32
tensor ``w`` [2, 2] beside a ``__metadata__`` entry); the rest pin the rules its parser states in code
(lib.rs:59-167, 219-252) and the MLX layout of crates/ullm-model/src/mlx.rs:30-141."""
import json
import os
import struct

import numpy as np
import pytest

import oracle
from ullm_b200 import backend, safetensors as stm, synth
from ullm_b200.safetensors import ERR_FORMAT, ERR_IO, ERR_UNSUPPORTED, SafeTensors, SafeTensorsError


def blob(header: str, data: bytes = b"") -> bytes:
    h = header.encode()
    return struct.pack("<Q", len(h)) + h + data


def reference_blob() -> bytes:
    return blob('{"w":{"dtype":"F32","shape":[2,2],"data_offsets":[0,16]},"__metadata__":{"x":"y"}}', struct.pack("<4f", 1.0, 2.0, 3.0, 4.0))


def raises(code, fn, *a, **k):
    with pytest.raises(SafeTensorsError) as e:
        fn(*a, **k)
    assert e.value.code == code, str(e.value)
    return str(e.value)


def test_reference_one_tensor_file(tmp_path):
    path = os.path.join(tmp_path, "one.safetensors")
    with open(path, "wb") as f:
        f.write(reference_blob())
    for src in (path, reference_blob()):
        m = SafeTensors(src)
        ts = m.tensors()
        assert len(ts) == 1, "__metadata__ must be skipped"
        t = m.tensor("w")
        assert t["dtype"] == backend.F32 and t["shape"] == (2, 2) and t["nbytes"] == 16
        assert t["data"].view(np.float32).tolist() == [1.0, 2.0, 3.0, 4.0]
        assert m.has_tensor("w") and not m.has_tensor("__metadata__") and m.tensor("nope") is None
        assert m.n_shards == 1 and m.config_u64("hidden_size") is None  # a bare file has the empty config
        m.close()


def test_dtype_mapping_and_unsupported_types():
    a16 = np.arange(6, dtype=np.float16)
    words = np.arange(4, dtype=np.uint32)
    b = stm.write_safetensors([("a", "F16", (2, 3), a16), ("b", "BF16", (3,), np.arange(3, dtype=np.uint16)), ("c", "U32", (4,), words),
                               ("d", "I32", (1, 4), words)], metadata={"format": "mlx"})
    m = SafeTensors(b)
    assert [t["name"] for t in m.tensors()] == ["a", "b", "c", "d"]
    assert [m.tensor(n)["dtype"] for n in "abcd"] == [backend.F16, backend.BF16, backend.MLX_U32, backend.MLX_U32]  # lib.rs:229-235
    assert [m.tensor(n)["nbytes"] for n in "abcd"] == [12, 6, 16, 16]
    assert np.array_equal(m.tensor("a")["data"].view(np.float16), a16) and np.array_equal(m.tensor("d")["data"].view(np.uint32), words)
    for bad in ("F64", "I64", "U8", "BOOL", "F8_E4M3", "f32"):
        msg = raises(ERR_UNSUPPORTED, SafeTensors, blob('{"w":{"dtype":"%s","shape":[1],"data_offsets":[0,8]}}' % bad, bytes(8)))
        assert bad in msg


def test_malformed_files_are_clean_format_errors():
    full = reference_blob()
    hlen = struct.unpack("<Q", full[:8])[0]
    for n in range(0, 8 + hlen):  # every cut inside the length word or the header
        raises(ERR_FORMAT, SafeTensors, full[:n])
    raises(ERR_FORMAT, SafeTensors, struct.pack("<Q", 2**63) + b"{}")  # header length past the end, no overflow
    raises(ERR_FORMAT, SafeTensors, struct.pack("<Q", 2**64 - 1) + b"{}")
    raises(ERR_FORMAT, SafeTensors, blob("[1,2]"))  # not an object
    raises(ERR_FORMAT, SafeTensors, blob('{"w":{"shape":[1],"data_offsets":[0,4]}}', bytes(4)))
    raises(ERR_FORMAT, SafeTensors, blob('{"w":{"dtype":7,"shape":[1],"data_offsets":[0,4]}}', bytes(4)))
    raises(ERR_FORMAT, SafeTensors, blob('{"w":{"dtype":"F32","data_offsets":[0,4]}}', bytes(4)))
    raises(ERR_FORMAT, SafeTensors, blob('{"w":{"dtype":"F32","shape":[1]}}', bytes(4)))
    for bad_json in ('{"w":}', '{"w":{"dtype":"F32",}}', '{"a":1} x', '{"a":"\\q"}', '{"a":"\\ud800"}', '{"a":01}', "{'a':1}", '{"a":"\x01"}',
                     "[" * 200 + "]" * 200):
        assert "header" in raises(ERR_FORMAT, SafeTensors, blob(bad_json))
    # a tensor reaching past the end of the file is listed but has no data (tensor_data -> None, lib.rs:224)
    m = SafeTensors(full[:-1])
    t = m.tensor("w")
    assert t["shape"] == (2, 2) and t["data"] is None and t["nbytes"] == 0
    m = SafeTensors(blob('{"w":{"dtype":"F32","shape":[4294967296,4294967296,4],"data_offsets":[0,4]}}', bytes(4)))  # size overflows 64 bits
    assert m.tensor("w")["data"] is None
    m = SafeTensors(blob('{"w":{"dtype":"F32","shape":[1],"data_offsets":[18446744073709551615,4]}}', bytes(4)))  # offset wraps
    assert m.tensor("w")["data"] is None


def test_json_readings_follow_serde():
    # shape entries that are not non-negative integers count as 0; a missing first offset as 0 (lib.rs:144-151);
    # the second offset is not consulted (lib.rs:245-252); a repeated key keeps the last value; escapes in names
    b = blob('{"w":{"dtype":"F32","shape":[2,-1],"data_offsets":[0,16]},"v":{"dtype":"F32","shape":[2.0,2],"data_offsets":[0,16]},'
             '"u":{"dtype":"F32","shape":[3],"data_offsets":[]},"t":{"dtype":"F32","shape":[3],"data_offsets":[4,5]},'
             '"dup":{"dtype":"F16","shape":[1],"data_offsets":[0,2]},"dup":{"dtype":"F32","shape":[2],"data_offsets":[8,16]},'
             '"n\\u00e9\\n\\ud83d\\ude00":{"dtype":"F32","shape":[],"data_offsets":[12,16]}}   ', struct.pack("<4f", 1.0, 2.0, 3.0, 4.0))
    m = SafeTensors(b)
    assert m.tensor("w")["shape"] == (2, 0) and m.tensor("w")["nbytes"] == 0 and m.tensor("w")["data"] is not None
    assert m.tensor("v")["shape"] == (0, 2)
    assert m.tensor("u")["data"].view(np.float32).tolist() == [1.0, 2.0, 3.0]
    assert m.tensor("t")["data"].view(np.float32).tolist() == [2.0, 3.0, 4.0]
    assert m.tensor("dup")["dtype"] == backend.F32 and m.tensor("dup")["data"].view(np.float32).tolist() == [3.0, 4.0]
    t = m.tensor("né\n😀")
    assert t["shape"] == () and t["data"].view(np.float32).tolist() == [4.0]  # a scalar: one element
    assert [x["name"] for x in m.tensors()] == sorted(x["name"] for x in m.tensors())  # BTreeMap order (bytewise)


QWEN_CFG = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 256, "num_attention_heads": 8, "num_hidden_layers": 2,
            "num_key_value_heads": 2, "head_dim": 64, "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
            "max_position_embeddings": 40960, "rope_theta": 1000000.0, "rms_norm_eps": 1e-06, "vocab_size": 1000,
            "quantization": {"group_size": 64, "bits": 4}, "tie_word_embeddings": False}


def moe_tensors(prefix, n_experts, hidden, inter, group, seed):
    out, arrays = [], {}
    for j, (name, o, i) in enumerate((("gate_proj", inter, hidden), ("up_proj", inter, hidden), ("down_proj", hidden, inter))):
        w, s, b = synth.gen_mlx4(n_experts * o, i, group, seed + j)
        arrays[name] = (w, s, b)
        out += stm.mlx_linear_tensors(f"{prefix}.{name}", w.reshape(n_experts, o, i // 8), s.reshape(n_experts, o, -1), b.reshape(n_experts, o, -1))
    return out, arrays


def test_model_directory_shards_config_and_index(tmp_path):
    d = os.path.join(tmp_path, "model")
    e0, _ = moe_tensors("model.layers.0.mlp.switch_mlp", 8, 256, 128, 64, 100)
    e1, _ = moe_tensors("model.layers.1.mlp.switch_mlp", 8, 256, 128, 64, 200)
    norm = [("model.norm.weight", "BF16", (256,), synth.f32_to_bf16(np.ones(256, np.float32)))]
    # shard names chosen so that ascending file order differs from the order of first mention in the index
    stm.write_model_dir(d, QWEN_CFG, {"model-00002-of-00002.safetensors": e1 + norm, "model-00001-of-00002.safetensors": e0})
    m = SafeTensors(d)
    assert m.n_shards == 2 and len(m.tensors()) == 19
    assert m.tensor("model.layers.0.mlp.switch_mlp.up_proj.weight")["shard"] == 0 and m.tensor("model.norm.weight")["shard"] == 1
    assert not m.has_tokenizer_json and not m.has_text_config
    open(os.path.join(d, "tokenizer.json"), "w").write("{}")
    assert m.has_tokenizer_json
    # config readings (config_usize / config_f32 / config_str, lib.rs:182-202)
    assert m.config_u64("hidden_size") == 256 and m.config_u64("quantization.group_size") == 64
    assert m.config_str("architectures.0") == "Qwen3MoeForCausalLM" and m.config_str("architectures.1") is None
    assert abs(m.config_f32("rms_norm_eps") - 1e-6) < 1e-12 and m.config_f32("vocab_size") == 1000.0
    assert m.config_u64("rope_theta") is None  # 1000000.0 is a float: `as_u64` has no reading of it
    assert m.config_u64("tie_word_embeddings") is None and m.config_str("hidden_size") is None
    p = m.mlx_params()
    assert (p["n_embd"], p["n_layer"], p["n_head"], p["n_kv_head"], p["head_dim"]) == (256, 2, 8, 2, 64)
    assert (p["n_experts"], p["n_experts_used"], p["moe_inter"], p["vocab"], p["group"]) == (8, 2, 128, 1000, 64)
    assert p["n_ctx"] == 8192 and p["rope_theta"] == 1e6  # context capped (mlx.rs:131-134)
    # a single model.safetensors without an index
    d1 = os.path.join(tmp_path, "single")
    stm.write_model_dir(d1, {"text_config": {"hidden_size": 64}}, {"model.safetensors": norm}, index=False)
    m1 = SafeTensors(d1)
    assert m1.n_shards == 1 and m1.has_text_config and m1.config_u64("text_config.hidden_size") == 64 and m1.config_u64("hidden_size") is None
    # failures: nothing to open; an index without weight_map; a shard the index names but the directory lacks; bad config
    d2 = os.path.join(tmp_path, "empty")
    os.makedirs(d2)
    assert "no model.safetensors" in raises(ERR_FORMAT, SafeTensors, d2)
    open(os.path.join(d2, "model.safetensors.index.json"), "w").write('{"metadata":{}}')
    assert "weight_map" in raises(ERR_FORMAT, SafeTensors, d2)
    open(os.path.join(d2, "model.safetensors.index.json"), "w").write('{"weight_map":{"a":"gone.safetensors","b":7}}')
    assert "gone.safetensors" in raises(ERR_FORMAT, SafeTensors, d2)
    open(os.path.join(d1, "config.json"), "w").write("{broken")
    assert "config.json" in raises(ERR_FORMAT, SafeTensors, d1)
    raises(ERR_FORMAT, SafeTensors, os.path.join(tmp_path, "missing.safetensors"))  # open failure is a format error (lib.rs:109-110)
    open(os.path.join(tmp_path, "zero.safetensors"), "wb").close()
    raises(ERR_IO, SafeTensors, os.path.join(tmp_path, "zero.safetensors"))  # an empty file cannot be mapped (lib.rs:112)


def test_mlx_params_defaults_and_required_keys():
    def params(cfg, tmp):
        stm.write_model_dir(tmp, cfg, {"model.safetensors": [("x", "F32", (1,), np.zeros(1, np.float32))]}, index=False)
        return SafeTensors(tmp)

    import tempfile

    with tempfile.TemporaryDirectory() as td:
        base = {k: QWEN_CFG[k] for k in ("architectures", "hidden_size", "num_attention_heads", "num_hidden_layers", "num_experts",
                                         "num_experts_per_tok", "moe_intermediate_size", "vocab_size")}
        p = params(base, os.path.join(td, "a")).mlx_params()
        # mlx.rs:117-136: kv heads = heads, head_dim = hidden / heads, ctx 8192, theta 1e6, eps 1e-6, group 64
        assert (p["n_kv_head"], p["head_dim"], p["n_ctx"], p["group"]) == (8, 32, 8192, 64)
        assert p["rope_theta"] == 1e6 and abs(p["eps"] - 1e-6) < 1e-12
        p = params(dict(base, max_position_embeddings=4096, quantization={"group_size": 32}), os.path.join(td, "b")).mlx_params()
        assert p["n_ctx"] == 4096 and p["group"] == 32
        for i, k in enumerate(("hidden_size", "num_attention_heads", "num_hidden_layers", "num_experts", "num_experts_per_tok",
                               "moe_intermediate_size", "vocab_size")):
            cfg = {x: v for x, v in base.items() if x != k}
            assert k in raises(ERR_FORMAT, params(cfg, os.path.join(td, f"c{i}")).mlx_params)
        for j, arch in enumerate((["LlamaForCausalLM"], [], None)):
            cfg = dict(base, architectures=arch) if arch is not None else {x: v for x, v in base.items() if x != "architectures"}
            raises(ERR_UNSUPPORTED, params(cfg, os.path.join(td, f"d{j}")).mlx_params)  # mlx.rs:104-115


def test_mlx_linear_and_stacked_expert_slices():
    n_e, hidden, inter, g = 8, 256, 128, 64
    ts, arrays = moe_tensors("model.layers.0.mlp.switch_mlp", n_e, hidden, inter, g, 300)
    qw, qs, qb = synth.gen_mlx4(96, 256, g, 7)
    ts += stm.mlx_linear_tensors("model.layers.0.self_attn.q_proj", qw, qs, qb)
    m = SafeTensors(stm.write_safetensors(ts))
    q = m.mlx_weight("model.layers.0.self_attn.q_proj", g)  # mlx_qweight: out = shape[0], in = 8 * shape[1] (mlx.rs:35-36)
    assert (q["out"], q["cols"], q["group"]) == (96, 256, g)
    assert np.array_equal(q["weight"], qw) and np.array_equal(q["scales"], qs) and np.array_equal(q["biases"], qb)
    for name, o, i in (("gate_proj", inter, hidden), ("up_proj", inter, hidden), ("down_proj", hidden, inter)):
        w, s, b = arrays[name]
        full = m.mlx_experts(f"model.layers.0.mlp.switch_mlp.{name}", n_e, o, i, g)
        assert full["out"] == n_e * o and np.array_equal(full["weight"], w) and np.array_equal(full["scales"], s)
        for e in (0, 3, n_e - 1):  # expert e = words e*out*(in/8).., table entries e*out*(in/group).. (mlx.rs:71-87)
            sl = m.mlx_experts(f"model.layers.0.mlp.switch_mlp.{name}", n_e, o, i, g, expert=e)
            assert sl["out"] == o and np.array_equal(sl["weight"], w[e * o:(e + 1) * o]) and np.array_equal(sl["biases"], b[e * o:(e + 1) * o])
            # the slice dequantizes to the same values as that expert's rows of the stack
            ref = oracle.dequantize_mlx_q4(w[e * o:(e + 1) * o], synth.bf16_to_f32(s[e * o:(e + 1) * o]), synth.bf16_to_f32(b[e * o:(e + 1) * o]), o, i, g)
            got = oracle.dequantize_mlx_q4(sl["weight"], synth.bf16_to_f32(sl["scales"]), synth.bf16_to_f32(sl["biases"]), o, i, g)
            assert np.array_equal(ref, got)
    name = "model.layers.0.mlp.switch_mlp.gate_proj"
    assert "missing" in raises(ERR_FORMAT, m.mlx_weight, "model.layers.0.self_attn.k_proj", g)
    raises(ERR_FORMAT, m.mlx_experts, name, n_e + 1, inter, hidden, g)  # the stack is shorter than asked
    raises(ERR_FORMAT, m.mlx_experts, name, n_e, inter, hidden, 48)     # in % group != 0
    raises(ERR_FORMAT, m.mlx_experts, name, n_e, inter, hidden, g, expert=n_e + 1)
    raises(ERR_FORMAT, m.mlx_weight, "model.layers.0.self_attn.q_proj", 128 + 64)
    # tables that are not bf16, words that are not u32
    bad = stm.write_safetensors([("l.weight", "U32", qw.shape, qw), ("l.scales", "F16", qs.shape, qs), ("l.biases", "BF16", qb.shape, qb)])
    assert "BF16" in raises(ERR_FORMAT, SafeTensors(bad).mlx_weight, "l", g)
    bad = stm.write_safetensors([("l.weight", "F32", qw.shape, qw), ("l.scales", "BF16", qs.shape, qs), ("l.biases", "BF16", qb.shape, qb)])
    assert "U32" in raises(ERR_FORMAT, SafeTensors(bad).mlx_weight, "l", g)


def test_reference_mlx_golden_word_through_a_file():
    """crates/ullm-core/src/dequant.rs:324-334: one captured word + scale + bias, read back from a file image."""
    scale, bias = np.float32(0.004425049), np.float32(-0.039794922)
    sb, bb = synth.f32_to_bf16(np.array([scale])), synth.f32_to_bf16(np.array([bias]))
    assert synth.bf16_to_f32(sb)[0] == scale and synth.bf16_to_f32(bb)[0] == bias  # both are exact bf16 values
    m = SafeTensors(stm.write_safetensors(stm.mlx_linear_tensors("l", np.array([[2569837433]], np.uint32), sb.reshape(1, 1), bb.reshape(1, 1))))
    q = m.mlx_weight("l", 8)
    got = oracle.dequantize_mlx_q4(q["weight"], synth.bf16_to_f32(q["scales"]), synth.bf16_to_f32(q["biases"]), 1, 8, 8)
    expect = [3e-5, -0.00882, 0.00888, 3e-5, 0.01331, -0.03094, 3e-5, 3e-5]  # the reference's captured values, tolerance 1e-4
    assert np.abs(got.reshape(-1) - np.array(expect)).max() < 1e-4
