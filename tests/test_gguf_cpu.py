"""CPU tests of the GGUF reader in ``libullm_cuda.so`` (``include/ullm_gguf.h``).

The first two cases are the reference's own reader tests (crates/ullm-gguf/src/lib.rs:347-416:
a minimal valid v3 file and a bad magic); the rest pin the rules the reference's parser
states in code (lib.rs:72-169, value.rs:65-112, reader.rs, types.rs:7-29)."""
import os
import struct

import numpy as np
import pytest

from ullm_b200 import gguf, synth
from ullm_b200.gguf import T_ARRAY, T_BOOL, T_F32, T_F64, T_I8, T_I16, T_I32, T_I64, T_STRING, T_U8, T_U16, T_U32, T_U64


def s(x):
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def minimal():
    """magic, v3, 1 tensor, 2 metadata keys (general.architecture = "llama", llama.block_count = 1),
    tensor token_embd.weight 1-D [4] F32 at relative offset 0, padded to 32, data 1, 2, 3, 4."""
    b = struct.pack("<IIQQ", 0x46554747, 3, 1, 2)
    b += s("general.architecture") + struct.pack("<I", 8) + s("llama")
    b += s("llama.block_count") + struct.pack("<II", 4, 1)
    b += s("token_embd.weight") + struct.pack("<IQIQ", 1, 4, 0, 0)
    b += b"\0" * (-len(b) % 32)
    return b + struct.pack("<4f", 1.0, 2.0, 3.0, 4.0)


def test_reference_minimal_file():
    g = gguf.Gguf(minimal())
    assert g.version == 3 and g.architecture == "llama"
    assert g.get("llama.block_count") == 1
    ts = g.tensors()
    assert len(ts) == 1
    t = g.tensor("token_embd.weight")
    assert t["nbytes"] == 16 and t["shape"] == (4,) and t["dtype"] == 0
    assert t["data"].view(np.float32).tolist() == [1.0, 2.0, 3.0, 4.0]
    assert g.tensor("nope") is None and g.get("nope") is None


def test_reference_bad_magic_is_a_format_error():
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(bytes(64))
    assert e.value.code == gguf.ERR_FORMAT


def test_unsupported_version_and_type():
    b = bytearray(minimal())
    b[4:8] = struct.pack("<I", 1)
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(bytes(b))
    assert e.value.code == gguf.ERR_UNSUPPORTED  # lib.rs:82-87
    assert gguf.Gguf(minimal().replace(struct.pack("<I", 3), struct.pack("<I", 2), 1)).version == 2
    bad = gguf.write_gguf([], [("t", 9, (32,), bytes(64))])  # ggml type 9 (Q8_1) is not mapped, types.rs:23-27
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(bad)
    assert e.value.code == gguf.ERR_UNSUPPORTED


def test_every_truncation_is_a_clean_format_error():
    full = minimal()
    for n in list(range(0, 24)) + list(range(24, len(full) - 16, 7)) + [len(full) - 1]:
        with pytest.raises(gguf.GgufError) as e:
            gguf.Gguf(full[:n])
        assert e.value.code == gguf.ERR_FORMAT, n


def test_value_types_and_coercions():
    md = [("a.u8", T_U8, 200), ("a.i8", T_I8, -3), ("a.u16", T_U16, 60000), ("a.i16", T_I16, -2), ("a.u32", T_U32, 4_000_000_000),
          ("a.i32", T_I32, -1), ("a.u64", T_U64, 2**63 + 5), ("a.i64", T_I64, -7), ("a.f32", T_F32, 0.25), ("a.f64", T_F64, 1e-5),
          ("a.bool", T_BOOL, 1), ("a.str", T_STRING, "héllo"), ("a.arr_u", T_ARRAY, (T_U16, [1, 2, 3])),
          ("a.arr_s", T_ARRAY, (T_STRING, ["x", "", "yz"])), ("a.arr_f", T_ARRAY, (T_F32, [0.5, -1.5])),
          ("a.empty", T_ARRAY, (T_I32, []))]
    g = gguf.Gguf(gguf.write_gguf(md, []))
    assert g.keys() == sorted(k for k, _, _ in md)  # a BTreeMap: ascending keys
    assert g.get("a.u8") == 200 and g.get("a.u16") == 60000 and g.get("a.u32") == 4_000_000_000 and g.get("a.u64") == 2**63 + 5
    # signed values go through `as u64` (value.rs:44-55): sign-extended
    assert g.get("a.i8") == 2**64 - 3 and g.get("a.i16") == 2**64 - 2 and g.get("a.i32") == 2**64 - 1 and g.get("a.i64") == 2**64 - 7
    assert g.get("a.f32") == 0.25 and abs(g.get("a.f64") - 1e-5) < 1e-12 and g.get("a.bool") == 1
    assert g.get("a.str") == "héllo"
    assert g.get("a.arr_u") == [1, 2, 3] and g.get("a.arr_s") == ["x", "", "yz"] and g.get("a.arr_f") == [0.5, -1.5]
    assert g.get("a.empty") == []


def test_nested_arrays_and_unknown_value_types_are_format_errors():
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + s("k")
    for body in (struct.pack("<IIQ", 9, 9, 0), struct.pack("<I", 13)):  # array of arrays; type id 13
        with pytest.raises(gguf.GgufError) as e:
            gguf.Gguf(head + body)
        assert e.value.code == gguf.ERR_FORMAT


def test_alignment_shape_order_and_offsets():
    a = np.arange(2 * 3 * 256, dtype=np.float32)
    q = synth.gen_q4k(6, 512, 3)
    for align in (None, 64, 1):
        blob = gguf.write_gguf([("general.architecture", T_STRING, "llama")],
                               [("w.f32", 0, (2, 3, 256), a), ("w.q4k", 12, (6, 512), q), ("w.f16", 1, (5,), np.arange(5, dtype=np.float16))], align)
        g = gguf.Gguf(blob)
        assert g.alignment == (align or 32) and g.data_start % g.alignment == 0
        t = g.tensor("w.f32")
        assert t["shape"] == (2, 3, 256) and t["offset"] == g.data_start  # outermost first (lib.rs:135-138)
        assert np.array_equal(t["data"].view(np.float32), a)
        t = g.tensor("w.q4k")
        assert t["shape"] == (6, 512) and t["nbytes"] == 6 * 2 * 144 and t["offset"] % g.alignment == 0
        assert np.array_equal(t["data"], q.reshape(-1))
        assert g.tensor("w.f16")["nbytes"] == 10
        assert [x["name"] for x in g.tensors()] == ["w.f32", "w.q4k", "w.f16"]  # file order
    # general.alignment = 0 is raised to 1 (lib.rs:123-128)
    assert gguf.Gguf(gguf.write_gguf([("general.alignment", T_U32, 0)], [])).alignment == 1
    # a negative i32 widens to a huge u64 (value.rs:49): rounding the data offset up to it must not wrap to 0
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(gguf.write_gguf([("general.alignment", T_I32, -32)], [("w", 0, (8,), np.zeros(8, np.float32))]))
    assert e.value.code == gguf.ERR_FORMAT


def test_tensor_past_the_end_and_ragged_block_counts():
    blob = gguf.write_gguf([], [("w", 0, (8,), np.zeros(8, np.float32))])
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(blob[:-4])  # lib.rs:143-150
    assert e.value.code == gguf.ERR_FORMAT and "past end" in str(e.value)
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(gguf.write_gguf([], [("w", 12, (100,), bytes(144))]))  # 100 elements: not whole Q4_K blocks (lib.rs:289-296)
    assert e.value.code == gguf.ERR_FORMAT


def test_open_from_disk_and_llama_hyperparameters(tmp_path):
    p = dict(synth.LLAMA_TINY)
    m = synth.gen_llama_model(p, 9)
    path = os.path.join(tmp_path, "tiny.gguf")
    with open(path, "wb") as f:
        f.write(gguf.llama_to_gguf(m))
    g = gguf.Gguf(path)
    lp = g.llama_params()
    for k in ("n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_ff", "vocab"):
        assert lp[k] == p[k], k
    assert lp["n_ctx"] == min(p["n_ctx"], 8192) and abs(lp["rope_theta"] - p["rope_theta"]) < 1e-3 and abs(lp["eps"] - p["eps"]) < 1e-12
    assert len(g.tensors()) == 3 + 9 * p["n_layer"]
    t = g.tensor("blk.0.ffn_down.weight")
    assert t["dtype"] == 14 and t["shape"] == (p["n_embd"], p["n_ff"]) and np.array_equal(t["data"], m["layers"][0]["w_down"][1].reshape(-1))
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(os.path.join(tmp_path, "missing.gguf"))
    assert e.value.code == gguf.ERR_IO


def test_llama_defaults_and_required_keys():
    base = [("general.architecture", T_STRING, "llama"), ("llama.embedding_length", T_U32, 512), ("llama.block_count", T_U32, 2),
            ("llama.attention.head_count", T_U32, 8), ("llama.feed_forward_length", T_U32, 1024)]
    toks = ("tokenizer.ggml.tokens", T_ARRAY, (T_STRING, ["a", "b", "c"]))
    lp = gguf.Gguf(gguf.write_gguf(base + [toks], [])).llama_params()
    # defaults of lib.rs:174-225: kv heads = heads, ctx 2048, head_dim = embd / heads, theta 1e4, eps 1e-5, vocab from the token list
    assert (lp["n_kv_head"], lp["n_ctx"], lp["head_dim"], lp["vocab"]) == (8, 2048, 64, 3)
    assert lp["rope_theta"] == 10000.0 and abs(lp["eps"] - 1e-5) < 1e-12
    lp = gguf.Gguf(gguf.write_gguf(base + [("llama.context_length", T_U32, 131072)], [])).llama_params()
    assert lp["n_ctx"] == 8192 and lp["vocab"] == 0
    with pytest.raises(gguf.GgufError) as e:
        gguf.Gguf(gguf.write_gguf(base[:-1], [])).llama_params()
    assert e.value.code == gguf.ERR_FORMAT and "feed_forward_length" in str(e.value)
    for arch in ("qwen3", "gemma3", ""):  # lib.rs:200-209 reads llama, qwen2 and gemma3; gemma3's kernels are not built here
        with pytest.raises(gguf.GgufError) as e:
            gguf.Gguf(gguf.write_gguf([("general.architecture", T_STRING, arch)], [])).llama_params()
        assert e.value.code == gguf.ERR_UNSUPPORTED
    q2 = [(k.replace("llama.", "qwen2."), t, "qwen2" if k == "general.architecture" else v) for k, t, v in base]
    assert gguf.Gguf(gguf.write_gguf(q2, [])).llama_params()["n_ff"] == 1024  # keys are namespaced by the architecture (lib.rs:212-219)
