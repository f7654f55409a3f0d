"""SafeTensors / MLX model directories: a ctypes face on the C reader
(``include/ullm_safetensors.h``, the counterpart of ``SafeTensorsModel`` in
crates/ullm-safetensors/src/lib.rs and of the layout rules of crates/ullm-model/src/mlx.rs) and a
writer for synthetic models.

The reader is the product (C++, in ``libullm_cuda.so``); the writer exists so that tests and
benchmarks can hand the backend real ``.safetensors`` bytes when no model directory is available.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct

import numpy as np

from . import backend

OK, ERR_UNSUPPORTED, ERR_FORMAT, ERR_IO, ERR_INVALID, ERR_MISSING = 0, 1, 2, 6, 7, 8
DTYPE_NAMES = {backend.F32: "F32", backend.F16: "F16", backend.BF16: "BF16", backend.MLX_U32: "U32"}

_vp, _sz, _i, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64


class TensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", _i), ("n_dims", C.c_uint32), ("shape", _u64 * 8), ("shard", C.c_uint32), ("offset", _u64),
                ("nbytes", _u64), ("data", _vp)]


class MlxWeightC(C.Structure):
    _fields_ = [("weight", _vp), ("scales", _vp), ("biases", _vp), ("out", _u64), ("in_", _u64), ("group", _u64)]


class MlxParamsC(C.Structure):
    _fields_ = [(n, _u64) for n in ("n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_experts", "n_experts_used", "moe_inter", "n_ctx",
                                    "vocab", "group")] + [("rope_theta", C.c_float), ("eps", C.c_float)]


SIGNATURES = {
    "ullm_st_open": (_i, [C.c_char_p, C.POINTER(_vp), C.c_char_p, _sz]),
    "ullm_st_from_bytes": (_i, [_vp, _sz, C.POINTER(_vp), C.c_char_p, _sz]),
    "ullm_st_close": (None, [_vp]),
    "ullm_st_shard_count": (_sz, [_vp]),
    "ullm_st_tensor_count": (_sz, [_vp]),
    "ullm_st_tensor_at": (_i, [_vp, _sz, C.POINTER(TensorC)]),
    "ullm_st_tensor_find": (_i, [_vp, C.c_char_p, C.POINTER(TensorC)]),
    "ullm_st_has_tensor": (_i, [_vp, C.c_char_p]),
    "ullm_st_config_u64": (_i, [_vp, C.c_char_p, C.POINTER(_u64)]),
    "ullm_st_config_f32": (_i, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "ullm_st_config_str": (_i, [_vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_sz)]),
    "ullm_st_has_text_config": (_i, [_vp]),
    "ullm_st_has_tokenizer_json": (_i, [_vp]),
    "ullm_st_mlx_weight_get": (_i, [_vp, C.c_char_p, _u64, C.POINTER(MlxWeightC), C.c_char_p, _sz]),
    "ullm_st_mlx_experts_get": (_i, [_vp, C.c_char_p, _u64, _u64, _u64, _u64, _u64, C.POINTER(MlxWeightC), C.c_char_p, _sz]),
    "ullm_st_mlx_params_get": (_i, [_vp, C.POINTER(MlxParamsC), C.c_char_p, _sz]),
}
_bound = False


def _lib():
    global _bound
    lib = backend.load_library()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return lib


class SafeTensorsError(Exception):
    def __init__(self, code, msg):
        super().__init__(f"safetensors error {code}: {msg}")
        self.code = code


def _view(ptr, nbytes, dtype=np.uint8):
    if not nbytes:
        return np.empty(0, dtype)
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(nbytes,)).view(dtype)


class SafeTensors:
    """An open model (``SafeTensorsModel::open``): a directory, one ``.safetensors`` file, or the bytes of one."""

    def __init__(self, source):
        lib, h, err = _lib(), _vp(), C.create_string_buffer(400)
        if isinstance(source, (bytes, bytearray, memoryview)):
            b = np.frombuffer(bytes(source), np.uint8)
            rc = lib.ullm_st_from_bytes(b.ctypes.data if b.size else None, b.size, C.byref(h), err, 400)
        else:
            rc = lib.ullm_st_open(os.fspath(source).encode(), C.byref(h), err, 400)
        if rc:
            raise SafeTensorsError(rc, err.value.decode(errors="replace"))
        self._h = h.value

    def close(self):
        if self._h:
            _lib().ullm_st_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def n_shards(self):
        return _lib().ullm_st_shard_count(self._h)

    # -- tensors (TensorBag / WeightSource) -----------------------------------
    def _tensor(self, t: TensorC) -> dict:
        return dict(name=t.name.decode(), dtype=t.dtype, shape=tuple(t.shape[: t.n_dims]), shard=t.shard, offset=t.offset, nbytes=t.nbytes,
                    data=None if not t.data else _view(t.data, t.nbytes))

    def tensors(self) -> list:
        lib, out, t = _lib(), [], TensorC()
        for i in range(lib.ullm_st_tensor_count(self._h)):
            lib.ullm_st_tensor_at(self._h, i, C.byref(t))
            out.append(self._tensor(t))
        return out

    def tensor(self, name: str):
        t = TensorC()
        rc = _lib().ullm_st_tensor_find(self._h, name.encode(), C.byref(t))
        return None if rc else self._tensor(t)

    def has_tensor(self, name: str) -> bool:
        return bool(_lib().ullm_st_has_tensor(self._h, name.encode()))

    # -- config.json ---------------------------------------------------------------
    def config_u64(self, path: str):
        v = _u64()
        return None if _lib().ullm_st_config_u64(self._h, path.encode(), C.byref(v)) else v.value

    def config_f32(self, path: str):
        v = C.c_float()
        return None if _lib().ullm_st_config_f32(self._h, path.encode(), C.byref(v)) else v.value

    def config_str(self, path: str):
        s, n = C.c_char_p(), _sz()
        return None if _lib().ullm_st_config_str(self._h, path.encode(), C.byref(s), C.byref(n)) else s.value[: n.value].decode()

    @property
    def has_text_config(self) -> bool:
        return bool(_lib().ullm_st_has_text_config(self._h))

    @property
    def has_tokenizer_json(self) -> bool:
        return bool(_lib().ullm_st_has_tokenizer_json(self._h))

    # -- MLX 4-bit layout ------------------------------------------------------------
    def _mlx(self, rc, w: MlxWeightC, err):
        if rc:
            raise SafeTensorsError(rc, err.value.decode(errors="replace"))
        out, cols, g = w.out, w.in_, w.group
        return dict(out=out, cols=cols, group=g, weight=_view(w.weight, out * (cols // 8) * 4, np.uint32).reshape(out, cols // 8),
                    scales=_view(w.scales, out * (cols // g) * 2, np.uint16).reshape(out, cols // g),
                    biases=_view(w.biases, out * (cols // g) * 2, np.uint16).reshape(out, cols // g))

    def mlx_weight(self, name: str, group: int) -> dict:
        """``mlx_qweight`` (mlx.rs:30-56): packed words and the bf16 bits of the tables, views of the mapped file."""
        w, err = MlxWeightC(), C.create_string_buffer(400)
        return self._mlx(_lib().ullm_st_mlx_weight_get(self._h, name.encode(), group, C.byref(w), err, 400), w, err)

    def mlx_experts(self, name: str, n_experts: int, out_dim: int, in_dim: int, group: int, expert=None) -> dict:
        """``mlx_experts`` (mlx.rs:58-88): one expert's slice, or the whole stack when ``expert`` is None."""
        w, err = MlxWeightC(), C.create_string_buffer(400)
        e = n_experts if expert is None else expert
        return self._mlx(_lib().ullm_st_mlx_experts_get(self._h, name.encode(), n_experts, out_dim, in_dim, group, e, C.byref(w), err, 400), w, err)

    def mlx_params(self) -> dict:
        p, err = MlxParamsC(), C.create_string_buffer(400)
        rc = _lib().ullm_st_mlx_params_get(self._h, C.byref(p), err, 400)
        if rc:
            raise SafeTensorsError(rc, err.value.decode(errors="replace"))
        return {n: getattr(p, n) for n, _ in MlxParamsC._fields_}


# ---- writer (synthetic models for tests and benchmarks) ----------------------------------------

def write_safetensors(tensors, metadata=None, pad_to: int = 8) -> bytes:
    """``tensors``: list of ``(name, dtype id or dtype string, shape, array-or-bytes)``; data laid out in the order given."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dtype, shape, data in tensors:
        b = data.tobytes() if isinstance(data, np.ndarray) else bytes(data)
        header[name] = {"dtype": DTYPE_NAMES.get(dtype, dtype), "shape": list(shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % pad_to)  # writers pad the header with spaces so the data starts aligned
    return struct.pack("<Q", len(h)) + h + b"".join(blobs)


def mlx_linear_tensors(name: str, words, scales_bf16, biases_bf16):
    """The three tensors of one MLX quantized linear (any leading expert dimension included)."""
    w, s, b = np.ascontiguousarray(words, np.uint32), np.ascontiguousarray(scales_bf16, np.uint16), np.ascontiguousarray(biases_bf16, np.uint16)
    return [(name + ".weight", "U32", w.shape, w), (name + ".scales", "BF16", s.shape, s), (name + ".biases", "BF16", b.shape, b)]


def write_model_dir(path, config: dict, shards: dict, index: bool = True):
    """A model directory: ``config.json``, the shard files ``{file name: tensor list}`` and, when ``index`` is set
    (or there is more than one shard), ``model.safetensors.index.json``."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f)
    weight_map = {}
    for fname, tensors in shards.items():
        with open(os.path.join(path, fname), "wb") as f:
            f.write(write_safetensors(tensors))
        for t in tensors:
            weight_map[t[0]] = fname
    if index or len(shards) > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": weight_map}, f)


def qwen3moe_to_dir(path, model: dict, shards: int = 2):
    """Writes a model of :func:`ullm_b200.synth.gen_qwen3moe_model` as an MLX model directory with the tensor
    names and the ``config.json`` keys ``LlamaModel::from_mlx`` reads (crates/ullm-model/src/mlx.rs:103-213)."""
    from . import synth

    p = model["params"]

    def lin(name, t):
        _, words, out, cols, sc, bi, _ = t
        return mlx_linear_tensors(name, np.asarray(words).reshape(out, cols // 8), np.asarray(sc).reshape(out, -1), np.asarray(bi).reshape(out, -1))

    def vec(name, a):
        return [(name, "BF16", (len(a),), synth.f32_to_bf16(np.asarray(a, np.float32)))]

    files = [[] for _ in range(shards)]
    files[0] += lin("model.embed_tokens", model["tok_embd"])
    files[-1] += lin("lm_head", model["output"]) + vec("model.norm.weight", model["final_norm"])
    for i, l in enumerate(model["layers"]):
        q, ts = f"model.layers.{i}", []
        ts += vec(q + ".input_layernorm.weight", l["attn_norm"]) + vec(q + ".post_attention_layernorm.weight", l["ffn_norm"])
        ts += vec(q + ".self_attn.q_norm.weight", l["q_norm"]) + vec(q + ".self_attn.k_norm.weight", l["k_norm"])
        for n, k in (("q_proj", "wq"), ("k_proj", "wk"), ("v_proj", "wv"), ("o_proj", "wo")):
            ts += lin(f"{q}.self_attn.{n}", l[k])
        ts += lin(q + ".mlp.gate", l["moe_gate"])
        x = l["experts"]
        ne, hid, inter = x["n_experts"], x["hidden"], x["inter"]
        for n, k, o, c in (("gate_proj", "gate", inter, hid), ("up_proj", "up", inter, hid), ("down_proj", "down", hid, inter)):
            w, sc, bi = x[k]
            ts += mlx_linear_tensors(f"{q}.mlp.switch_mlp.{n}", np.asarray(w).reshape(ne, o, c // 8), np.asarray(sc).reshape(ne, o, -1),
                                     np.asarray(bi).reshape(ne, o, -1))
        files[i * shards // max(1, len(model["layers"]))] += ts
    config = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": p["n_embd"], "num_attention_heads": p["n_head"],
              "num_hidden_layers": p["n_layer"], "num_key_value_heads": p["n_kv_head"], "head_dim": p["head_dim"],
              "num_experts": p["n_experts"], "num_experts_per_tok": p["n_experts_used"], "moe_intermediate_size": p["moe_inter"],
              "max_position_embeddings": p["n_ctx"], "rope_theta": p["rope_theta"], "rms_norm_eps": p["eps"], "vocab_size": p["vocab"],
              "quantization": {"group_size": p["group"], "bits": 4}}
    write_model_dir(path, config, {f"model-{j + 1:05d}-of-{shards:05d}.safetensors": ts for j, ts in enumerate(files)})
