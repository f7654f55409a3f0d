"""GGUF files: a ctypes face on the C reader (``include/ullm_gguf.h``, the counterpart of
``GgufModel`` in crates/ullm-gguf/src/lib.rs:45-169) and a writer for synthetic models.

The reader is the product (C++, in ``libullm_cuda.so``); the writer exists so that tests and
benchmarks can hand the backend real ``.gguf`` bytes when no model file is available.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import backend

OK, ERR_UNSUPPORTED, ERR_FORMAT, ERR_IO, ERR_INVALID, ERR_MISSING = 0, 1, 2, 6, 7, 8
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 = range(13)
MAGIC = 0x46554747

_vp, _sz, _i = C.c_void_p, C.c_size_t, C.c_int


class TensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", _i), ("n_dims", C.c_uint32), ("shape", C.c_uint64 * 8), ("offset", C.c_uint64),
                ("nbytes", C.c_uint64), ("data", _vp)]


class LlamaParamsC(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_ff", "n_ctx", "vocab")] + [
        ("rope_theta", C.c_float), ("eps", C.c_float)]


SIGNATURES = {
    "ullm_gguf_open": (_i, [C.c_char_p, C.POINTER(_vp), C.c_char_p, _sz]),
    "ullm_gguf_from_bytes": (_i, [_vp, _sz, C.POINTER(_vp), C.c_char_p, _sz]),
    "ullm_gguf_close": (None, [_vp]),
    "ullm_gguf_version": (C.c_uint32, [_vp]),
    "ullm_gguf_architecture": (C.c_char_p, [_vp]),
    "ullm_gguf_alignment": (C.c_uint64, [_vp]),
    "ullm_gguf_data_start": (C.c_uint64, [_vp]),
    "ullm_gguf_tensor_count": (_sz, [_vp]),
    "ullm_gguf_tensor_at": (_i, [_vp, _sz, C.POINTER(TensorC)]),
    "ullm_gguf_tensor_find": (_i, [_vp, C.c_char_p, C.POINTER(TensorC)]),
    "ullm_gguf_meta_count": (_sz, [_vp]),
    "ullm_gguf_meta_key_at": (C.c_char_p, [_vp, _sz]),
    "ullm_gguf_meta_type": (_i, [_vp, C.c_char_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(C.c_uint64)]),
    "ullm_gguf_meta_u64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "ullm_gguf_meta_f32": (_i, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "ullm_gguf_meta_str": (_i, [_vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_sz)]),
    "ullm_gguf_meta_array_u64": (_i, [_vp, C.c_char_p, _sz, C.POINTER(C.c_uint64)]),
    "ullm_gguf_meta_array_f32": (_i, [_vp, C.c_char_p, _sz, C.POINTER(C.c_float)]),
    "ullm_gguf_meta_array_str": (_i, [_vp, C.c_char_p, _sz, C.POINTER(C.c_char_p), C.POINTER(_sz)]),
    "ullm_gguf_llama_params_get": (_i, [_vp, C.POINTER(LlamaParamsC), C.c_char_p, _sz]),
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


class GgufError(Exception):
    def __init__(self, code, msg):
        super().__init__(f"gguf error {code}: {msg}")
        self.code = code


class Gguf:
    """An open GGUF file (``GgufModel::open`` / ``from_bytes``)."""

    def __init__(self, source):
        lib, h, err = _lib(), _vp(), C.create_string_buffer(256)
        if isinstance(source, (bytes, bytearray, memoryview, np.ndarray)):
            b = np.frombuffer(bytes(source), np.uint8) if not isinstance(source, np.ndarray) else np.ascontiguousarray(source, np.uint8)
            rc = lib.ullm_gguf_from_bytes(b.ctypes.data if b.size else None, b.size, C.byref(h), err, 256)
        else:
            rc = lib.ullm_gguf_open(str(source).encode(), C.byref(h), err, 256)
        if rc:
            raise GgufError(rc, err.value.decode(errors="replace"))
        self._h = h.value

    # -- header ------------------------------------------------------------
    @property
    def version(self):
        return _lib().ullm_gguf_version(self._h)

    @property
    def architecture(self):
        return _lib().ullm_gguf_architecture(self._h).decode()

    @property
    def alignment(self):
        return _lib().ullm_gguf_alignment(self._h)

    @property
    def data_start(self):
        return _lib().ullm_gguf_data_start(self._h)

    # -- tensors -----------------------------------------------------------
    def _tensor(self, t: TensorC) -> dict:
        data = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(t.nbytes,)) if t.nbytes else np.empty(0, np.uint8)
        return dict(name=t.name.decode(), dtype=t.dtype, shape=tuple(t.shape[: t.n_dims]), offset=t.offset, nbytes=t.nbytes, data=data)

    def tensors(self) -> list[dict]:
        lib, out = _lib(), []
        for i in range(lib.ullm_gguf_tensor_count(self._h)):
            t = TensorC()
            lib.ullm_gguf_tensor_at(self._h, i, C.byref(t))
            out.append(self._tensor(t))
        return out

    def tensor(self, name: str):
        t = TensorC()
        return self._tensor(t) if _lib().ullm_gguf_tensor_find(self._h, name.encode(), C.byref(t)) == OK else None

    # -- metadata ----------------------------------------------------------
    def keys(self) -> list[str]:
        lib = _lib()
        return [lib.ullm_gguf_meta_key_at(self._h, i).decode() for i in range(lib.ullm_gguf_meta_count(self._h))]

    def get(self, key: str):
        """The value as Python data (ints via ``to_u64``, floats via ``to_f32``, str, list), or None."""
        lib, k = _lib(), key.encode()
        ty, et, n = _i(), _i(), C.c_uint64()
        if lib.ullm_gguf_meta_type(self._h, k, C.byref(ty), C.byref(et), C.byref(n)) != OK:
            return None

        def scalar(t, getter_u, getter_f, getter_s):
            if t == T_STRING:
                s, ln = C.c_char_p(), _sz()
                getter_s(C.byref(s), C.byref(ln))
                return C.string_at(s, ln.value).decode(errors="replace")
            if t in (T_F32, T_F64):
                f = C.c_float()
                getter_f(C.byref(f))
                return f.value
            u = C.c_uint64()
            getter_u(C.byref(u))
            return u.value

        if ty.value != T_ARRAY:
            return scalar(ty.value, lambda p: lib.ullm_gguf_meta_u64(self._h, k, p), lambda p: lib.ullm_gguf_meta_f32(self._h, k, p),
                          lambda s, ln: lib.ullm_gguf_meta_str(self._h, k, s, ln))
        return [scalar(et.value, lambda p, i=i: lib.ullm_gguf_meta_array_u64(self._h, k, i, p),
                       lambda p, i=i: lib.ullm_gguf_meta_array_f32(self._h, k, i, p),
                       lambda s, ln, i=i: lib.ullm_gguf_meta_array_str(self._h, k, i, s, ln)) for i in range(n.value)]

    def llama_params(self) -> dict:
        p, err = LlamaParamsC(), C.create_string_buffer(256)
        rc = _lib().ullm_gguf_llama_params_get(self._h, C.byref(p), err, 256)
        if rc:
            raise GgufError(rc, err.value.decode(errors="replace"))
        return {n: getattr(p, n) for n, _ in LlamaParamsC._fields_}

    def close(self):
        if getattr(self, "_h", None):
            _lib().ullm_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------
# writer (GGUF v3, little-endian)
# ---------------------------------------------------------------------------
def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


_PACK = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B", T_U64: "<Q",
         T_I64: "<q", T_F64: "<d"}


def _value(t: int, v) -> bytes:
    if t == T_STRING:
        return _s(v)
    if t == T_ARRAY:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    return struct.pack(_PACK[t], v)


def write_gguf(metadata, tensors, alignment: int | None = None, version: int = 3) -> bytes:
    """``metadata``: list of ``(key, type_id, value)`` (arrays: ``(elem_type, [items])``);
    ``tensors``: list of ``(name, ggml_type, shape_outermost_first, bytes)``.  Tensor data is placed
    at multiples of the alignment (``general.alignment`` is written when one is given)."""
    md = list(metadata)
    if alignment is not None:
        md.append(("general.alignment", T_U32, alignment))
    align = alignment or 32
    head = struct.pack("<IIQQ", MAGIC, version, len(tensors), len(md))
    for k, t, v in md:
        head += _s(k) + struct.pack("<I", t) + _value(t, v)
    infos, blobs, off = b"", [], 0
    for name, ggml_type, shape, data in tensors:
        b = np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes() if not isinstance(data, bytes) else data
        infos += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        infos += struct.pack("<IQ", ggml_type, off)
        blobs.append((off, b))
        off = (off + len(b) + align - 1) // align * align
    out = bytearray(head + infos)
    out += b"\0" * (-len(out) % align)
    start = len(out)
    for o, b in blobs:
        out += b"\0" * (start + o - len(out))
        out += b
    return bytes(out)


def llama_to_gguf(model: dict, alignment: int | None = None, arch: str = "llama") -> bytes:
    """The synthetic model of :func:`ullm_b200.synth.gen_llama_model` as a GGUF file with the keys and
    tensor names ``LlamaModel::from_gguf`` reads (crates/ullm-model/src/lib.rs:174-301)."""
    p = model["params"]
    md = [("general.architecture", T_STRING, arch), (arch + ".embedding_length", T_U32, p["n_embd"]),
          (arch + ".block_count", T_U32, p["n_layer"]), (arch + ".attention.head_count", T_U32, p["n_head"]),
          (arch + ".attention.head_count_kv", T_U32, p["n_kv_head"]), (arch + ".feed_forward_length", T_U32, p["n_ff"]),
          (arch + ".context_length", T_U32, p["n_ctx"]), (arch + ".attention.key_length", T_U32, p["head_dim"]),
          (arch + ".rope.freq_base", T_F32, p["rope_theta"]), (arch + ".attention.layer_norm_rms_epsilon", T_F32, p["eps"]),
          (arch + ".vocab_size", T_U32, p["vocab"])]

    def w(name, t):
        dtype, data, out, cols = t
        return (name, dtype, (out, cols), data)

    ts = [w("token_embd.weight", model["tok_embd"])]
    for i, l in enumerate(model["layers"]):
        b = f"blk.{i}."
        ts += [(b + "attn_norm.weight", 0, (p["n_embd"],), np.asarray(l["attn_norm"], np.float32)),
               w(b + "attn_q.weight", l["wq"]), w(b + "attn_k.weight", l["wk"]), w(b + "attn_v.weight", l["wv"]),
               w(b + "attn_output.weight", l["wo"]),
               (b + "ffn_norm.weight", 0, (p["n_embd"],), np.asarray(l["ffn_norm"], np.float32)),
               w(b + "ffn_gate.weight", l["w_gate"]), w(b + "ffn_up.weight", l["w_up"]), w(b + "ffn_down.weight", l["w_down"])]
        # optional tensors (lib.rs:277-281); the K bias goes out as F16 and the K norm as BF16 to exercise tensor_f32's widening
        for key, name, dt in (("q_bias", "attn_q.bias", 0), ("k_bias", "attn_k.bias", 1), ("v_bias", "attn_v.bias", 0),
                              ("q_norm", "attn_q_norm.weight", 0), ("k_norm", "attn_k_norm.weight", 30)):
            if l.get(key) is not None:
                a = np.asarray(l[key], np.float32)
                data = a if dt == 0 else (a.astype(np.float16) if dt == 1 else (a.view(np.uint32) >> 16).astype(np.uint16))
                ts.append((b + name, dt, (a.size,), data))
    ts += [("output_norm.weight", 0, (p["n_embd"],), np.asarray(model["final_norm"], np.float32)), w("output.weight", model["output"])]
    return write_gguf(md, ts, alignment)
