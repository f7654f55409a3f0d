"""ctypes binding of the CPU oracle (``libullm_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py``.  The CUDA library and its host
wrappers never import this package.  The C functions restate the reference's CPU
path; each one cites the reference lines it follows in ``ullm_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libullm_oracle.so")

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, BF16, MLX_U32 = 0, 1, 2, 8, 12, 14, 30, 1000
OK, ERR_FORMAT, ERR_UNSUPPORTED = 0, 1, 2


def build() -> str:
    """Compile the oracle with its Makefile (gcc, -ffp-contract=off, OpenMP)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    return _SO


class QWeight(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_int),
        ("out", C.c_size_t),
        ("cols", C.c_size_t),
        ("mlx_scales", C.c_void_p),
        ("mlx_biases", C.c_void_p),
        ("mlx_group", C.c_size_t),
    ]


class MoeExperts(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("gate_w", "up_w", "down_w", "gate_s", "gate_b", "up_s", "up_b", "down_s", "down_b")] + [
        (n, C.c_size_t) for n in ("n_experts", "hidden", "inter", "group")
    ]


class Layer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p)] + [
        (n, QWeight) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")
    ] + [(n, C.c_void_p) for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm")] + [
        ("moe_gate", QWeight), ("experts", C.c_void_p), ("n_experts_used", C.c_size_t)]


class Model(C.Structure):
    _fields_ = (
        [(n, C.c_size_t) for n in ("n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_ff", "n_ctx", "vocab")]
        + [("rope_theta", C.c_float), ("eps", C.c_float), ("tok_embeddings", QWeight), ("output", QWeight)]
        + [("final_norm", C.c_void_p), ("layers", C.c_void_p), ("key_cache", C.c_void_p), ("val_cache", C.c_void_p), ("kv_f16", C.c_int),
           ("rope_neox", C.c_int)]
    )


_lib = None


def lib():
    global _lib
    if _lib is None:
        src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("ullm_oracle.c", "ullm_oracle.h"))
        if not os.path.exists(_SO) or os.path.getmtime(_SO) < src_m:
            build()
        L = C.CDLL(_SO)
        L.uo_f16_to_f32.restype = C.c_float
        L.uo_f16_to_f32.argtypes = [C.c_uint16]
        L.uo_bf16_to_f32.restype = C.c_float
        L.uo_bf16_to_f32.argtypes = [C.c_uint16]
        L.uo_round_f16.restype = C.c_float
        L.uo_round_f16.argtypes = [C.c_float]
        L.uo_silu.restype = C.c_float
        L.uo_silu.argtypes = [C.c_float]
        L.uo_block_size.restype = C.c_size_t
        L.uo_type_size.restype = C.c_size_t
        L.uo_argmax.restype = C.c_size_t
        L.uo_argmax.argtypes = [C.c_void_p, C.c_size_t]
        L.uo_dequantize_into.restype = C.c_int
        L.uo_dequantize_into.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]
        L.uo_dequantize_mlx_q4.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]
        L.uo_scale_min_k4.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.uo_matvec_q.argtypes = [C.POINTER(QWeight), C.c_void_p, C.c_void_p]
        L.uo_matmul_q.argtypes = [C.POINTER(QWeight), C.c_void_p, C.c_size_t, C.c_void_p]
        L.uo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_void_p]
        L.uo_softmax.argtypes = [C.c_void_p, C.c_size_t]
        L.uo_rope.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float]
        L.uo_moe_topk.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]
        L.uo_moe_ffn.argtypes = [C.POINTER(MoeExperts), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
        L.uo_forward_llama.argtypes = [C.POINTER(Model), C.c_uint32, C.c_size_t, C.c_void_p]
        L.uo_forward_llama_embd.argtypes = [C.POINTER(Model), C.c_void_p, C.c_size_t, C.c_void_p]
        L.uo_embed.argtypes = [C.POINTER(Model), C.c_uint32, C.c_void_p]
        L.uo_max_threads.restype = C.c_int
        _lib = L
    return _lib


class OracleError(Exception):
    """Mirrors ullm_core::Error::{Format, Unsupported} (error.rs:11-20)."""

    def __init__(self, code):
        super().__init__({ERR_FORMAT: "format error", ERR_UNSUPPORTED: "unsupported"}.get(code, f"error {code}"))
        self.code = code


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def max_threads() -> int:
    return lib().uo_max_threads()


def f16_to_f32(h: int) -> float:
    return lib().uo_f16_to_f32(h)


def dequantize(dtype: int, data, n: int) -> np.ndarray:
    """``ullm_core::dequant::dequantize`` (dequant.rs:52-56)."""
    data = _u8(data)
    out = np.zeros(n, np.float32)
    rc = lib().uo_dequantize_into(dtype, _p(data), data.size, _p(out), n)
    if rc != OK:
        raise OracleError(rc)
    return out


def dequantize_mlx_q4(weight, scales, biases, out: int, in_dim: int, group: int) -> np.ndarray:
    w = np.ascontiguousarray(weight, np.uint32)
    s = np.ascontiguousarray(scales, np.float32)
    b = np.ascontiguousarray(biases, np.float32)
    y = np.zeros(out * in_dim, np.float32)
    lib().uo_dequantize_mlx_q4(_p(w), _p(s), _p(b), out, in_dim, group, _p(y))
    return y.reshape(out, in_dim)


def scale_min_k4(j: int, q) -> tuple[int, int]:
    q = _u8(q)
    sc, mn = C.c_uint8(), C.c_uint8()
    lib().uo_scale_min_k4(j, _p(q), C.byref(sc), C.byref(mn))
    return sc.value, mn.value


class Weight:
    """Keeps the arrays a ``uo_qweight`` points at alive."""

    def __init__(self, dtype, data, out, cols, scales=None, biases=None, group=0):
        self.data = _u8(data)
        self.scales = None if scales is None else np.ascontiguousarray(scales, np.float32).reshape(-1)
        self.biases = None if biases is None else np.ascontiguousarray(biases, np.float32).reshape(-1)
        self.out, self.cols, self.dtype, self.group = out, cols, dtype, group
        self.c = QWeight(
            self.data.ctypes.data, dtype, out, cols,
            None if self.scales is None else self.scales.ctypes.data,
            None if self.biases is None else self.biases.ctypes.data, group,
        )


def matvec_q(w: Weight, x) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    assert x.size == w.cols
    y = np.zeros(w.out, np.float32)
    lib().uo_matvec_q(C.byref(w.c), _p(x), _p(y))
    return y


def matmul_q(w: Weight, xs, s_len: int) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.float32)
    assert xs.size == s_len * w.cols
    y = np.zeros((s_len, w.out), np.float32)
    lib().uo_matmul_q(C.byref(w.c), _p(xs), s_len, _p(y))
    return y


def rmsnorm(x, weight, eps) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(weight, np.float32)
    y = np.zeros_like(x)
    lib().uo_rmsnorm(_p(x), _p(w), x.size, eps, _p(y))
    return y


def softmax(x) -> np.ndarray:
    y = np.array(x, np.float32, copy=True)
    lib().uo_softmax(_p(y), y.size)
    return y


def silu(x: float) -> float:
    return lib().uo_silu(x)


def rope(vec, n_heads, head_dim, rotary_dim, pos, theta) -> np.ndarray:
    v = np.array(vec, np.float32, copy=True)
    lib().uo_rope(_p(v), n_heads, head_dim, rotary_dim, pos, theta)
    return v


def argmax(x) -> int:
    x = np.ascontiguousarray(x, np.float32)
    return lib().uo_argmax(_p(x), x.size)


def round_f16(v: float) -> float:
    return lib().uo_round_f16(v)


def moe_topk(logits, k):
    lg = np.ascontiguousarray(logits, np.float32)
    idx = np.zeros(k, np.uint32)
    wts = np.zeros(k, np.float32)
    lib().uo_moe_topk(_p(lg), lg.size, k, _p(idx), _p(wts))
    return idx, wts


class Experts:
    """Stacked MLX 4-bit experts; scale/bias tables widened to f32 (mlx.rs:17-26)."""

    def __init__(self, gate, up, down, n_experts, hidden, inter, group):
        # gate/up/down: tuples (words u32, scales f32, biases f32)
        self.keep = []
        f = {}
        for name, (w, s, b) in (("gate", gate), ("up", up), ("down", down)):
            w = _u8(np.ascontiguousarray(w, np.uint32))
            s = np.ascontiguousarray(s, np.float32).reshape(-1)
            b = np.ascontiguousarray(b, np.float32).reshape(-1)
            self.keep += [w, s, b]
            f[name] = (w.ctypes.data, s.ctypes.data, b.ctypes.data)
        self.c = MoeExperts(
            f["gate"][0], f["up"][0], f["down"][0],
            f["gate"][1], f["gate"][2], f["up"][1], f["up"][2], f["down"][1], f["down"][2],
            n_experts, hidden, inter, group,
        )
        self.hidden = hidden


def moe_ffn(e: Experts, logits, k, xb) -> np.ndarray:
    lg = np.ascontiguousarray(logits, np.float32)
    xb = np.ascontiguousarray(xb, np.float32)
    out = np.zeros(e.hidden, np.float32)
    lib().uo_moe_ffn(C.byref(e.c), _p(lg), k, _p(xb), _p(out))
    return out


class LlamaModel:
    """Dense Llama decode on the oracle (lib.rs:807-969).  ``layers`` is a list of
    dicts with f32 ``attn_norm``/``ffn_norm`` and :class:`Weight` projections."""

    def __init__(self, params: dict, tok_embeddings: Weight, output: Weight, final_norm, layers, kv_f16: bool, rope_neox: bool = False):
        self.p = params
        self.keep = [tok_embeddings, output, layers]
        self.final_norm = np.ascontiguousarray(final_norm, np.float32)
        arr = (Layer * len(layers))()
        for i, l in enumerate(layers):
            an = np.ascontiguousarray(l["attn_norm"], np.float32)
            fn = np.ascontiguousarray(l["ffn_norm"], np.float32)
            self.keep += [an, fn]
            arr[i].attn_norm, arr[i].ffn_norm = an.ctypes.data, fn.ctypes.data
            for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"):
                if l.get(n) is not None:  # a mixture-of-experts layer has no dense FFN matrices
                    setattr(arr[i], n, l[n].c)
            if l.get("experts") is not None:  # router :class:`Weight`, :class:`Experts`, experts per token
                arr[i].moe_gate, arr[i].experts, arr[i].n_experts_used = l["moe_gate"].c, C.addressof(l["experts"].c), l["n_experts_used"]
            for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm"):  # optional variants (lib.rs:877-901)
                if l.get(n) is not None:
                    a = np.ascontiguousarray(l[n], np.float32)
                    self.keep.append(a)
                    setattr(arr[i], n, a.ctypes.data)
        self.layers = arr
        kv_dim = params["n_kv_head"] * params["head_dim"]
        self.key_cache = np.zeros((params["n_layer"], params["n_ctx"], kv_dim), np.float32)
        self.val_cache = np.zeros_like(self.key_cache)
        self.c = Model(
            params["n_embd"], params["n_layer"], params["n_head"], params["n_kv_head"], params["head_dim"],
            params["n_ff"], params["n_ctx"], params["vocab"], params["rope_theta"], params["eps"],
            tok_embeddings.c, output.c, self.final_norm.ctypes.data, C.addressof(arr),
            self.key_cache.ctypes.data, self.val_cache.ctypes.data, 1 if kv_f16 else 0, 1 if rope_neox else 0,
        )

    def embed(self, token: int) -> np.ndarray:
        x = np.zeros(self.p["n_embd"], np.float32)
        lib().uo_embed(C.byref(self.c), token, _p(x))
        return x

    def forward(self, token: int, pos: int) -> np.ndarray:
        logits = np.zeros(self.p["vocab"], np.float32)
        lib().uo_forward_llama(C.byref(self.c), token, pos, _p(logits))
        return logits

    def forward_debug(self, x_init, pos: int):
        """``[(label, maxabs), ...]`` of layer 0's intermediates (GpuForward::forward_debug, forward.rs:530-635)."""
        x = np.ascontiguousarray(x_init, np.float32)
        idx = (C.c_int * 16)()
        mx = (C.c_float * 16)()
        L = lib()
        L.uo_debug_label.restype = C.c_char_p
        L.uo_forward_debug.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int]
        n = L.uo_forward_debug(C.byref(self.c), _p(x), pos, idx, mx, 16)
        if n < 0:
            raise OracleError("forward_debug: layer 0 is a mixture-of-experts layer")
        return [(L.uo_debug_label(idx[i]).decode(), float(mx[i])) for i in range(n)]

    def forward_embd(self, x_init, pos: int) -> np.ndarray:
        x = np.ascontiguousarray(x_init, np.float32)
        logits = np.zeros(self.p["vocab"], np.float32)
        lib().uo_forward_llama_embd(C.byref(self.c), _p(x), pos, _p(logits))
        return logits
