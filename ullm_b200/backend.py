"""Host-side mirror of the reference's GPU backend surface over the C ABI.

``CudaContext`` carries the method set of ``ullm_metal::MetalContext``
(crates/ullm-metal/src/lib.rs:18-318): ``device_name``, ``upload``,
``matvec_quant``, ``matvec_resident``, ``matvec_mlx4``, ``matmul_mlx4`` — same
names, argument meaning and error behaviour (``Unsupported`` / ``Format``).
Everything runs in ``libullm_cuda.so``; there is no Python or CPU compute path,
and loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libullm_cuda.so")

# ullm_status
OK, ERR_UNSUPPORTED, ERR_FORMAT, ERR_CUDA, ERR_TIMEOUT, ERR_OOM, ERR_INVALID = range(7)
# ullm_dtype (ggml ids, crates/ullm-gguf/src/types.rs:7-29)
F32, F16, Q4_K, Q6_K, BF16, MLX_U32 = 0, 1, 12, 14, 30, 1000

Q4K_BLOCK_BYTES, Q6K_BLOCK_BYTES, QK_K = 144, 210, 256


class UllmError(Exception):
    """ullm_core::Error (crates/ullm-core/src/error.rs:11-20) plus CUDA statuses."""

    def __init__(self, code: int, msg: str):
        names = {1: "unsupported", 2: "format error", 3: "cuda error", 4: "timeout", 5: "out of memory", 6: "invalid argument"}
        super().__init__(f"{names.get(code, code)}: {msg}")
        self.code = code


class Unsupported(UllmError):
    pass


class FormatError(UllmError):
    pass


OPT_PDL, OPT_SHARD_TIMEOUT_MS = 1, 2
SHARD_HANDLE_BYTES, SHARD_NCCL_ID_BYTES, SHARD_NO_WAIT, SHARD_FUSED_STORES, SHARD_SM_PUSH = 64, 128, 1, 2, 4

_lib = None

_vp, _sz, _i = C.c_void_p, C.c_size_t, C.c_int

# name -> (restype, argtypes): every symbol include/ullm_cuda.h declares.
SIGNATURES = {
    "ullm_cuda_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "ullm_cuda_ctx_destroy": (None, [_vp]),
    "ullm_cuda_last_error": (C.c_char_p, [_vp]),
    "ullm_cuda_ctx_set_option": (_i, [_vp, _i, _i]),
    "ullm_cuda_device_name": (_i, [_vp, C.c_char_p, _sz]),
    "ullm_cuda_sm_count": (_i, [_vp]),
    "ullm_cuda_synchronize": (_i, [_vp]),
    "ullm_cuda_upload": (_i, [_vp, _vp, _sz, C.POINTER(_vp)]),
    "ullm_cuda_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "ullm_cuda_download": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "ullm_cuda_buf_ptr": (_vp, [_vp]),
    "ullm_cuda_buf_len": (_sz, [_vp]),
    "ullm_cuda_buf_free": (None, [_vp, _vp]),
    "ullm_cuda_dequantize": (_i, [_vp, _i, _vp, _sz, _vp, _sz]),
    "ullm_cuda_dequantize_mlx4": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "ullm_cuda_matvec_quant": (_i, [_vp, _i, _vp, _sz, _vp, _vp, _sz, _sz]),
    "ullm_cuda_matvec_resident": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _sz]),
    "ullm_cuda_matvec_mlx4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ullm_cuda_matvec_dev": (_i, [_vp, _i, _vp, _vp, _vp, _i, _sz, _vp, _vp, _sz, _sz, _vp]),
    "ullm_cuda_weight_create": (_i, [_vp, _vp, _i, C.POINTER(_vp)]),
    "ullm_cuda_weight_destroy": (None, [_vp, _vp]),
    "ullm_cuda_weight_matvec": (_i, [_vp, _vp, _vp, _vp]),
    "ullm_cuda_weight_matvec_dev": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "ullm_cuda_weight_matvec_batch_dev": (_i, [_vp, _sz, _vp, _vp, _vp, _vp]),
    "ullm_cuda_weight_matvec_batch": (_i, [_vp, _sz, _vp, _vp, _vp]),
    "ullm_cuda_weight_matvec_chain_dev": (_i, [_vp, _sz, _vp, _vp]),
    "ullm_cuda_weight_matmul": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "ullm_cuda_weight_matmul_dev": (_i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "ullm_cuda_weight_export": (_i, [_vp, _vp, _vp, _sz]),
    "ullm_cuda_weight_bytes": (_sz, [_vp]),
    "ullm_cuda_weight_create_st": (_i, [_vp, _vp, C.c_char_p, _sz, C.POINTER(_vp)]),
    "ullm_cuda_matmul_quant": (_i, [_vp, _i, _vp, _sz, _vp, _vp, _sz, _sz, _sz]),
    "ullm_cuda_matmul_mlx4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz]),
    "ullm_cuda_matmul_dev": (_i, [_vp, _i, _vp, _vp, _vp, _i, _sz, _vp, _vp, _sz, _sz, _sz, _vp]),
    "ullm_cuda_shard_create": (_i, [_vp, _i, _i, _sz, C.POINTER(_vp)]),
    "ullm_cuda_shard_destroy": (None, [_vp]),
    "ullm_cuda_shard_export": (_i, [_vp, _vp]),
    "ullm_cuda_shard_connect": (_i, [_vp, _vp]),
    "ullm_cuda_shard_connect_local": (_i, [_vp, _i]),
    "ullm_cuda_shard_reset": (_i, [_vp]),
    "ullm_cuda_shard_y": (_vp, [_vp]),
    "ullm_cuda_shard_read": (_i, [_vp, _sz, _vp, _sz]),
    "ullm_cuda_shard_row_range": (_i, [_sz, _i, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "ullm_cuda_shard_weight_create": (_i, [_vp, _vp, _i, C.POINTER(_vp)]),
    "ullm_cuda_shard_matvec_dev": (_i, [_vp, _sz, _vp, _i, _vp]),
    "ullm_cuda_shard_matvec": (_i, [_vp, _sz, _vp, _vp, _vp, _sz, _sz]),
    "ullm_cuda_shard_wait_dev": (_i, [_vp, _vp]),
    "ullm_cuda_shard_matmul_dev": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _i, _vp]),
    "ullm_cuda_shard_nccl_id": (_i, [_vp]),
    "ullm_cuda_shard_nccl_init": (_i, [_vp, _vp]),
    "ullm_cuda_shard_allgather_nccl_dev": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "ullm_cuda_shard_nccl_check": (_i, [_vp]),
    "ullm_cuda_experts_create": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "ullm_cuda_experts_create_st": (_i, [_vp, _vp, C.c_char_p, _sz, _sz, _sz, _sz, C.POINTER(_vp)]),
    "ullm_cuda_experts_destroy": (None, [_vp, _vp]),
    "ullm_cuda_moe_ffn": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp]),
    "ullm_cuda_moe_ffn_dev": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp, _vp]),
    "ullm_cuda_moe_ffn_noalloc": (_i, [_i, _vp, _vp, _vp, _sz, _sz, _vp, _vp, C.c_char_p, _sz]),
    "ullm_cuda_forward_create": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "ullm_cuda_forward_create_gguf": (_i, [_vp, _vp, _i, C.POINTER(_vp)]),
    "ullm_cuda_forward_create_st": (_i, [_vp, _vp, _i, C.POINTER(_vp)]),
    "ullm_cuda_forward_batch": (_i, [_vp, _vp, _sz, _vp]),
    "ullm_cuda_forward_destroy": (None, [_vp]),
    "ullm_cuda_forward": (_i, [_vp, _vp, _sz, _vp]),
    "ullm_cuda_forward_set_kv": (_i, [_vp, _sz, _sz, _vp, _vp]),
    "ullm_cuda_forward_debug": (_i, [_vp, _vp, _sz, _vp, _sz, C.POINTER(_sz)]),
    "ullm_cuda_forward_supports_batched_prefill": (_i, [_vp]),
    "ullm_cuda_forward_greedy": (_i, [_vp, _vp, _i, C.c_uint32, _sz, _sz, _vp]),
    "ullm_cuda_forward_greedy_weight": (_i, [_vp, _vp, C.c_uint32, _sz, _sz, _vp]),
}
# Test / tuning knobs outside the mirrored surface.
DEBUG_SIGNATURES = {
    "ullm_cuda_debug_set": (_i, [_vp, C.c_char_p, _i]),
    "ullm_cuda_debug_last_plan": (_i, [_vp, _vp, _i]),
    "ullm_cuda_debug_read_probe": (_i, [_vp, _i, _sz, _i, _i, _i, _i, _vp]),
    "ullm_cuda_debug_chain_deal": (_i, [_i, _vp, _vp, _vp, _i, _vp]),
}


def load_library() -> C.CDLL:
    """Loads ``libullm_cuda.so``; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library first (python -m ullm_b200.build); there is no CPU fallback"
            )
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in {**SIGNATURES, **DEBUG_SIGNATURES}.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _ptr(a) -> int:
    return a.ctypes.data if a is not None else None


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, np.float32)


def _bytes(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        return np.frombuffer(a, np.uint8)
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


class Buffer:
    """A resident device buffer (``metal::Buffer`` in the reference surface)."""

    def __init__(self, ctx: "CudaContext", handle: int):
        self._ctx, self._h = ctx, handle

    @property
    def ptr(self) -> int:
        return load_library().ullm_cuda_buf_ptr(self._h)

    def __len__(self) -> int:
        return load_library().ullm_cuda_buf_len(self._h)

    def download(self, offset: int = 0, length: int | None = None) -> np.ndarray:
        n = len(self) - offset if length is None else length
        out = np.empty(n, np.uint8)
        self._ctx._check(load_library().ullm_cuda_download(self._ctx._h, self._h, offset, _ptr(out), n))
        return out

    def free(self):
        if self._h:
            load_library().ullm_cuda_buf_free(self._ctx._h, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CudaContext:
    """``MetalContext`` on a B200 (crates/ullm-metal/src/lib.rs:18-318)."""

    def __init__(self, device: int = 0):
        lib = load_library()
        h = _vp()
        rc = lib.ullm_cuda_ctx_create(device, C.byref(h))
        if rc == ERR_UNSUPPORTED:
            raise Unsupported(rc, "no CUDA device available")  # lib.rs:33
        if rc != OK:
            raise UllmError(rc, "context creation failed")
        self._h = h.value
        self._lib = lib

    def close(self):
        if getattr(self, "_h", None):
            self._lib.ullm_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc == OK:
            return
        msg = (self._lib.ullm_cuda_last_error(self._h) or b"").decode()
        cls = {ERR_UNSUPPORTED: Unsupported, ERR_FORMAT: FormatError}.get(rc, UllmError)
        raise cls(rc, msg)

    # -- MetalContext surface ------------------------------------------------
    def device_name(self) -> str:
        buf = C.create_string_buffer(256)
        self._check(self._lib.ullm_cuda_device_name(self._h, buf, 256))
        return buf.value.decode()

    def sm_count(self) -> int:
        return self._lib.ullm_cuda_sm_count(self._h)

    def synchronize(self):
        self._check(self._lib.ullm_cuda_synchronize(self._h))

    def upload(self, data) -> Buffer:
        b = _bytes(data)
        h = _vp()
        self._check(self._lib.ullm_cuda_upload(self._h, _ptr(b), b.size, C.byref(h)))
        return Buffer(self, h.value)

    def alloc(self, nbytes: int) -> Buffer:
        h = _vp()
        self._check(self._lib.ullm_cuda_alloc(self._h, nbytes, C.byref(h)))
        return Buffer(self, h.value)

    def dequantize(self, dtype: int, data, n: int) -> np.ndarray:
        b = _bytes(data)
        out = np.empty(n, np.float32)
        self._check(self._lib.ullm_cuda_dequantize(self._h, dtype, _ptr(b), b.size, _ptr(out), n))
        return out

    def dequantize_mlx_q4(self, weight, scales, biases, out_dim: int, in_dim: int, group: int) -> np.ndarray:
        w = np.ascontiguousarray(weight, np.uint32)
        s, b = _f32(scales), _f32(biases)
        y = np.empty((out_dim, in_dim), np.float32)
        self._check(self._lib.ullm_cuda_dequantize_mlx4(self._h, _ptr(w), _ptr(s), _ptr(b), out_dim, in_dim, group, _ptr(y)))
        return y

    def matvec_quant(self, dtype: int, w_bytes, x, out_dim: int, in_dim: int) -> np.ndarray:
        w, x = _bytes(w_bytes), _f32(x)
        y = np.empty(out_dim, np.float32)
        self._check(self._lib.ullm_cuda_matvec_quant(self._h, dtype, _ptr(w), w.size, _ptr(x), _ptr(y), out_dim, in_dim))
        return y

    def matvec_resident(self, dtype: int, wbuf: Buffer, x, out_dim: int, in_dim: int, out: np.ndarray | None = None) -> np.ndarray:
        x = _f32(x)
        y = np.empty(out_dim, np.float32) if out is None else out
        self._check(self._lib.ullm_cuda_matvec_resident(self._h, dtype, wbuf._h, _ptr(x), _ptr(y), out_dim, in_dim))
        return y

    def matvec_mlx4(self, w, scales, biases, x, out_dim: int, in_dim: int, group_size: int) -> np.ndarray:
        w, s, b, x = _bytes(w), _f32(scales), _f32(biases), _f32(x)
        y = np.empty(out_dim, np.float32)
        self._check(self._lib.ullm_cuda_matvec_mlx4(self._h, _ptr(w), _ptr(s), _ptr(b), _ptr(x), _ptr(y), out_dim, in_dim, group_size))
        return y

    def matmul_quant(self, dtype: int, w_bytes, x, out_dim: int, in_dim: int, s: int) -> np.ndarray:
        w, x = _bytes(w_bytes), _f32(x)
        y = np.empty((s, out_dim), np.float32)
        self._check(self._lib.ullm_cuda_matmul_quant(self._h, dtype, _ptr(w), w.size, _ptr(x), _ptr(y), out_dim, in_dim, s))
        return y

    def matmul_mlx4(self, w, scales, biases, x, out_dim: int, in_dim: int, group_size: int, s: int) -> np.ndarray:
        w, sc, b, x = _bytes(w), _f32(scales), _f32(biases), _f32(x)
        y = np.empty((s, out_dim), np.float32)
        self._check(self._lib.ullm_cuda_matmul_mlx4(self._h, _ptr(w), _ptr(sc), _ptr(b), _ptr(x), _ptr(y), out_dim, in_dim, group_size, s))
        return y

    # -- device-pointer forms (resident pipelines, benchmarks) ------------------
    def matvec_dev(self, dtype, d_w, d_x, d_y, out_dim, in_dim, stream=None, d_scales=None, d_biases=None, table_dtype=0, group=0):
        self._check(
            self._lib.ullm_cuda_matvec_dev(self._h, dtype, d_w, d_scales, d_biases, table_dtype, group, d_x, d_y, out_dim, in_dim, stream)
        )

    def matmul_dev(self, dtype, d_w, d_x, d_y, out_dim, in_dim, s, stream=None, d_scales=None, d_biases=None, table_dtype=0, group=0):
        self._check(
            self._lib.ullm_cuda_matmul_dev(self._h, dtype, d_w, d_scales, d_biases, table_dtype, group, d_x, d_y, out_dim, in_dim, s, stream)
        )

    def set_option(self, option: int, value: int):
        """``ullm_cuda_ctx_set_option``: ``OPT_PDL`` or ``OPT_SHARD_TIMEOUT_MS``."""
        self._check(self._lib.ullm_cuda_ctx_set_option(self._h, option, value))

    # -- knobs used by tests --------------------------------------------------
    def debug_set(self, key: str, value: int):
        self._check(self._lib.ullm_cuda_debug_set(self._h, key.encode(), value))

    def read_probe(self, mode: int, nbytes: int, stage_bytes: int = 94208, stages: int = 2, chunk: int = 16384, reps: int = 8) -> dict:
        """Read-only bandwidth of this GPU over ``nbytes``: ``mode`` 0 = plain 16-byte loads, 1 = a bulk-copy ring
        without a consumer (the streaming side of the matvec kernels alone).  Median / min / max microseconds."""
        us = (C.c_float * 3)()
        self._check(self._lib.ullm_cuda_debug_read_probe(self._h, mode, nbytes, stage_bytes, stages, chunk, reps, us))
        return {"us": us[0], "us_min": us[1], "us_max": us[2], "gbs": nbytes / (us[0] * 1e-6) / 1e9}

    def last_plan(self) -> dict:
        v = (C.c_int * 6)()
        self._lib.ullm_cuda_debug_last_plan(self._h, v, 6)
        return dict(zip(("streamed", "rows_per_tile", "warps", "stages", "smem_bytes", "grid"), list(v)))


def chain_deal(mats, grid: int = 148) -> list[int]:
    """CTAs per matrix when the persistent matvec launch deals ``grid`` CTAs out to the independent matrices
    ``[(dtype, out, cols), ...]`` (host arithmetic of the library; no device needed)."""
    n = len(mats)
    dt = (C.c_int * n)(*[m[0] for m in mats])
    out = (C.c_size_t * n)(*[m[1] for m in mats])
    cols = (C.c_size_t * n)(*[m[2] for m in mats])
    res = (C.c_uint * n)()
    rc = load_library().ullm_cuda_debug_chain_deal(n, dt, out, cols, grid, res)
    if rc:
        raise UllmError(rc, "ullm_cuda_debug_chain_deal")
    return list(res)


class GpuWeight(C.Structure):
    """``GpuWeight`` (forward.rs:56-64)."""

    _fields_ = [("dtype", _i), ("bytes", _vp), ("len", _sz), ("out", _sz), ("cols", _sz), ("mlx_scales", _vp), ("mlx_biases", _vp), ("mlx_group", _sz)]


class Weight:
    """A resident weight matrix (``WBuf``, crates/ullm-metal/src/forward.rs:119-126):
    built from a ``GpuWeight`` the way ``GpuForward::new`` does (forward.rs:253-268)."""

    def __init__(self, ctx: CudaContext, dtype: int, data, out_dim: int, cols: int, scales=None, biases=None, group: int = 0):
        self._ctx = ctx
        b = _bytes(data)
        tdt = F32
        s = bi = None
        if scales is not None:
            if np.asarray(scales).dtype == np.uint16:
                tdt, s, bi = BF16, np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
            else:
                s, bi = _f32(scales), _f32(biases)
        gw = GpuWeight(dtype, b.ctypes.data, b.size, out_dim, cols, _ptr(s), _ptr(bi), group)
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_weight_create(ctx._h, C.byref(gw), tdt, C.byref(h)))
        self._h, self.out, self.cols, self.dtype = h.value, out_dim, cols, dtype

    @classmethod
    def from_safetensors(cls, ctx: CudaContext, st, name: str, group: int) -> "Weight":
        """The MLX linear ``<name>.weight/.scales/.biases`` of an open :class:`ullm_b200.safetensors.SafeTensors`
        (``ullm_cuda_weight_create_st``): bytes go from the mapped file to the device."""
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_weight_create_st(ctx._h, st._h, name.encode(), group, C.byref(h)))
        t = st.tensor(name + ".weight")
        self = cls.__new__(cls)
        self._ctx, self._h, self.out, self.cols, self.dtype = ctx, h.value, t["shape"][0], t["shape"][1] * 8, MLX_U32
        return self

    def matvec(self, x, out: np.ndarray | None = None) -> np.ndarray:
        x = _f32(x)
        y = np.empty(self.out, np.float32) if out is None else out
        self._ctx._check(self._ctx._lib.ullm_cuda_weight_matvec(self._ctx._h, self._h, _ptr(x), _ptr(y)))
        return y

    def matvec_dev(self, d_x: int, d_y: int, stream=None):
        self._ctx._check(self._ctx._lib.ullm_cuda_weight_matvec_dev(self._ctx._h, self._h, d_x, d_y, stream))

    def matmul(self, xs, s: int) -> np.ndarray:
        """``[s, in]`` token-major activations -> ``[s, out]`` (GpuForward::matmul, forward.rs:679)."""
        xs = _f32(xs)
        y = np.empty((s, self.out), np.float32)
        self._ctx._check(self._ctx._lib.ullm_cuda_weight_matmul(self._ctx._h, self._h, _ptr(xs), _ptr(y), s))
        return y

    def matmul_dev(self, d_x: int, d_y: int, s: int, stream=None):
        self._ctx._check(self._ctx._lib.ullm_cuda_weight_matmul_dev(self._ctx._h, self._h, d_x, d_y, s, stream))

    def export(self) -> np.ndarray:
        n = self._ctx._lib.ullm_cuda_weight_bytes(self._h)
        out = np.empty(n, np.uint8)
        self._ctx._check(self._ctx._lib.ullm_cuda_weight_export(self._ctx._h, self._h, _ptr(out), n))
        return out

    def free(self):
        if getattr(self, "_h", None):
            self._ctx._lib.ullm_cuda_weight_destroy(self._ctx._h, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class WeightBatch:
    """A fixed list of independent matvecs (weights, device x, device y) launched by one
    call of ``ullm_cuda_weight_matvec_batch_dev``."""

    def __init__(self, ctx: CudaContext, weights, d_xs, d_ys):
        n = len(weights)
        self._ctx, self._n, self._keep = ctx, n, weights
        self._w = (_vp * n)(*[w._h for w in weights])
        self._x = (_vp * n)(*d_xs)
        self._y = (_vp * n)(*d_ys)

    def launch(self, stream=None):
        c = self._ctx
        c._check(c._lib.ullm_cuda_weight_matvec_batch_dev(c._h, self._n, self._w, self._x, self._y, stream))


class HostBatch:
    """The same list from host vectors in one blocking call (``ullm_cuda_weight_matvec_batch``):
    ``xs`` / ``ys`` are float32 numpy arrays (page-locked ones are moved without the copy engines)."""

    def __init__(self, ctx: CudaContext, weights, xs, ys):
        n = len(weights)
        self._ctx, self._n, self._keep = ctx, n, (weights, xs, ys)
        self._w = (_vp * n)(*[w._h for w in weights])
        self._x = (_vp * n)(*[x.ctypes.data for x in xs])
        self._y = (_vp * n)(*[y.ctypes.data for y in ys])

    def run(self):
        c = self._ctx
        c._check(c._lib.ullm_cuda_weight_matvec_batch(c._h, self._n, self._w, self._x, self._y))


class ShardOpC(C.Structure):
    """``ullm_shard_op``."""

    _fields_ = [("w", _vp), ("d_x", _vp), ("y_offset", _sz), ("row0", _sz)]


class Shard:
    """One rank's end of a row-sharded group (``ullm_cuda_shard``): a gather buffer of
    ``y_floats`` floats with the same layout on every rank, into which every rank's kernels
    store the rows they computed.  Connect the ranks with :meth:`export` / :meth:`connect`
    (one process per GPU; the handles are plain bytes to be exchanged by any means) or with
    :func:`connect_local` (one process, several GPUs)."""

    def __init__(self, ctx: CudaContext, world: int, rank: int, y_floats: int):
        self._ctx, self.world, self.rank, self.y_floats = ctx, world, rank, y_floats
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_shard_create(ctx._h, world, rank, y_floats, C.byref(h)))
        self._h = h.value

    def export(self) -> bytes:
        buf = C.create_string_buffer(SHARD_HANDLE_BYTES)
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_export(self._h, buf))
        return buf.raw

    def connect(self, handles):
        """``handles``: the ``world`` exported handles in rank order."""
        blob = b"".join(handles)
        assert len(blob) == self.world * SHARD_HANDLE_BYTES
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_connect(self._h, C.c_char_p(blob)))

    @staticmethod
    def connect_local(shards):
        arr = (_vp * len(shards))(*[s._h for s in shards])
        shards[0]._ctx._check(shards[0]._ctx._lib.ullm_cuda_shard_connect_local(arr, len(shards)))

    def reset(self):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_reset(self._h))

    @property
    def y_ptr(self) -> int:
        return self._ctx._lib.ullm_cuda_shard_y(self._h)

    def read_y(self, offset: int, n: int) -> np.ndarray:
        """``n`` floats of this rank's gather buffer (``ullm_cuda_shard_read``: blocking; the step that
        wrote them must have finished)."""
        out = np.empty(n, np.float32)
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_read(self._h, offset, _ptr(out), n))
        return out

    def row_range(self, out_dim: int) -> tuple[int, int]:
        r0, n = _sz(), _sz()
        rc = self._ctx._lib.ullm_cuda_shard_row_range(out_dim, self.world, self.rank, C.byref(r0), C.byref(n))
        if rc:
            raise FormatError(rc, f"{out_dim} rows do not split evenly over {self.world} ranks")
        return r0.value, n.value

    def weight(self, dtype: int, data, out_dim: int, cols: int, scales=None, biases=None, group: int = 0) -> "Weight":
        """This rank's rows of the full host matrix (``ullm_cuda_shard_weight_create``)."""
        b = _bytes(data)
        tdt, s, bi = F32, None, None
        if scales is not None:
            if np.asarray(scales).dtype == np.uint16:
                tdt, s, bi = BF16, np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
            else:
                s, bi = _f32(scales), _f32(biases)
        gw = GpuWeight(dtype, b.ctypes.data, b.size, out_dim, cols, _ptr(s), _ptr(bi), group)
        h = _vp()
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_weight_create(self._h, C.byref(gw), tdt, C.byref(h)))
        w = Weight.__new__(Weight)
        w._ctx, w._h, w.out, w.cols, w.dtype = self._ctx, h.value, out_dim // self.world, cols, dtype
        return w

    def ops(self, items):
        """``items``: dicts ``w`` (:class:`Weight`), ``x`` (device address), ``y_offset`` and optionally ``row0``."""
        arr = (ShardOpC * len(items))()
        for c, o in zip(arr, items):
            c.w, c.d_x, c.y_offset, c.row0 = o["w"]._h, o["x"], o["y_offset"], o.get("row0", 0)
        arr._keep = [o["w"] for o in items]
        return arr

    def matvec_dev(self, ops, stream=None, flags: int = 0):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_matvec_dev(self._h, len(ops), ops, flags, stream))

    def matvec_host(self, ops, xs_host, y_host: np.ndarray, y_offset: int):
        """One blocking step from host vectors (``ullm_cuda_shard_matvec``); ``y_host`` receives the gathered floats."""
        xp = (_vp * len(ops))(*[x.ctypes.data if x is not None else None for x in xs_host])
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_matvec(self._h, len(ops), ops, xp, y_host.ctypes.data, y_offset, y_host.size))

    def wait_dev(self, stream=None):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_wait_dev(self._h, stream))

    def matmul_dev(self, w: "Weight", d_x: int, tokens: int, y_offset: int, row0: int, out_total: int, stream=None, flags: int = 0):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_matmul_dev(self._h, w._h, d_x, tokens, y_offset, row0, out_total, flags, stream))

    # NCCL comparison arm
    def nccl_id(self) -> bytes:
        buf = C.create_string_buffer(SHARD_NCCL_ID_BYTES)
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_nccl_id(buf))
        return buf.raw

    def nccl_init(self, ident: bytes):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_nccl_init(self._h, C.c_char_p(ident)))

    def allgather_nccl_dev(self, d_send: int, d_recv: int, count: int, stream=None):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_allgather_nccl_dev(self._h, d_send, d_recv, count, stream))

    def nccl_check(self):
        self._ctx._check(self._ctx._lib.ullm_cuda_shard_nccl_check(self._h))

    def free(self):
        if getattr(self, "_h", None):
            self._ctx._lib.ullm_cuda_shard_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2


class ChainOpC(C.Structure):
    """``ullm_chain_op``."""

    _fields_ = [("w", _vp), ("d_x", _vp), ("d_y", _vp), ("d_norm_w", _vp), ("eps", C.c_float), ("epi", _i), ("d_res", _vp), ("dep", _i)]


class WeightChain:
    """A fixed list of matvecs on resident weights run as one persistent launch
    (``ullm_cuda_weight_matvec_chain_dev``).  ``ops``: dicts with ``w`` (:class:`Weight`), ``x``,
    ``y`` (device addresses) and optionally ``norm_w``, ``eps``, ``epi``, ``res``, ``dep``."""

    def __init__(self, ctx: CudaContext, ops):
        self._ctx, self._n, self._keep = ctx, len(ops), [o["w"] for o in ops]
        self._ops = (ChainOpC * len(ops))()
        for c, o in zip(self._ops, ops):
            c.w, c.d_x, c.d_y = o["w"]._h, o["x"], o["y"]
            c.d_norm_w, c.eps, c.epi = o.get("norm_w"), o.get("eps", 0.0), o.get("epi", EPI_STORE)
            c.d_res, c.dep = o.get("res"), 1 if o.get("dep") else 0

    def launch(self, stream=None):
        c = self._ctx
        c._check(c._lib.ullm_cuda_weight_matvec_chain_dev(c._h, self._n, self._ops, stream))


class MoeExpertsInput(C.Structure):
    """``ullm_moe_experts_input`` (GpuExperts x3, crates/ullm-metal/src/forward.rs:67-75)."""

    _fields_ = [(n, _vp) for n in ("gate_w", "gate_scales", "gate_biases", "up_w", "up_scales", "up_biases", "down_w", "down_scales", "down_biases")] + [
        ("table_dtype", _i), ("n_experts", _sz), ("hidden", _sz), ("inter", _sz), ("group", _sz)]


class Experts:
    """Stacked MLX 4-bit experts resident on the device.  ``gate``/``up``/``down``
    are ``(words u32, scales, biases)``; tables either f32 or bf16 bit patterns
    (uint16), kept on the device in the type given."""

    def __init__(self, ctx: CudaContext, gate, up, down, n_experts: int, hidden: int, inter: int, group: int):
        self._ctx = ctx
        bf16 = np.asarray(gate[1]).dtype == np.uint16
        tdt = np.uint16 if bf16 else np.float32
        keep, ptrs = [], []
        for w, s, b in (gate, up, down):
            arrs = [np.ascontiguousarray(w, np.uint32), np.ascontiguousarray(s, tdt), np.ascontiguousarray(b, tdt)]
            keep += arrs
            ptrs += [a.ctypes.data for a in arrs]
        inp = MoeExpertsInput(*ptrs, BF16 if bf16 else F32, n_experts, hidden, inter, group)
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_experts_create(ctx._h, C.byref(inp), C.byref(h)))
        self._h, self.n_experts, self.hidden, self.inter = h.value, n_experts, hidden, inter

    @classmethod
    def from_safetensors(cls, ctx: CudaContext, st, prefix: str, n_experts: int, hidden: int, inter: int, group: int) -> "Experts":
        """The stacked experts ``<prefix>.gate_proj / .up_proj / .down_proj`` of an open
        :class:`ullm_b200.safetensors.SafeTensors` (``ullm_cuda_experts_create_st``)."""
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_experts_create_st(ctx._h, st._h, prefix.encode(), n_experts, hidden, inter, group, C.byref(h)))
        self = cls.__new__(cls)
        self._ctx, self._h, self.n_experts, self.hidden, self.inter = ctx, h.value, n_experts, hidden, inter
        return self

    def moe_ffn(self, x, logits, k: int, want_routing: bool = False):
        """``moe_ffn`` for every token of x [n_tok, hidden] (crates/ullm-model/src/lib.rs:1453-1488)."""
        x, lg = _f32(x).reshape(-1, self.hidden), _f32(logits).reshape(-1, self.n_experts)
        n_tok = x.shape[0]
        y = np.empty_like(x)
        idx = np.empty((n_tok, k), np.uint32)
        wts = np.empty((n_tok, k), np.float32)
        c = self._ctx
        c._check(c._lib.ullm_cuda_moe_ffn(c._h, self._h, _ptr(x), _ptr(lg), n_tok, k, _ptr(y), _ptr(idx), _ptr(wts)))
        return (y, idx, wts) if want_routing else y

    def moe_ffn_dev(self, d_x, d_logits, n_tok, k, d_y, stream=None):
        c = self._ctx
        c._check(c._lib.ullm_cuda_moe_ffn_dev(c._h, self._h, d_x, d_logits, n_tok, k, d_y, None, None, stream))

    def free(self):
        if self._h:
            self._ctx._lib.ullm_cuda_experts_destroy(self._ctx._h, self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# ---- full decode step: GpuForward (crates/ullm-metal/src/forward.rs:162-757) ----
class GpuParams(C.Structure):
    """``GpuParams`` (forward.rs:24-51) plus ``kv_f16``."""

    _fields_ = ([(n, _sz) for n in ("n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "n_ff", "n_ctx", "vocab")]
                + [("rope_theta", C.c_float), ("eps", C.c_float)]
                + [(n, _i) for n in ("rope_neox", "qk_norm", "sandwich_norm", "geglu")]
                + [(n, _sz) for n in ("n_experts", "n_experts_used", "moe_inter", "sliding_window")]
                + [("kv_f16", _i)])


class GpuLayerInput(C.Structure):
    _fields_ = [("attn_norm", _vp), ("ffn_norm", _vp)] + [(n, GpuWeight) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")] + [
        (n, _vp) for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm")] + [("moe_gate", GpuWeight), ("experts", _vp)]


class GpuModelInput(C.Structure):
    _fields_ = [("params", GpuParams), ("output", GpuWeight), ("final_norm", _vp), ("layers", _vp), ("mlx_table_dtype", _i)]


class DebugStatC(C.Structure):
    """``ullm_debug_stat``."""

    _fields_ = [("label", C.c_char * 16), ("nan", C.c_uint64), ("inf", C.c_uint64), ("maxabs", C.c_float)]


class GpuForward:
    """``GpuForward::{new, forward, forward_batch, supports_batched_prefill, forward_debug}`` on the B200.

    ``model`` is the dict :func:`ullm_b200.synth.gen_llama_model` builds (or the
    same structure filled from a real file): weights as ``(dtype, bytes, out,
    cols)`` tuples, norms as f32 arrays."""

    def __init__(self, ctx: CudaContext, model: dict, kv_f16: bool = False, **flags):
        self._ctx, p = ctx, model["params"]
        self.params = dict(p)
        keep = []

        tdt = [F32]  # element type of the MLX tables: bf16 bits when the arrays are uint16

        def table(a):
            if np.asarray(a).dtype == np.uint16:
                tdt[0] = BF16
                a = np.ascontiguousarray(a, np.uint16)
            else:
                a = _f32(a)
            keep.append(a)
            return a.ctypes.data

        def gw(t):
            dtype, data, out, cols = t[:4]
            b = _bytes(data)
            keep.append(b)
            if len(t) > 4:  # MLX 4-bit: (MLX_U32, words, out, cols, scales, biases, group)
                return GpuWeight(dtype, b.ctypes.data, b.size, out, cols, table(t[4]), table(t[5]), t[6])
            return GpuWeight(dtype, b.ctypes.data, b.size, out, cols, None, None, 0)

        def f32p(a):
            a = _f32(a)
            keep.append(a)
            return a.ctypes.data

        layers = (GpuLayerInput * len(model["layers"]))()
        for i, l in enumerate(model["layers"]):
            layers[i].attn_norm, layers[i].ffn_norm = f32p(l["attn_norm"]), f32p(l["ffn_norm"])
            for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"):
                if l.get(n) is not None:
                    setattr(layers[i], n, gw(l[n]))
            for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm"):
                if l.get(n) is not None:
                    setattr(layers[i], n, f32p(l[n]))
            if l.get("experts") is not None:  # MoE layer: router weight + stacked experts (gate, up, down) = (words, scales, biases)
                x = l["experts"]
                ptrs = []
                for w, s_, b_ in (x["gate"], x["up"], x["down"]):
                    bf = np.asarray(s_).dtype == np.uint16
                    arrs = [np.ascontiguousarray(w, np.uint32), np.ascontiguousarray(s_, np.uint16 if bf else np.float32),
                            np.ascontiguousarray(b_, np.uint16 if bf else np.float32)]
                    keep.extend(arrs)
                    ptrs += [a.ctypes.data for a in arrs]
                xi = MoeExpertsInput(*ptrs, BF16 if bf else F32, x["n_experts"], x["hidden"], x["inter"], x["group"])
                keep.append(xi)
                layers[i].moe_gate, layers[i].experts = gw(l["moe_gate"]), C.addressof(xi)
        for n in ("n_experts", "n_experts_used", "moe_inter"):
            if p.get(n):
                flags.setdefault(n, p[n])
        gp = GpuParams(p["n_embd"], p["n_layer"], p["n_head"], p["n_kv_head"], p["head_dim"], p["n_ff"], p["n_ctx"], p["vocab"],
                       p["rope_theta"], p["eps"], flags.get("rope_neox", 0), flags.get("qk_norm", 0), flags.get("sandwich_norm", 0),
                       flags.get("geglu", 0), flags.get("n_experts", 0), flags.get("n_experts_used", 0), flags.get("moe_inter", 0),
                       flags.get("sliding_window", 0), 1 if kv_f16 else 0)
        out_w, fin = gw(model["output"]), f32p(model["final_norm"])
        inp = GpuModelInput(gp, out_w, fin, C.addressof(layers), tdt[0])
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_forward_create(ctx._h, C.byref(inp), C.byref(h)))
        self._h = h.value
        self._logits = np.empty(p["vocab"], np.float32)

    @classmethod
    def from_gguf(cls, ctx: CudaContext, gguf, kv_f16: bool = False) -> "GpuForward":
        """Builds the engine from an open :class:`ullm_b200.gguf.Gguf` (``ullm_cuda_forward_create_gguf``)."""
        self = cls.__new__(cls)
        self._ctx = ctx
        lp = gguf.llama_params()
        self.params = dict(lp)
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_forward_create_gguf(ctx._h, gguf._h, 1 if kv_f16 else 0, C.byref(h)))
        self._h = h.value
        self._logits = np.empty(lp["vocab"], np.float32)
        return self

    @classmethod
    def from_safetensors(cls, ctx: CudaContext, st, kv_f16: bool = False) -> "GpuForward":
        """Builds the engine from an open MLX model directory (:class:`ullm_b200.safetensors.SafeTensors`,
        ``ullm_cuda_forward_create_st``)."""
        self = cls.__new__(cls)
        self._ctx = ctx
        h = _vp()
        ctx._check(ctx._lib.ullm_cuda_forward_create_st(ctx._h, st._h, 1 if kv_f16 else 0, C.byref(h)))
        mp = st.mlx_params()
        self.params = dict(mp)
        self._h = h.value
        self._logits = np.empty(mp["vocab"], np.float32)
        return self

    def forward(self, x_init, pos: int) -> np.ndarray:
        """One token: ``x_init`` is its embedding row; returns the vocab logits (forward.rs:384)."""
        x = _f32(x_init)
        out = np.empty(self.params["vocab"], np.float32)
        self._ctx._check(self._ctx._lib.ullm_cuda_forward(self._h, _ptr(x), pos, _ptr(out)))
        return out

    def forward_debug(self, x_init, pos: int):
        """``GpuForward::forward_debug`` (forward.rs:530-635): ``[(label, nan, inf, maxabs), ...]`` of layer 0, op by op."""
        x = _f32(x_init)
        recs = (DebugStatC * 32)()
        n = _sz()
        self._ctx._check(self._ctx._lib.ullm_cuda_forward_debug(self._h, _ptr(x), pos, recs, 32, C.byref(n)))
        return [(recs[i].label.decode(), int(recs[i].nan), int(recs[i].inf), float(recs[i].maxabs)) for i in range(n.value)]

    def set_kv(self, pos0: int, k, v):
        k, v = _f32(k), _f32(v)
        n = k.shape[1]
        self._ctx._check(self._ctx._lib.ullm_cuda_forward_set_kv(self._h, pos0, n, _ptr(k), _ptr(v)))

    def forward_batch(self, embeds, s: int) -> np.ndarray:
        """All ``s`` prompt tokens in one pass (``forward_batch``, forward.rs:757): fills the KV cache for
        positions 0..s-1 and returns the last token's logits."""
        e = _f32(embeds)
        out = np.empty(self.params["vocab"], np.float32)
        self._ctx._check(self._ctx._lib.ullm_cuda_forward_batch(self._h, _ptr(e), s, _ptr(out)))
        return out

    def supports_batched_prefill(self) -> bool:
        return bool(self._ctx._lib.ullm_cuda_forward_supports_batched_prefill(self._h))

    def greedy(self, embd: Buffer, embd_dtype: int, first_token: int, pos: int, n: int) -> np.ndarray:
        """``n`` greedy tokens kept on the device: argmax feeds the next embedding lookup."""
        out = np.empty(n, np.uint32)
        self._ctx._check(self._ctx._lib.ullm_cuda_forward_greedy(self._h, embd._h, embd_dtype, first_token, pos, n, _ptr(out)))
        return out

    def greedy_weight(self, embd: "Weight", first_token: int, pos: int, n: int) -> np.ndarray:
        """The same with the embedding matrix as a resident :class:`Weight` (MLX 4-bit tables included)."""
        out = np.empty(n, np.uint32)
        self._ctx._check(self._ctx._lib.ullm_cuda_forward_greedy_weight(self._h, embd._h, first_token, pos, n, _ptr(out)))
        return out

    def free(self):
        if getattr(self, "_h", None):
            self._ctx._lib.ullm_cuda_forward_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
