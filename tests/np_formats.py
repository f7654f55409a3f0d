"""A second, independent statement of the three weight formats, vectorised in
numpy and written in the *factored* form the reference's GPU shader uses
(crates/ullm-metal/src/shader.metal:185-255 for Q4_K: word loads with the
0x3f3f / 0x0f0f / 0xc0c0 mask trick; :121-180 for Q6_K), not the element-by-
element form of crates/ullm-core/src/dequant.rs that the C oracle restates.
Agreement of the two pins the Q4_K / Q6_K layouts, for which the reference has
no known-answer vector.  Also fast enough for full-size workloads.
"""
import numpy as np


def f16(bits_lo_hi: np.ndarray) -> np.ndarray:
    """[..., 2] little-endian bytes -> f32."""
    return np.ascontiguousarray(bits_lo_hi).view(np.float16)[..., 0].astype(np.float32)


def q4k_scales_mins(sc12: np.ndarray):
    """12 packed bytes -> (scales[8], mins[8]) through 16-bit masks."""
    u = np.ascontiguousarray(sc12).view(np.uint16).astype(np.uint32)  # [..., 6]
    lo_s = u[..., 0:2] & 0x3F3F  # scales 0..3
    lo_m = u[..., 2:4] & 0x3F3F  # mins 0..3
    hi_s = (u[..., 4:6] & 0x0F0F) | ((u[..., 0:2] & 0xC0C0) >> 2)  # scales 4..7
    hi_m = ((u[..., 4:6] >> 4) & 0x0F0F) | ((u[..., 2:4] & 0xC0C0) >> 2)  # mins 4..7

    def split(x):
        return np.stack([x[..., 0] & 0xFF, x[..., 0] >> 8, x[..., 1] & 0xFF, x[..., 1] >> 8], -1)

    return np.concatenate([split(lo_s), split(hi_s)], -1), np.concatenate([split(lo_m), split(hi_m)], -1)


def dequant_q4k(data: np.ndarray, n: int) -> np.ndarray:
    blk = np.ascontiguousarray(data).view(np.uint8).reshape(-1, 144)[: n // 256]
    d, dmin = f16(blk[:, 0:2]), f16(blk[:, 2:4])
    sc, mn = q4k_scales_mins(blk[:, 4:16])
    qs = blk[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)  # sub-blocks 2c, 2c+1
    d1 = (d[:, None] * sc.astype(np.float32))[:, :, None]
    m1 = (dmin[:, None] * mn.astype(np.float32))[:, :, None]
    return (d1 * q - m1).astype(np.float32).reshape(-1)


def dequant_q6k(data: np.ndarray, n: int) -> np.ndarray:
    blk = np.ascontiguousarray(data).view(np.uint8).reshape(-1, 210)[: n // 256]
    ql = blk[:, 0:128].reshape(-1, 2, 2, 32)  # [b, half, lo/hi 32-byte run, l]
    qh = blk[:, 128:192].reshape(-1, 2, 32)
    sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = f16(blk[:, 208:210])
    lows = np.stack([ql[:, :, 0] & 0x0F, ql[:, :, 1] & 0x0F, ql[:, :, 0] >> 4, ql[:, :, 1] >> 4], 2)  # [b,h,4,32]
    highs = np.stack([(qh >> s) & 3 for s in (0, 2, 4, 6)], 2)
    q = (lows | (highs << 4)).astype(np.int32) - 32
    scale = sc.reshape(-1, 2, 4, 2).repeat(16, axis=3)  # scale index is + l/16 + 2g
    vals = (d[:, None, None, None] * scale) * q.astype(np.float32)
    return vals.astype(np.float32).reshape(-1)


def dequant_mlx4(words: np.ndarray, scales: np.ndarray, biases: np.ndarray, group: int) -> np.ndarray:
    w = np.ascontiguousarray(words, np.uint32)
    out = w.shape[0]
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    q = ((w[:, :, None] >> shifts) & 0xF).reshape(out, -1).astype(np.float32)
    s = np.repeat(np.asarray(scales, np.float32).reshape(out, -1), group, axis=1)
    b = np.repeat(np.asarray(biases, np.float32).reshape(out, -1), group, axis=1)
    return (q * s).astype(np.float32) + b


def matvec_f64(wf: np.ndarray, x: np.ndarray) -> np.ndarray:
    """High-precision product used for size-independent property checks."""
    return (wf.astype(np.float64) @ np.asarray(x, np.float64)).astype(np.float32)
