"""Row sharding of a quantized matrix over the ranks of one node: the index arithmetic.

Output rows of ``y = W x`` are independent (the reference parallelises its CPU
matvec over them, crates/ullm-model/src/math.rs:11-21), and a row of a GGUF /
MLX matrix is a self-contained byte range, so rank ``r`` of ``N`` keeps rows
``[r*out/N, (r+1)*out/N)`` and the path has one exchange: every rank's output
rows must reach every rank.  The library does that inside its kernels
(``ullm_cuda_shard_*``: each rank stores its rows into all ranks' full-length
result vectors, laid out by :func:`vector_offsets`); the NCCL comparison arm
all-gathers the ranks' concatenated rows instead, which produces the
``[rank][matrix][rows]`` layout that :func:`split_gathered` undoes.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = {12: 144, 14: 210}  # ggml ids -> bytes per 256-element super-block


def row_range(out_dim: int, world: int, rank: int) -> tuple[int, int]:
    if out_dim % world:
        raise ValueError(f"{out_dim} rows do not split evenly over {world} ranks")
    n = out_dim // world
    return rank * n, (rank + 1) * n


def row_bytes(dtype: int, cols: int) -> int:
    return cols // 256 * BLOCK_BYTES[dtype]


def slice_rows(dtype: int, w_bytes, out_dim: int, cols: int, world: int, rank: int) -> np.ndarray:
    """The bytes of this rank's rows of a row-major quantized matrix."""
    rb = row_bytes(dtype, cols)
    b = np.ascontiguousarray(w_bytes).view(np.uint8).reshape(-1)
    if b.size < out_dim * rb:
        raise ValueError("weight buffer shorter than out_dim rows")
    lo, hi = row_range(out_dim, world, rank)
    return b[lo * rb : hi * rb]


def vector_offsets(out_dims, align: int = 64) -> list[int]:
    """Where the full-length result vector of each matrix starts inside a rank's gather buffer (floats), every
    vector on an ``align``-float boundary; the last entry is the total length.  Identical on all ranks."""
    offs, o = [], 0
    for d in out_dims:
        offs.append(o)
        o += -(-d // align) * align
    return offs + [o]


def step_region(step: int, total: int) -> int:
    """Offset of the region of the gather buffer that step ``step`` fills: two regions, used by alternate steps,
    because a rank may run one step ahead of a peer that is still reading the previous result."""
    return (step & 1) * total


def owed_element(j: int, gather_off: int, out_dim: int, world: int, rank: int) -> int:
    """Tagged exchange: the ``j``-th float of a matrix' full-length vector that rank ``rank`` does NOT compute
    itself (0 <= j < out_dim - out_dim/world), as an index into the gather buffer.  The receiving kernel's threads
    share these out: each polls the {value, step} pair of its elements and writes the value into the vector."""
    lo, hi = row_range(out_dim, world, rank)
    if not 0 <= j < out_dim - (hi - lo):
        raise ValueError("no such owed element")
    return gather_off + (j if j < lo else j + (hi - lo))


def pair_slot(step: int, gather_floats: int, e: int) -> int:
    """Index of the {value, step} pair of gather-buffer float ``e`` in a rank's pair area: two halves used by
    alternate steps, so that a rank one step ahead writes beside, not over, pairs its peer has yet to take."""
    return (step & 1) * gather_floats + e


def local_offsets(out_dims, world: int) -> list[int]:
    """Offsets of each matrix' rows inside a rank's concatenated output."""
    offs, o = [], 0
    for d in out_dims:
        if d % world:
            raise ValueError(f"{d} rows do not split evenly over {world} ranks")
        offs.append(o)
        o += d // world
    return offs + [o]


def split_gathered(y_all, out_dims, world: int) -> list[np.ndarray]:
    """``y_all`` is the all-gathered ``[rank][matrix][rows]`` buffer; returns the full
    output vector of every matrix (rank-major rows, i.e. original row order)."""
    offs = local_offsets(out_dims, world)
    per_rank = np.asarray(y_all).reshape(world, offs[-1])
    return [per_rank[:, offs[i] : offs[i + 1]].reshape(-1) for i in range(len(out_dims))]


def split_gathered_tokens(y_all, out_dims, world: int, tokens: int) -> list[np.ndarray]:
    """Prefill form: ``y_all`` is ``[rank][matrix][token][rows/N]`` (each rank's token-major GEMM
    outputs on its row slices, concatenated, then all-gathered); returns ``[tokens, out]`` per matrix."""
    offs = local_offsets(out_dims, world)
    per_rank = np.asarray(y_all).reshape(world, tokens * offs[-1])
    res = []
    for i, d in enumerate(out_dims):
        n = d // world
        blk = per_rank[:, tokens * offs[i] : tokens * offs[i + 1]].reshape(world, tokens, n)
        res.append(np.ascontiguousarray(blk.transpose(1, 0, 2)).reshape(tokens, d))
    return res
