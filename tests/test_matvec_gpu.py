"""GPU parity tests (through the C ABI) for dequantization and the batch-1 matvec
against the CPU oracle.  Dequantized values are compared bit for bit; matvec
outputs with the reference's own metric (crates/ullm-metal/src/lib.rs:336-343):
max|gpu-cpu| / max(max|cpu|, 1e-6) < 1e-3."""
import os

import numpy as np
import pytest

import np_formats as nf
import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the tolerance stated for the fp32-accumulate matvec
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_small.npz"))

GEN = {backend.Q4_K: synth.gen_q4k, backend.Q6_K: synth.gen_q6k}
BLK = {backend.Q4_K: 144, backend.Q6_K: 210}


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- dequantization: bit-exact ----------------------------------------------
@pytest.mark.parametrize("dtype", [backend.Q4_K, backend.Q6_K])
@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 768), (64, 4096)])
def test_dequant_bit_exact_config_distribution(ctx, dtype, rows, cols):
    w = GEN[dtype](rows, cols, 11)
    got = ctx.dequantize(dtype, w, rows * cols)
    assert np.array_equal(bits(got), bits(oracle.dequantize(dtype, w, rows * cols)))


@pytest.mark.parametrize("dtype,doffs", [(backend.Q4_K, (0, 2)), (backend.Q6_K, (208,))])
def test_dequant_bit_exact_arbitrary_bytes(ctx, dtype, doffs):
    blk = BLK[dtype]
    w = synth.rand_bytes(123, 512 * blk).reshape(512, blk).copy()
    for off in doffs:
        w[:, off + 1] &= 0xBB  # finite f16 only (NaN payloads are not comparable)
    w[0, doffs[0] : doffs[0] + 2] = (0x01, 0x00)  # subnormal d (dequant.rs:20)
    w[1, doffs[0] : doffs[0] + 2] = (0x00, 0x80)  # -0
    got = ctx.dequantize(dtype, w, 512 * 256)
    assert np.array_equal(bits(got), bits(oracle.dequantize(dtype, w, 512 * 256)))


def test_dequant_mlx_bit_exact(ctx):
    w, s, b = synth.gen_mlx4(48, 768, 64, 5)
    s32, b32 = synth.bf16_to_f32(s), synth.bf16_to_f32(b)
    assert np.array_equal(bits(ctx.dequantize_mlx_q4(w, s32, b32, 48, 768, 64)), bits(oracle.dequantize_mlx_q4(w, s32, b32, 48, 768, 64)))
    # f32 tables that are not bf16-representable: q*scale rounds before the add
    s32 = synth.uniform_range(1, s.size, 0.005, 0.03).astype(np.float32).reshape(s.shape)
    b32 = synth.uniform_range(2, s.size, -0.1, 0.1).astype(np.float32).reshape(s.shape)
    assert np.array_equal(bits(ctx.dequantize_mlx_q4(w, s32, b32, 48, 768, 64)), bits(oracle.dequantize_mlx_q4(w, s32, b32, 48, 768, 64)))


def test_dequant_mlx_reference_kat(ctx):  # dequant.rs:324-334
    y = ctx.dequantize_mlx_q4([[2569837433]], [[0.004425049]], [[-0.039794922]], 1, 8, 8)[0]
    assert np.all(np.abs(y - np.array([3e-5, -0.00882, 0.00888, 3e-5, 0.01331, -0.03094, 3e-5, 3e-5], np.float32)) < 1e-4)


def test_dequant_golden_fixture(ctx):
    for name, dt in (("q4k", backend.Q4_K), ("q6k", backend.Q6_K)):
        w = GOLD[f"{name}_w"]
        assert np.array_equal(bits(ctx.dequantize(dt, w, GOLD[f"{name}_deq"].size)), bits(GOLD[f"{name}_deq"]))
    s32, b32 = synth.bf16_to_f32(GOLD["mlx_s"]), synth.bf16_to_f32(GOLD["mlx_b"])
    assert np.array_equal(bits(ctx.dequantize_mlx_q4(GOLD["mlx_w"], s32, b32, 24, 512, 64)), bits(GOLD["mlx_deq"]))


def test_dequant_errors(ctx):  # dequant.rs:65-77, :103-107
    with pytest.raises(backend.FormatError):
        ctx.dequantize(backend.Q4_K, np.zeros(144, np.uint8), 255)
    with pytest.raises(backend.FormatError):
        ctx.dequantize(backend.Q6_K, np.zeros(100, np.uint8), 256)
    with pytest.raises(backend.Unsupported):
        ctx.dequantize(backend.MLX_U32, np.zeros(16, np.uint8), 4)
    assert ctx.dequantize(backend.Q4_K, np.zeros(0, np.uint8), 0).size == 0


# ---- matvec: the reference's own unit-test pattern ------------------------------
@pytest.mark.parametrize("dtype,doffs", [(backend.Q4_K, (0, 2)), (backend.Q6_K, (208,))])
@pytest.mark.parametrize("generic", [0, 1])
def test_check_quant_pattern(ctx, dtype, doffs, generic):  # crates/ullm-metal/src/lib.rs:358-391
    w = synth.check_quant_weights(BLK[dtype], doffs)
    x = synth.check_quant_x()
    cpu = oracle.matvec_q(oracle.Weight(dtype, w, 256, 512), x)
    ctx.debug_set("force_generic", generic)
    try:
        gpu = ctx.matvec_quant(dtype, w, x, 256, 512)
        assert ctx.last_plan()["streamed"] == (0 if generic else 1)
    finally:
        ctx.debug_set("force_generic", 0)
    assert synth.rel_err(gpu, cpu) < TOL


@pytest.mark.parametrize("generic", [0, 1])
def test_mlx4_gemv_pattern(ctx, generic):  # crates/ullm-metal/src/lib.rs:395-430
    w, s, b = synth.check_mlx4()
    x = synth.check_quant_x(256)
    cpu = oracle.matvec_q(oracle.Weight(oracle.MLX_U32, w, 96, 256, s, b, 64), x)
    ctx.debug_set("force_generic", generic)
    try:
        gpu = ctx.matvec_mlx4(w, s, b, x, 96, 256, 64)
    finally:
        ctx.debug_set("force_generic", 0)
    assert synth.rel_err(gpu, cpu) < TOL


# ---- matvec: benchmark configurations and edge shapes ---------------------------
SHAPES = [
    # (dtype, out, in)                 what it covers
    (backend.Q4_K, 4096, 4096),      # config 0
    (backend.Q6_K, 14336, 4096),     # config 1, up
    (backend.Q6_K, 4096, 14336),     # config 1, down (14 column groups)
    (backend.Q4_K, 512, 2048),       # config 3, attn_k
    (backend.Q6_K, 2048, 8192),      # config 3, ffn_down
    (backend.Q4_K, 1024, 8192),      # config 4, k/v
    (backend.Q6_K, 64, 28672),       # config 4 down width: two column groups per warp
    (backend.Q4_K, 64, 28672),       # config 4 gate/up width transposed: 14 column groups
    (backend.Q4_K, 1, 256),          # a single block
    (backend.Q6_K, 1, 256),
    (backend.Q4_K, 7, 2304),         # ragged rows, column group only partly filled
    (backend.Q6_K, 24, 768),         # rows that are not 16-byte multiples (630 B)
    (backend.Q6_K, 21, 768),         # ... with a ragged row count: fallback kernel
    (backend.Q4_K, 1000, 512),       # out not a multiple of any tile
    (backend.Q6_K, 333, 1024),
]


@pytest.mark.parametrize("dtype,out,cols", SHAPES)
def test_matvec_matches_oracle(ctx, dtype, out, cols):
    w = GEN[dtype](out, cols, synth.seed_for(0, out % 13))
    x = synth.normal(synth.seed_for(0, 1), cols)
    cpu = oracle.matvec_q(oracle.Weight(dtype, w, out, cols), x)
    gpu = ctx.matvec_quant(dtype, w, x, out, cols)
    assert synth.rel_err(gpu, cpu) < TOL, ctx.last_plan()
    ctx.debug_set("force_generic", 1)
    try:
        gen = ctx.matvec_quant(dtype, w, x, out, cols)
    finally:
        ctx.debug_set("force_generic", 0)
    assert synth.rel_err(gen, cpu) < TOL


@pytest.mark.parametrize("out,cols,group", [(768, 2048, 64), (2048, 768, 64), (100, 256, 32), (33, 1024, 128), (16, 64, 8)])
@pytest.mark.parametrize("bf16_tables", [0, 1])
def test_matvec_mlx_matches_oracle(ctx, out, cols, group, bf16_tables):
    w, s, b = synth.gen_mlx4(out, cols, group, synth.seed_for(2, 0))
    x = synth.normal(synth.seed_for(2, 1), cols)
    s32, b32 = synth.bf16_to_f32(s), synth.bf16_to_f32(b)
    cpu = oracle.matvec_q(oracle.Weight(oracle.MLX_U32, w, out, cols, s32, b32, group), x)
    if not bf16_tables:
        gpu = ctx.matvec_mlx4(w, s32, b32, x, out, cols, group)
    else:  # tables kept as the bf16 bits on disk, resident, device-pointer form
        bw, bs, bb, bx = ctx.upload(w), ctx.upload(s), ctx.upload(b), ctx.upload(x)
        by = ctx.alloc(out * 4)
        ctx.matvec_dev(backend.MLX_U32, bw.ptr, bx.ptr, by.ptr, out, cols, d_scales=bs.ptr, d_biases=bb.ptr,
                       table_dtype=backend.BF16, group=group)
        ctx.synchronize()
        gpu = by.download().view(np.float32)
    assert synth.rel_err(gpu, cpu) < TOL, ctx.last_plan()


def test_matvec_resident_and_golden_fixture(ctx):
    for name, dt in (("q4k", backend.Q4_K), ("q6k", backend.Q6_K)):
        w, x, y = GOLD[f"{name}_w"], GOLD[f"{name}_x"], GOLD[f"{name}_y"]
        buf = ctx.upload(w)
        got = ctx.matvec_resident(dt, buf, x, y.size, x.size)
        assert synth.rel_err(got, y) < TOL
        again = ctx.matvec_resident(dt, buf, x, y.size, x.size)
        assert np.array_equal(got, again)  # deterministic reduction order
    s32, b32 = synth.bf16_to_f32(GOLD["mlx_s"]), synth.bf16_to_f32(GOLD["mlx_b"])
    assert synth.rel_err(ctx.matvec_mlx4(GOLD["mlx_w"], s32, b32, GOLD["mlx_x"], 24, 512, 64), GOLD["mlx_y"]) < TOL


def test_matvec_activation_outliers_and_zeros(ctx):
    """The fixed-point re-expression of x is scaled per small group, so a huge
    outlier must not wipe out its neighbours; all-zero groups must give zero."""
    out, cols = 256, 4096
    for dtype in (backend.Q4_K, backend.Q6_K):
        w = GEN[dtype](out, cols, 21)
        x = synth.normal(22, cols)
        x[100] = 3.0e4
        x[2000:2300] = 0.0
        x[3000] = -1.0e-30
        cpu = oracle.matvec_q(oracle.Weight(dtype, w, out, cols), x)
        # compare against the exact product: the outlier makes the f32 oracle itself noisy
        wf = (nf.dequant_q4k if dtype == backend.Q4_K else nf.dequant_q6k)(w, out * cols).reshape(out, cols)
        exact = nf.matvec_f64(wf, x)
        gpu = ctx.matvec_quant(dtype, w, x, out, cols)
        assert synth.rel_err(gpu, exact) < TOL
        assert synth.rel_err(cpu, exact) < TOL
        zero = ctx.matvec_quant(dtype, w, np.zeros(cols, np.float32), out, cols)
        assert np.all(zero == 0)


def _group_bound(dtype, wf, x):
    """Analytic bound on |gpu_row - exact_row| of the streamed kernels.  They re-express x as 16-bit fixed point
    with one scale per group of values that share a weight scale (32 for Q4_K, 64 for prepared Q6_K rows), so an
    element is off by at most half a step, max|x_g| / 65534, and a row by at most
    sum_g max|x_g| / 65534 * sum_{i in g} |w_i|; twice that is asserted (fp32 accumulation comes on top)."""
    g = 32 if dtype == backend.Q4_K else 64
    out, cols = wf.shape
    xm = np.abs(x.astype(np.float64)).reshape(cols // g, g).max(axis=1)
    wa = np.abs(wf).reshape(out, cols // g, g).sum(axis=2)
    return 2.0 * (wa @ xm) / 65534.0


@pytest.mark.parametrize("dtype", [backend.Q4_K, backend.Q6_K])
@pytest.mark.parametrize("mag", [1.0, 100.0, 1000.0])
def test_matvec_per_row_error_with_outlier_channels(ctx, dtype, mag):
    """Activations as a decoder produces them: a few channels far above the rest, inside ordinary groups (8 of
    4096 at `mag` times the others).  Three statements about the streamed, fixed-point-x kernel: the reference's
    max-norm metric stays far inside 1e-3; every row stays inside the analytic bound of `_group_bound`; and the
    error of a row, relative to that row's own value (rows of at least 5 % of the largest), stays inside 1e-3
    too, with or without the outliers - the scale is per group, so an outlier costs its own group only."""
    out, cols = 1024, 4096
    w = GEN[dtype](out, cols, 21)
    wf = (nf.dequant_q4k if dtype == backend.Q4_K else nf.dequant_q6k)(w, out * cols).reshape(out, cols).astype(np.float64)
    x = synth.normal(22, cols)
    pos = synth.rand_ints(23, 8, 0, cols - 1)
    if mag > 1:
        x[pos] = mag * np.where(x[pos] < 0, -1.0, 1.0).astype(np.float32)
    exact = wf @ x.astype(np.float64)
    wo = backend.Weight(ctx, dtype, w, out, cols)  # resident weight: Q6_K rows in the prepared layout
    gpu = wo.matvec(x).astype(np.float64)
    assert ctx.last_plan()["streamed"] == 1
    wo.free()
    err = np.abs(gpu - exact)
    top = np.abs(exact).max()
    assert err.max() / top < 1e-4  # the reference's metric: ten times inside the bar
    assert np.all(err <= _group_bound(dtype, wf, x) + 1e-6 * top)
    rows = np.abs(exact) >= 0.05 * top
    assert rows.sum() > out // 2
    assert (err[rows] / np.abs(exact)[rows]).max() < TOL


@pytest.mark.parametrize("dtype", [backend.Q4_K, backend.Q6_K])
@pytest.mark.parametrize("poison", [np.nan, np.inf])
def test_matvec_non_finite_activations_stay_non_finite(ctx, dtype, poison):
    """A NaN or an infinity in x reaches every output row in the reference's f32 product (math.rs:17); the
    fixed-point re-expression of x must not round it away (resident weights, streamed kernel; raw bytes too)."""
    out, cols = 256, 4096
    w = GEN[dtype](out, cols, 41)
    x = synth.normal(42, cols)
    x[1234] = poison
    wo = backend.Weight(ctx, dtype, w, out, cols)
    y = wo.matvec(x)
    assert ctx.last_plan()["streamed"] == 1
    assert not np.isfinite(y).any()
    assert not np.isfinite(ctx.matvec_quant(dtype, w, x, out, cols)).any()
    wo.free()


def test_matvec_linearity_at_full_size(ctx):
    """Size-independent property on the largest single matrices: W(a+b) = Wa + Wb."""
    for dtype, out, cols in ((backend.Q4_K, 28672, 8192), (backend.Q6_K, 8192, 28672)):
        w = GEN[dtype](out, cols, 31)
        buf = ctx.upload(w)
        a, b = synth.normal(32, cols), synth.normal(33, cols)
        ya = ctx.matvec_resident(dtype, buf, a, out, cols)
        yb = ctx.matvec_resident(dtype, buf, b, out, cols)
        yab = ctx.matvec_resident(dtype, buf, a + b, out, cols)
        assert synth.rel_err(yab, ya + yb) < TOL
        # and a spot check of 64 rows against the oracle
        rows = np.linspace(0, out - 1, 64).astype(int)
        sub = np.ascontiguousarray(w[rows])
        cpu = oracle.matvec_q(oracle.Weight(dtype, sub, 64, cols), a)
        assert synth.rel_err(ya[rows], cpu) < TOL
        buf.free()


def test_matvec_errors(ctx):
    w = synth.gen_q4k(4, 512, 1)
    x = np.zeros(512, np.float32)
    with pytest.raises(backend.Unsupported):  # MetalContext::pso_for, lib.rs:268-276
        ctx.matvec_quant(backend.F32, w, x, 4, 512)
    with pytest.raises(backend.Unsupported):
        ctx.matvec_quant(8, w, x, 4, 512)  # Q8_0 has no GPU kernel in the reference either
    with pytest.raises(backend.FormatError):
        ctx.matvec_quant(backend.Q4_K, w, x, 4, 500)
    with pytest.raises(backend.FormatError):
        ctx.matvec_quant(backend.Q4_K, w, x, 5, 512)  # short weight buffer
    with pytest.raises(backend.FormatError):
        ctx.matvec_mlx4(np.zeros((4, 8), np.uint32), np.zeros((4, 1)), np.zeros((4, 1)), np.zeros(64), 4, 64, 48)
    assert "NVIDIA" in ctx.device_name()


# ---- batched matmul ------------------------------------------------------------
@pytest.mark.parametrize("dtype", [backend.Q4_K, backend.Q6_K])
def test_matmul_quant_matches_oracle(ctx, dtype):
    out, cols, s = 96, 512, 7  # s not a multiple of any tile (lib.rs:438)
    w = GEN[dtype](out, cols, 41)
    xs = synth.normal(42, s * cols).reshape(s, cols)
    cpu = oracle.matmul_q(oracle.Weight(dtype, w, out, cols), xs, s)
    gpu = ctx.matmul_quant(dtype, w, xs, out, cols, s)
    assert gpu.shape == (s, out) and synth.rel_err(gpu, cpu) < TOL


def test_matmul_mlx4_pattern(ctx):  # crates/ullm-metal/src/lib.rs:474-515: abs tol 1e-3
    w, sc, b = synth.check_mlx4()
    s = 5
    x = ((np.arange(s * 256) % 13).astype(np.float32) - 6.0) * np.float32(0.1)
    cpu = oracle.matmul_q(oracle.Weight(oracle.MLX_U32, w, 96, 256, sc, b, 64), x.reshape(s, 256), s)
    gpu = ctx.matmul_mlx4(w, sc, b, x, 96, 256, 64, s)
    assert np.max(np.abs(gpu - cpu)) < 1e-3


# ---- resident weight objects (prepared layouts) -----------------------------------
WEIGHT_SHAPES = [
    (backend.Q6_K, 14336, 4096),   # config 1 up: rows prepared (in % 2048 == 0)
    (backend.Q6_K, 4096, 14336),   # config 1 down
    (backend.Q6_K, 2048, 8192),
    (backend.Q6_K, 37, 2048),      # ragged row count, one column group partly filled
    (backend.Q6_K, 64, 28672),     # two column groups per warp
    (backend.Q6_K, 24, 768),       # rows not 16-byte multiples: stays verbatim
    (backend.Q4_K, 4096, 4096),
    (backend.Q4_K, 1000, 512),
]


@pytest.mark.parametrize("dtype,out,cols", WEIGHT_SHAPES)
def test_weight_object_matvec_and_lossless_export(ctx, dtype, out, cols):
    w = GEN[dtype](out, cols, synth.seed_for(1, out % 7))
    x = synth.normal(synth.seed_for(1, 3), cols)
    wt = backend.Weight(ctx, dtype, w, out, cols)
    got = wt.matvec(x)
    cpu = oracle.matvec_q(oracle.Weight(dtype, w, out, cols), x)
    assert synth.rel_err(got, cpu) < TOL, ctx.last_plan()
    assert np.array_equal(wt.export(), w.reshape(-1))  # the prepared layout loses nothing
    assert np.array_equal(got, wt.matvec(x))
    wt.free()


def test_weight_object_mlx_and_errors(ctx):
    w, s, b = synth.gen_mlx4(768, 2048, 64, 9)
    x = synth.normal(10, 2048)
    cpu = oracle.matvec_q(oracle.Weight(oracle.MLX_U32, w, 768, 2048, synth.bf16_to_f32(s), synth.bf16_to_f32(b), 64), x)
    for tables in ((s, b), (synth.bf16_to_f32(s), synth.bf16_to_f32(b))):
        wt = backend.Weight(ctx, backend.MLX_U32, w, 768, 2048, tables[0], tables[1], 64)
        assert synth.rel_err(wt.matvec(x), cpu) < TOL
        wt.free()
    with pytest.raises(backend.Unsupported):
        backend.Weight(ctx, backend.F32, np.zeros(16, np.float32), 4, 4)
    with pytest.raises(backend.FormatError):
        backend.Weight(ctx, backend.Q4_K, np.zeros(100, np.uint8), 4, 256)


@pytest.mark.parametrize("wr,rw", [(1, 1), (2, 2), (3, 4), (6, 1), (12, 1)])
def test_streamed_plan_variants_agree(ctx, wr, rw):
    """Every tile shape the planner may pick computes the same product."""
    out, cols = 1111 * 0 + 1024, 4096
    for dtype in (backend.Q6_K, backend.Q4_K):
        w = GEN[dtype](out, cols, 51)
        x = synth.normal(52, cols)
        cpu = oracle.matvec_q(oracle.Weight(dtype, w, out, cols), x)
        wt = backend.Weight(ctx, dtype, w, out, cols)
        ctx.debug_set("plan_wr", wr)
        ctx.debug_set("plan_rw", rw)
        try:
            got = wt.matvec(x)
            plan = ctx.last_plan()
        finally:
            ctx.debug_set("plan_wr", 0)
            ctx.debug_set("plan_rw", 0)
        assert plan["streamed"] == 1 and plan["rows_per_tile"] == wr * rw, plan
        assert synth.rel_err(got, cpu) < TOL
        wt.free()


def test_host_vectors_pinned_and_pageable_take_the_same_values(ctx):
    """``ullm_cuda_weight_matvec`` moves page-locked host vectors with small kernels and pageable ones with
    cudaMemcpyAsync: same results either way, odd lengths and unaligned views included."""
    import torch

    out, cols = 1030, 2048  # out not a multiple of 4: the copy kernel's scalar tail
    wb = synth.gen_q4k(out, cols, 21)
    w = backend.Weight(ctx, backend.Q4_K, wb, out, cols)
    x = synth.normal(22, cols)
    ref = oracle.matvec_q(oracle.Weight(backend.Q4_K, wb, out, cols), x)
    y_pageable = w.matvec(x.copy())
    xp = torch.from_numpy(x.copy()).pin_memory().numpy()
    yp = torch.empty(out + 1, dtype=torch.float32).pin_memory().numpy()
    y_pinned = w.matvec(xp, out=yp[:out]).copy()  # a copy: the next call writes the same buffer
    y_unaligned = w.matvec(xp, out=yp[1:]).copy()  # destination 4 bytes off a 16-byte boundary
    assert np.array_equal(y_pageable, y_pinned) and np.array_equal(y_pageable, y_unaligned)
    assert synth.rel_err(y_pinned, ref) < 1e-3
    ctx.debug_set("no_host_kernels", 1)
    try:
        assert np.array_equal(w.matvec(xp), y_pageable)
    finally:
        ctx.debug_set("no_host_kernels", 0)
    w.free()
