"""GPU parity tests for the prefill GEMM on quantized weights (tensor-core path behind
``ullm_cuda_matmul_quant`` / ``ullm_cuda_weight_matmul``) against the CPU oracle's
``matmul_q`` (crates/ullm-model/src/math.rs:38-63).

Two bars.  (1) The stated one for bf16 tensor-core products: the reference's relative
metric ``max|gpu-cpu| / max(max|cpu|, 1e-6) < 2e-2`` against the oracle's f32 result.
(2) A much tighter one that pins the data path itself: the oracle's exact dequantized
weights and the activations are rounded to bf16 on the host exactly as the kernel
rounds them, multiplied in float64, and the kernel must agree to 2e-5 — only the fp32
accumulation order is left to differ, so one misplaced element shows."""
import numpy as np
import pytest

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2  # the tolerance stated for the bf16 tensor-core GEMM
TOL_PATH = 2e-5  # fp32 accumulation order only

GEN = {backend.Q4_K: synth.gen_q4k, backend.Q6_K: synth.gen_q6k}


def bf16_round(a):
    return synth.bf16_to_f32(synth.f32_to_bf16(np.ascontiguousarray(a, np.float32)))


def expected(dtype, w, xs, out_dim, in_dim, s):
    ow = oracle.Weight(dtype, w, out_dim, in_dim)
    y_oracle = oracle.matmul_q(ow, xs, s)
    wd = bf16_round(oracle.dequantize(dtype, w, out_dim * in_dim)).reshape(out_dim, in_dim).astype(np.float64)
    xb = bf16_round(xs).reshape(s, in_dim).astype(np.float64)
    return y_oracle, (xb @ wd.T)


def check(got, y_oracle, y_path, in_dim=2048):
    assert synth.rel_err(got, y_oracle) < TOL_BF16
    # what the accumulation order leaves grows with the square root of the number of terms
    assert synth.rel_err(got, y_path.astype(np.float32)) < TOL_PATH * max(1.0, (in_dim / 2048.0) ** 0.5)


SHAPES = [
    # dtype, out, in, s
    (backend.Q4_K, 128, 256, 32),     # one tile, one k block
    (backend.Q4_K, 96, 512, 7),       # ragged rows and tokens (forced onto the GEMM)
    (backend.Q4_K, 300, 1024, 300),   # 3 row tiles (last ragged), 2 token tiles (last ragged)
    (backend.Q4_K, 2048, 2048, 512),  # Llama-3.2-1B wq at the headline prefill length
    (backend.Q6_K, 128, 2048, 64),
    (backend.Q6_K, 200, 4096, 33),
    (backend.Q6_K, 1024, 2048, 512),
    (backend.Q4_K, 75 * 256 + 44, 512, 40),   # 76 row tiles on 74 CTA pairs: the last two go to a split-K launch
    (backend.Q6_K, 38 * 256, 2048, 300),      # 76 tiles (38 x 2 token tiles), prepared Q6_K, split-K tail
]


@pytest.mark.parametrize("dtype,out_dim,in_dim,s", SHAPES)
def test_matmul_quant_matches_oracle(ctx, dtype, out_dim, in_dim, s):
    w = GEN[dtype](out_dim, in_dim, 31)
    xs = synth.normal(1000 + out_dim + 7 * s, s * in_dim)
    ctx.debug_set("gemm_min_s", 1)
    try:
        got = ctx.matmul_quant(dtype, w, xs, out_dim, in_dim, s)
        assert ctx.last_plan()["grid"] == -1, "the tensor-core GEMM did not run"
    finally:
        ctx.debug_set("gemm_min_s", 32)
    check(got, *expected(dtype, w, xs, out_dim, in_dim, s))


@pytest.mark.parametrize("dtype,out_dim,in_dim,s", [(backend.Q4_K, 512, 2048, 160), (backend.Q6_K, 512, 2048, 160)])
def test_weight_object_matmul(ctx, dtype, out_dim, in_dim, s):
    w = GEN[dtype](out_dim, in_dim, 32)
    xs = synth.normal(77, s * in_dim)
    wo = backend.Weight(ctx, dtype, w, out_dim, in_dim)
    got = wo.matmul(xs, s)
    assert ctx.last_plan()["grid"] == -1
    check(got, *expected(dtype, w, xs, out_dim, in_dim, s))
    # repeated calls re-use the TMEM allocation and barriers cleanly
    assert np.array_equal(got, wo.matmul(xs, s))
    wo.free()


# The 70B-shaped block at the headline prefill length (512 tokens): every matrix shape of benchmark
# configuration 4.  The full oracle product would take minutes, so three bands of 64 rows (first, middle and
# last rows: the first tile, an interior tile and the ragged / split-K end) are compared for all 512 tokens,
# at both bars.
C4_SHAPES = [(backend.Q4_K, 8192, 8192), (backend.Q4_K, 1024, 8192), (backend.Q4_K, 28672, 8192), (backend.Q6_K, 8192, 28672)]


@pytest.mark.parametrize("dtype,out_dim,in_dim", C4_SHAPES)
def test_c4_shapes_at_512_tokens_row_bands_match_oracle(ctx, dtype, out_dim, in_dim):
    import torch

    s = 512
    w = GEN[dtype](out_dim, in_dim, 35)
    xs = bf16_round(synth.normal(36, s * in_dim))  # bf16-representable activations, as the configuration states
    wo = backend.Weight(ctx, dtype, w, out_dim, in_dim)
    xd = torch.from_numpy(xs).cuda()
    yd = torch.empty(s * out_dim, dtype=torch.float32, device="cuda")
    wo.matmul_dev(xd.data_ptr(), yd.data_ptr(), s)
    ctx.synchronize()
    assert ctx.last_plan()["grid"] == -1, "the tensor-core GEMM did not run"
    got = yd.view(s, out_dim)
    rb = in_dim // 256 * (144 if dtype == backend.Q4_K else 210)
    wb = np.asarray(w).reshape(-1).view(np.uint8)
    for r0 in (0, (out_dim // 2) // 64 * 64 + 64, out_dim - 64):
        blk = np.ascontiguousarray(wb[r0 * rb:(r0 + 64) * rb])
        check(got[:, r0:r0 + 64].cpu().numpy(), *expected(dtype, blk, xs, 64, in_dim, s), in_dim=in_dim)
    wo.free()


def test_small_batches_keep_the_f32_matvec_path(ctx):
    out_dim, in_dim, s = 256, 2048, 4
    w = synth.gen_q4k(out_dim, in_dim, 33)
    xs = synth.normal(78, s * in_dim)
    got = ctx.matmul_quant(backend.Q4_K, w, xs, out_dim, in_dim, s)
    assert ctx.last_plan()["grid"] != -1
    assert synth.rel_err(got, oracle.matmul_q(oracle.Weight(backend.Q4_K, w, out_dim, in_dim), xs, s)) < 1e-3


def test_gemm_check_pattern(ctx):
    """The reference's own matmul test inputs (crates/ullm-metal/src/lib.rs:348-377 pattern)."""
    out_dim, in_dim, s = 256, 512, 40
    w = synth.check_quant_weights(144, (0, 2), out_dim, in_dim)
    xs = np.concatenate([synth.check_quant_x(in_dim) * (1.0 + 0.01 * t) for t in range(s)]).astype(np.float32)
    ctx.debug_set("gemm_min_s", 1)
    try:
        got = ctx.matmul_quant(backend.Q4_K, w, xs, out_dim, in_dim, s)
    finally:
        ctx.debug_set("gemm_min_s", 32)
    check(got, *expected(backend.Q4_K, w, xs, out_dim, in_dim, s))


# ---- MLX 4-bit (matmul_mlx4, crates/ullm-metal/src/shader.metal:568; CPU form math.rs:38-79) on the tensor cores ----
def expected_mlx(w, s32, b32, xs, out_dim, in_dim, group, s):
    ow = oracle.Weight(oracle.MLX_U32, w, out_dim, in_dim, s32, b32, group)
    y_oracle = oracle.matmul_q(ow, xs, s)
    wd = bf16_round(oracle.dequantize_mlx_q4(w, s32, b32, out_dim, in_dim, group)).astype(np.float64)
    xb = bf16_round(xs).reshape(s, in_dim).astype(np.float64)
    return y_oracle, (xb @ wd.T)


@pytest.mark.parametrize("out_dim,in_dim,s", [(128, 256, 32), (768, 2048, 100), (2048, 768, 512), (300, 1024, 300), (200, 8192, 64)])
def test_matmul_mlx4_tensor_core_path(ctx, out_dim, in_dim, s):
    """f32 tables through the host entry point (what the reference passes) and bf16 tables on a resident weight;
    ragged rows and tokens, a split-K shape, the Qwen3-30B-A3B expert shapes."""
    gs = 64
    w, sc, bi = synth.gen_mlx4(out_dim, in_dim, gs, 61)
    s32, b32 = synth.bf16_to_f32(sc), synth.bf16_to_f32(bi)
    xs = synth.normal(62, s * in_dim)
    want = expected_mlx(w, s32, b32, xs, out_dim, in_dim, gs, s)
    got = ctx.matmul_mlx4(w, s32, b32, xs, out_dim, in_dim, gs, s)
    assert ctx.last_plan()["grid"] == -1, "the tensor-core GEMM did not run"
    check(got, *want, in_dim=in_dim)
    wo = backend.Weight(ctx, backend.MLX_U32, w, out_dim, in_dim, sc, bi, gs)  # bf16 tables as stored on disk
    got2 = wo.matmul(xs, s)
    if (in_dim // gs * 2) % 16 == 0:  # bf16 table rows are TMA rows only when their length is a multiple of 16 bytes
        assert ctx.last_plan()["grid"] == -1
        check(got2, *want, in_dim=in_dim)
        assert np.array_equal(got, got2)  # the same values whichever width the tables are kept in
    else:  # per-token matvecs: the f32 bar
        assert ctx.last_plan()["grid"] != -1
        assert synth.rel_err(got2, want[0]) < 1e-3
    wo.free()


def test_matmul_mlx4_other_groups_keep_the_matvec_path(ctx):
    out_dim, in_dim, s, gs = 96, 512, 40, 32
    w, sc, bi = synth.gen_mlx4(out_dim, in_dim, gs, 63)
    s32, b32 = synth.bf16_to_f32(sc), synth.bf16_to_f32(bi)
    xs = synth.normal(64, s * in_dim)
    got = ctx.matmul_mlx4(w, s32, b32, xs, out_dim, in_dim, gs, s)
    assert ctx.last_plan()["grid"] != -1
    ref = oracle.matmul_q(oracle.Weight(oracle.MLX_U32, w, out_dim, in_dim, s32, b32, gs), xs, s)
    assert synth.rel_err(got, ref) < 1e-3
