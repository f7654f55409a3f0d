"""GPU parity tests of the persistent matvec chain (``ullm_cuda_weight_matvec_chain_dev``): a list
of matvecs in one launch, with a grid-wide barrier where an op consumes an earlier op's output.
Checked against the CPU oracle with the reference's metric and fp32 bar
(``max|gpu-cpu| / max(max|cpu|, 1e-6) < 1e-3``, crates/ullm-metal/src/lib.rs:336-343) and against
the same ops run as separate launches."""
import numpy as np
import pytest
import torch

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3
GEN = {backend.Q4_K: synth.gen_q4k, backend.Q6_K: synth.gen_q6k}


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def make(ctx, dtype, out, cols, seed):
    w = GEN[dtype](out, cols, seed)
    return backend.Weight(ctx, dtype, w, out, cols), oracle.Weight(dtype, w, out, cols)


def run(ctx, ops, chain=True):
    ctx.debug_set("no_chain", 0 if chain else 1)
    try:
        st = torch.cuda.Stream()
        backend.WeightChain(ctx, ops).launch(st.cuda_stream)
        st.synchronize()
        ctx.synchronize()
        return ctx.last_plan()["grid"]
    finally:
        ctx.debug_set("no_chain", 0)


def test_independent_ops_one_launch(ctx):
    """The projections of one layer that share no data (batch call): mixed formats and shapes."""
    shapes = [(backend.Q4_K, 1024, 2048), (backend.Q6_K, 256, 2048), (backend.Q4_K, 300, 512), (backend.Q6_K, 128, 4096),
              (backend.Q4_K, 2048, 8192)]
    ops, refs, ys = [], [], []
    for i, (dt, out, cols) in enumerate(shapes):
        gw, ow = make(ctx, dt, out, cols, 50 + i)
        x = synth.normal(60 + i, cols)
        y = torch.zeros(out, device="cuda")
        ops.append(dict(w=gw, x=dev_f32(x), y=y))
        ops[-1]["x_keep"] = ops[-1]["x"]
        ops[-1]["x"] = ops[-1]["x_keep"].data_ptr()
        ys.append(y)
        ops[-1]["y"] = y.data_ptr()
        refs.append(oracle.matvec_q(ow, x))
    assert run(ctx, ops) == -2, "the chain kernel did not run"
    for y, ref in zip(ys, refs):
        assert synth.rel_err(y.cpu().numpy(), ref) < TOL


@pytest.mark.parametrize("shape", ["small", "c1"])
def test_dependent_pair(ctx, shape):
    """up then down on its result (the benchmark's FFN pair): the second op waits at the grid barrier."""
    hid, ff = (512, 2048) if shape == "small" else (4096, 14336)
    up_g, up_o = make(ctx, backend.Q6_K if shape == "c1" else backend.Q4_K, ff, hid, 71)
    dn_g, dn_o = make(ctx, backend.Q6_K, hid, ff if shape == "small" else 14336, 72)
    x = synth.normal(73, hid)
    h_ref = oracle.matvec_q(up_o, x)
    y_ref = oracle.matvec_q(dn_o, h_ref)
    xd, h, y = dev_f32(x), torch.zeros(ff, device="cuda"), torch.zeros(hid, device="cuda")
    ops = [dict(w=up_g, x=xd.data_ptr(), y=h.data_ptr()), dict(w=dn_g, x=h.data_ptr(), y=y.data_ptr(), dep=True)]
    assert run(ctx, ops) == -2
    assert synth.rel_err(h.cpu().numpy(), h_ref) < TOL
    assert synth.rel_err(y.cpu().numpy(), y_ref) < TOL
    # the same list as separate launches gives the same numbers to fp32 summation order
    h2, y2 = torch.zeros_like(h), torch.zeros_like(y)
    ops2 = [dict(w=up_g, x=xd.data_ptr(), y=h2.data_ptr()), dict(w=dn_g, x=h2.data_ptr(), y=y2.data_ptr(), dep=True)]
    assert run(ctx, ops2, chain=False) != -2
    assert synth.rel_err(y.cpu().numpy(), y2.cpu().numpy()) < 1e-4
    # repeated launches re-arm the barrier
    for _ in range(3):
        y.zero_()
        run(ctx, ops)
    assert synth.rel_err(y.cpu().numpy(), y_ref) < TOL


def test_ffn_block_with_norm_swiglu_residual(ctx):
    """x += W_o a;  x += W_down (silu(W_gate n) * (W_up n)), n = rmsnorm(x)  — the dense tail of a layer
    (crates/ullm-model/src/lib.rs:940-969) as three dependent ops."""
    D, F, eps = 2048, 8192, 1e-5
    wo_g, wo_o = make(ctx, backend.Q4_K, D, D, 81)
    wg, wu = synth.gen_q4k(F, D, 82), synth.gen_q4k(F, D, 83)
    gu = np.empty((2 * F, wg.shape[1]), np.uint8)  # rows interleaved gate0, up0, gate1, up1 ...
    gu[0::2], gu[1::2] = wg.reshape(F, -1), wu.reshape(F, -1)
    gu_g = backend.Weight(ctx, backend.Q4_K, gu, 2 * F, D)
    dn_g, dn_o = make(ctx, backend.Q6_K, D, F, 84)
    a, x0 = synth.normal(85, D), synth.normal(86, D)
    nw = (1.0 + 0.1 * synth.normal(87, D)).astype(np.float32)
    x1 = x0 + oracle.matvec_q(wo_o, a)
    n = oracle.rmsnorm(x1, nw, eps)
    g = oracle.matvec_q(oracle.Weight(backend.Q4_K, wg, F, D), n)
    u = oracle.matvec_q(oracle.Weight(backend.Q4_K, wu, F, D), n)
    hh = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
    x2 = x1 + oracle.matvec_q(dn_o, hh)
    ad, xd, nwd, hd = dev_f32(a), dev_f32(x0), dev_f32(nw), torch.zeros(F, device="cuda")
    ops = [
        dict(w=wo_g, x=ad.data_ptr(), y=xd.data_ptr(), epi=backend.EPI_RESIDUAL, res=xd.data_ptr()),
        dict(w=gu_g, x=xd.data_ptr(), y=hd.data_ptr(), norm_w=nwd.data_ptr(), eps=eps, epi=backend.EPI_SWIGLU, dep=True),
        dict(w=dn_g, x=hd.data_ptr(), y=xd.data_ptr(), epi=backend.EPI_RESIDUAL, res=xd.data_ptr(), dep=True),
    ]
    assert run(ctx, ops) == -2
    assert synth.rel_err(hd.cpu().numpy(), hh) < TOL
    assert synth.rel_err(xd.cpu().numpy(), x2) < TOL


def test_unsupported_weights_fall_back_to_separate_launches(ctx):
    w, s, b = synth.gen_mlx4(64, 256, 64, 5)
    gw = backend.Weight(ctx, backend.MLX_U32, w, 64, 256, scales=s, biases=b, group=64)
    x = synth.normal(91, 256)
    xd, y = dev_f32(x), torch.zeros(64, device="cuda")
    assert run(ctx, [dict(w=gw, x=xd.data_ptr(), y=y.data_ptr())]) != -2
    ref = oracle.matvec_q(oracle.Weight(backend.MLX_U32, w, 64, 256, synth.bf16_to_f32(s), synth.bf16_to_f32(b), 64), x)
    assert synth.rel_err(y.cpu().numpy(), ref) < TOL


@pytest.mark.parametrize("world", [2, 8])
def test_rank_shares_of_the_70b_block_in_one_launch(ctx, world):
    """What one rank of the row-sharded 70B-shaped block launches per step (bench.py, N > 1): its 1/N of the
    rows of all seven matrices in one batch call.  At N = 8 the k / v shares are 128 rows: fewer rows than CTAs,
    so most CTAs stream nothing for those ops but still walk the ring and the barriers."""
    mats = [(backend.Q4_K, 8192, 8192), (backend.Q4_K, 1024, 8192), (backend.Q4_K, 1024, 8192), (backend.Q4_K, 8192, 8192),
            (backend.Q4_K, 28672, 8192), (backend.Q4_K, 28672, 8192), (backend.Q6_K, 8192, 28672)]
    ws, xs, ys, refs = [], [], [], []
    for i, (dt, out, cols) in enumerate(mats):
        rows = out // world
        gw, ow = make(ctx, dt, rows, cols, 300 + i)
        x = synth.normal(310 + i, cols)
        ws.append(gw), xs.append(dev_f32(x)), ys.append(torch.zeros(rows, device="cuda"))
        refs.append(oracle.matvec_q(ow, x))
    st = torch.cuda.Stream()
    backend.WeightBatch(ctx, ws, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys]).launch(st.cuda_stream)
    st.synchronize()
    ctx.synchronize()
    assert ctx.last_plan()["grid"] == -2, "the chain kernel did not run"
    for y, ref in zip(ys, refs):
        assert synth.rel_err(y.cpu().numpy(), ref) < TOL


def test_read_probe_reports_both_ways_of_reading(ctx):
    """The measurement tool behind ``roofline.read_only_ceiling``: both modes run, return ordered statistics and
    a plausible rate (above 1 TB/s on any B200, below 20), and bad arguments are refused before any launch."""
    for mode in (0, 1):
        r = ctx.read_probe(mode, 256 << 20, 94208, 2, 16384, reps=3)
        assert r["us_min"] <= r["us"] <= r["us_max"]
        assert 1000.0 < r["gbs"] < 20000.0, r
    with pytest.raises(backend.UllmError):
        ctx.read_probe(1, 256 << 20, 94208, 3, 16384)  # three such stages do not fit in shared memory
    with pytest.raises(backend.UllmError):
        ctx.read_probe(2, 256 << 20)
