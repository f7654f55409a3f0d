"""GPU parity tests of the row-sharded path (``ullm_cuda_shard_*``): each rank computes its rows of
``y = W x`` (the split the reference's CPU path uses, crates/ullm-model/src/math.rs:11-21) and its
kernels store them into every rank's gather buffer; a published step number replaces the all-gather.

On one GPU the ranks of a group are emulated by several group members on the same device whose steps
are run one after the other without waiting (``ULLM_SHARD_NO_WAIT``) and then waited for: no kernel
ever waits for a kernel that has not been launched.  With two or more GPUs a real two-device group is
run as well.  Results are compared with the CPU oracle's full-matrix product (``rel_err < 1e-3``, the
metric of crates/ullm-metal/src/lib.rs:336-343) on every rank's copy.
"""
import numpy as np
import pytest
import torch

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3
GEN = {backend.Q4_K: synth.gen_q4k, backend.Q6_K: synth.gen_q6k}

# (dtype, out, cols): k/v- and gate-like slices, a prepared Q6_K matrix, a ragged-tile row count
MATS = [(backend.Q4_K, 1024, 2048), (backend.Q4_K, 256, 2048), (backend.Q6_K, 512, 4096), (backend.Q4_K, 1528, 1024)]


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def group(ctx, world, y_floats):
    shards = [backend.Shard(ctx, world, r, y_floats) for r in range(world)]
    if world > 1:
        backend.Shard.connect_local(shards)
    return shards


def full_problem(seed):
    ws, xs, refs, offs, off = [], [], [], [], 0
    for i, (dt, out, cols) in enumerate(MATS):
        w = GEN[dt](out, cols, seed + i)
        x = synth.normal(seed + 50 + i, cols)
        ws.append(w), xs.append(x)
        refs.append(oracle.matvec_q(oracle.Weight(dt, w, out, cols), x))
        offs.append(off)
        off += out
    return ws, xs, refs, offs, off


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("fused", [1, 0])
def test_sharded_matvec_every_rank_gets_every_row(ctx, world, fused):
    ws, xs, refs, offs, total = full_problem(300)
    shards = group(ctx, world, 2 * total)
    xd = [dev_f32(x) for x in xs]
    st = torch.cuda.Stream()
    ctx.debug_set("no_chain", 0 if fused else 1)
    try:
        for step, base in enumerate((0, total)):  # two steps into alternating halves of the gather buffer
            for s in shards:
                wts = [s.weight(dt, w, out, cols) for w, (dt, out, cols) in zip(ws, MATS)]
                ops = s.ops([dict(w=wt, x=x.data_ptr(), y_offset=base + o) for wt, x, o in zip(wts, xd, offs)])
                s.matvec_dev(ops, st.cuda_stream, backend.SHARD_NO_WAIT if world > 1 else 0)
                assert (ctx.last_plan()["grid"] == -3) == bool(fused)
            for s in shards:
                s.wait_dev(st.cuda_stream)
            st.synchronize()
            ctx.synchronize()
            for s in shards:
                got = s.read_y(base, total)
                for ref, o, (_, out, _) in zip(refs, offs, MATS):
                    assert synth.rel_err(got[o:o + out], ref) < TOL, (step, s.rank)
    finally:
        ctx.debug_set("no_chain", 0)
        for s in shards:
            s.free()


def test_sharded_matvec_caller_made_slices_and_mlx(ctx):
    """Slices the caller uploaded itself (``row0`` in the op) and an MLX 4-bit matrix, which has no fused
    epilogue and goes through the ordinary kernel plus the copy to the peers."""
    world, out, cols, gs = 2, 512, 1024, 64
    wq = synth.gen_q4k(out, cols, 411)
    wm, sm, bm = synth.gen_mlx4(out, cols, gs, 412)
    x = synth.normal(413, cols)
    ref_q = oracle.matvec_q(oracle.Weight(backend.Q4_K, wq, out, cols), x)
    ref_m = oracle.matvec_q(oracle.Weight(oracle.MLX_U32, wm, out, cols, synth.bf16_to_f32(sm), synth.bf16_to_f32(bm), gs), x)
    shards = group(ctx, world, 2 * out)
    xd = dev_f32(x)
    try:
        for s in shards:
            r0, n = s.row_range(out)
            rb = cols // 256 * 144
            own = backend.Weight(ctx, backend.Q4_K, wq.reshape(-1)[r0 * rb:(r0 + n) * rb], n, cols)
            mlx = s.weight(backend.MLX_U32, wm, out, cols, sm, bm, gs)
            s.matvec_dev(s.ops([dict(w=own, x=xd.data_ptr(), y_offset=0, row0=r0), dict(w=mlx, x=xd.data_ptr(), y_offset=out)]),
                         None, backend.SHARD_NO_WAIT)
        for s in shards:
            s.wait_dev()
        ctx.synchronize()
        for s in shards:
            got = s.read_y(0, 2 * out)
            assert synth.rel_err(got[:out], ref_q) < TOL and synth.rel_err(got[out:], ref_m) < TOL, s.rank
    finally:
        for s in shards:
            s.free()


@pytest.mark.parametrize("fused", [0, backend.SHARD_FUSED_STORES, backend.SHARD_SM_PUSH])
@pytest.mark.parametrize("dtype,out,cols,tokens", [(backend.Q4_K, 1024, 2048, 96), (backend.Q6_K, 512, 2048, 300), (backend.Q4_K, 256, 8192, 64)])
def test_sharded_matmul_tiles_land_in_every_rank(ctx, dtype, out, cols, tokens, fused):
    """Prefill form: each rank's [tokens, rows] block goes to its columns of [tokens, out] on every rank
    (bf16 tensor-core GEMM: the 2e-2 bar); the third case takes the split-K path.  The three ways of moving the
    block: copy engines on the group's own streams (default), stores from the GEMM's epilogue, a copy kernel."""
    world = 2
    w = GEN[dtype](out, cols, 520)
    xs = synth.f32_to_bf16(synth.normal(521, tokens * cols))
    xs = synth.bf16_to_f32(xs).reshape(tokens, cols)
    ref = oracle.matmul_q(oracle.Weight(dtype, w, out, cols), xs, tokens).reshape(tokens, out)
    shards = group(ctx, world, tokens * out + 64)
    xd = dev_f32(xs)
    try:
        for s in shards:
            wt = s.weight(dtype, w, out, cols)
            s.matmul_dev(wt, xd.data_ptr(), tokens, 64, 0, 0, None, backend.SHARD_NO_WAIT | fused)
            assert ctx.last_plan()["grid"] == -1, "the tensor-core GEMM did not run"
        for s in shards:
            s.wait_dev()
        ctx.synchronize()
        for s in shards:
            got = s.read_y(64, tokens * out).reshape(tokens, out)
            assert synth.rel_err(got, ref) < 2e-2, s.rank
    finally:
        for s in shards:
            s.free()


def test_a_silent_peer_ends_in_a_timeout_status_and_the_group_recovers(ctx):
    """Failure detection without a fault: rank 1 never runs its step, so rank 0's bounded wait on rank 1's step
    number runs out, the kernel returns, and the host sees ULLM_ERR_TIMEOUT.  After a reset both ranks run
    an ordinary step."""
    out, cols = 512, 1024
    w = synth.gen_q4k(out, cols, 611)
    x = synth.normal(612, cols)
    ref = oracle.matvec_q(oracle.Weight(backend.Q4_K, w, out, cols), x)
    shards = group(ctx, 2, out)
    xd = dev_f32(x)
    ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 50)
    try:
        w0 = shards[0].weight(backend.Q4_K, w, out, cols)
        shards[0].matvec_dev(shards[0].ops([dict(w=w0, x=xd.data_ptr(), y_offset=0)]), None, backend.SHARD_NO_WAIT)
        shards[0].wait_dev()
        with pytest.raises(backend.UllmError) as e:
            ctx.synchronize()
        assert e.value.code == backend.ERR_TIMEOUT
        for s in shards:
            s.reset()
        ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 2000)
        for s in shards:
            wt = s.weight(backend.Q4_K, w, out, cols)
            s.matvec_dev(s.ops([dict(w=wt, x=xd.data_ptr(), y_offset=0)]), None, backend.SHARD_NO_WAIT)
        for s in shards:
            s.wait_dev()
        ctx.synchronize()
        for s in shards:
            assert synth.rel_err(s.read_y(0, out), ref) < TOL
    finally:
        ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 2000)
        for s in shards:
            s.free()


def test_a_silent_peer_ends_the_tagged_exchange_in_a_timeout_too(ctx):
    """The same failure in a launch that waits itself: rank 0's kernel polls the {value, step} pairs rank 1 owes
    it, rank 1 never runs, the poll's time limit (50 ms) runs out in every polling thread, the kernel returns and
    the host sees ULLM_ERR_TIMEOUT.  After a reset (which also clears stale tags) the group works again."""
    out, cols = 512, 1024
    w = synth.gen_q4k(out, cols, 621)
    x = synth.normal(622, cols)
    ref = oracle.matvec_q(oracle.Weight(backend.Q4_K, w, out, cols), x)
    shards = group(ctx, 2, out)
    xd = dev_f32(x)
    ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 50)
    try:
        w0 = shards[0].weight(backend.Q4_K, w, out, cols)
        shards[0].matvec_dev(shards[0].ops([dict(w=w0, x=xd.data_ptr(), y_offset=0)]))  # waits inside the kernel
        assert ctx.last_plan()["grid"] == -3
        with pytest.raises(backend.UllmError) as e:
            ctx.synchronize()
        assert e.value.code == backend.ERR_TIMEOUT
        for s in shards:
            s.reset()
        ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 2000)
        for s in shards:
            wt = s.weight(backend.Q4_K, w, out, cols)
            s.matvec_dev(s.ops([dict(w=wt, x=xd.data_ptr(), y_offset=0)]), None, backend.SHARD_NO_WAIT)
        for s in shards:
            s.wait_dev()
        ctx.synchronize()
        for s in shards:
            assert synth.rel_err(s.read_y(0, out), ref) < TOL
    finally:
        ctx.set_option(backend.OPT_SHARD_TIMEOUT_MS, 2000)
        for s in shards:
            s.free()


def test_shard_argument_errors(ctx):
    with pytest.raises(backend.UllmError):
        backend.Shard(ctx, 9, 0, 16)  # more than 8 ranks
    s = backend.Shard(ctx, 2, 0, 64)
    w = backend.Weight(ctx, backend.Q4_K, synth.gen_q4k(64, 256, 1), 64, 256)
    x = dev_f32(synth.normal(2, 256))
    with pytest.raises(backend.UllmError):  # not connected yet
        s.matvec_dev(s.ops([dict(w=w, x=x.data_ptr(), y_offset=0)]))
    with pytest.raises(backend.FormatError):
        s.row_range(65)  # 65 rows over 2 ranks
    s.free()
    s1 = backend.Shard(ctx, 1, 0, 64)
    with pytest.raises(backend.FormatError):  # rows beyond the gather buffer
        s1.matvec_dev(s1.ops([dict(w=w, x=x.data_ptr(), y_offset=8)]))
    s1.free()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("tagged", [1, 0])
def test_two_devices_one_process(tagged):
    """A real two-GPU group inside one process (``ullm_cuda_shard_connect_local``): both ranks launch their
    step with the wait inside the kernel; the launches are asynchronous, so both kernels are in flight.
    Both exchanges: rows as {value, step} pairs that the receiving kernel polls and unpacks (the default of a
    waiting launch), and plain stores followed by published step numbers."""
    ws, xs, refs, offs, total = full_problem(700)
    ctxs = [backend.CudaContext(d) for d in range(2)]
    for c in ctxs:
        c.debug_set("shard_no_tagged", 0 if tagged else 1)
    shards = [backend.Shard(c, 2, r, 2 * total) for r, c in enumerate(ctxs)]
    backend.Shard.connect_local(shards)
    try:
        xd = [[torch.from_numpy(x).to(f"cuda:{d}") for x in xs] for d in range(2)]
        wts = [[s.weight(dt, w, out, cols) for w, (dt, out, cols) in zip(ws, MATS)] for s in shards]
        for step, base in enumerate((0, total, 0)):
            for r, s in enumerate(shards):
                s.matvec_dev(s.ops([dict(w=wt, x=x.data_ptr(), y_offset=base + o) for wt, x, o in zip(wts[r], xd[r], offs)]))
            for c in ctxs:
                c.synchronize()
            for s in shards:
                got = s.read_y(base, total)
                for ref, o, (_, out, _) in zip(refs, offs, MATS):
                    assert synth.rel_err(got[o:o + out], ref) < TOL, (step, s.rank)
    finally:
        for s in shards:
            s.free()
        for c in ctxs:
            c.close()
