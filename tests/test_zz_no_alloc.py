"""The allocation-free MoE entry point, ``ullm_cuda_moe_ffn_noalloc``.

Some users of this library cannot let it allocate: a serving process whose own
memory pool already owns the GPU, or a decode loop that must not meet the
device-wide synchronisation hidden in cudaMalloc.  For them the library keeps the
MoE kernels' scratch in a fixed 4 MiB array inside its own image and takes every
input and output as a device pointer.  The array is shared by all calls and is
not cleared between them, so this test makes two different calls in a row and
checks each against the regular entry point (``ullm_cuda_moe_ffn``) and against
the CPU oracle: stale routing tables or intermediates from the first call would
show up in the second.  It also reads the device's free memory before and after
the two calls: a call that allocated would lower it.
Collected last on purpose, so a failure here cannot hide another test's result.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from ullm_b200 import backend, synth

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the tolerance of the other matvec / MoE parity tests


def _experts(ne, hid, inter, gs, seed):
    g = synth.gen_mlx4(ne * inter, hid, gs, seed)
    u = synth.gen_mlx4(ne * inter, hid, gs, seed + 1)
    d = synth.gen_mlx4(ne * hid, inter, gs, seed + 2)
    return g, u, d


def _free_bytes():
    import torch

    torch.cuda.synchronize()
    return torch.cuda.mem_get_info(0)[0]


def _widen(t):
    return (t[0], synth.bf16_to_f32(t[1]), synth.bf16_to_f32(t[2]))


def test_noalloc_matches_regular_entry_point_twice(ctx):
    lib = backend.load_library()
    ne, hid, inter, gs, k = 16, 1024, 256, 64, 4
    g, u, d = _experts(ne, hid, inter, gs, 901)
    regular = backend.Experts(ctx, g, u, d, ne, hid, inter, gs)
    # the caller's own device memory: nine expert arrays, x, logits, y
    bufs = [ctx.upload(a) for t in (g, u, d) for a in t]
    inp = backend.MoeExpertsInput(*[b.ptr for b in bufs], backend.BF16, ne, hid, inter, gs)
    err = C.create_string_buffer(256)
    cpu = oracle.Experts(_widen(g), _widen(u), _widen(d), ne, hid, inter, gs)

    cases = []
    for ntok, seed in ((8, 11), (5, 12)):
        x = synth.normal(seed, ntok * hid).reshape(ntok, hid)
        lg = synth.router_logits(ntok, ne, k, seed + 100)
        cases.append((ntok, x, lg, regular.moe_ffn(x, lg, k), ctx.upload(x), ctx.upload(lg), ctx.alloc(ntok * hid * 4)))
    # a first call so that the one-time per-device set-up is behind us, then the two measured calls
    ntok, x, lg, want, bx, bl, by = cases[0]
    assert lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(inp), bx.ptr, bl.ptr, ntok, k, by.ptr, None, err, 256) == backend.OK, err.value
    free_before = _free_bytes()
    for call, (ntok, x, lg, want, bx, bl, by) in enumerate(cases):
        rc = lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(inp), bx.ptr, bl.ptr, ntok, k, by.ptr, None, err, 256)
        assert rc == backend.OK, (call, rc, err.value)
    assert _free_bytes() == free_before, "the allocation-free entry point changed the device's free memory"
    for call, (ntok, x, lg, want, bx, bl, by) in enumerate(cases):
        got = by.download().view(np.float32).reshape(ntok, hid)
        assert synth.rel_err(got, want) < TOL, call
        ref = np.stack([oracle.moe_ffn(cpu, lg[t], k, x[t]) for t in range(ntok)])
        assert synth.rel_err(got, ref) < TOL, call
        for b in (bx, bl, by):
            b.free()
    regular.free()


def test_noalloc_rejects_what_does_not_fit_or_is_malformed(ctx):
    lib = backend.load_library()
    err = C.create_string_buffer(256)
    g, u, d = _experts(2, 64, 64, 64, 5)
    bufs = [ctx.upload(a) for t in (g, u, d) for a in t]
    ptrs = [b.ptr for b in bufs]
    x, lg, y = ctx.alloc(64 * 4), ctx.alloc(2 * 4), ctx.alloc(64 * 4)
    # scratch beyond the built-in 4 MiB: 128 pairs * (16384 + 8192) floats
    big = backend.MoeExpertsInput(*ptrs, backend.BF16, 2, 16384, 8192, 64)
    rc = lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(big), x.ptr, lg.ptr, 1, 1, y.ptr, None, err, 256)
    assert rc == backend.ERR_FORMAT and b"scratch" in err.value
    ok = backend.MoeExpertsInput(*ptrs, backend.BF16, 2, 64, 64, 64)
    assert lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(ok), x.ptr, lg.ptr, 1, 3, y.ptr, None, err, 256) == backend.ERR_FORMAT  # k > experts
    assert lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(ok), None, lg.ptr, 1, 1, y.ptr, None, err, 256) == backend.ERR_INVALID
    assert lib.ullm_cuda_moe_ffn_noalloc(0, None, x.ptr, lg.ptr, 1, 1, y.ptr, None, None, 0) == backend.ERR_INVALID
    # x is read with 128-bit loads: a pointer that is not 16-byte aligned is refused on the host, nothing is launched
    rc = lib.ullm_cuda_moe_ffn_noalloc(0, C.byref(ok), x.ptr + 4, lg.ptr, 1, 1, y.ptr, None, err, 256)
    assert rc == backend.ERR_FORMAT and b"aligned" in err.value
