"""CPU tests of the multi-GPU host logic: world_size-2 gloo ranks shard matrices by
rows, compute their slice with the oracle (the stand-in for a GPU here), all-gather
the concatenated outputs and must reproduce the unsharded products."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from ullm_b200 import shard, synth

MATS = [(oracle.Q4_K, 64, 512), (oracle.Q6_K, 32, 1024), (oracle.Q4_K, 16, 256)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        outs = [m[1] for m in MATS]
        offs = shard.local_offsets(outs, world)
        y_cat = np.zeros(offs[-1], np.float32)
        for i, (dt, out, cols) in enumerate(MATS):
            gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
            full = gen(out, cols, 100 + i)  # every rank could hold the file; it keeps only its rows
            mine = shard.slice_rows(dt, full, out, cols, world, rank)
            x = synth.normal(200 + i, cols)
            y_cat[offs[i] : offs[i + 1]] = oracle.matvec_q(oracle.Weight(dt, mine, out // world, cols), x)
        gathered = [torch.empty(offs[-1]) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(y_cat))
        y_all = torch.cat(gathered).numpy()
        full_vecs = shard.split_gathered(y_all, outs, world)
        ok = True
        for i, (dt, out, cols) in enumerate(MATS):
            gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
            ref = oracle.matvec_q(oracle.Weight(dt, gen(out, cols, 100 + i), out, cols), synth.normal(200 + i, cols))
            ok = ok and np.array_equal(full_vecs[i], ref)  # same rows, same arithmetic: bit-identical
        out_q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_row_sharded_matvecs_gather_to_the_unsharded_result():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]


def test_shard_index_math():
    assert shard.row_range(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        shard.row_range(10, 4, 0)
    assert shard.row_bytes(12, 8192) == 4608 and shard.row_bytes(14, 28672) == 23520
    assert shard.local_offsets([8192, 1024, 28672], 8) == [0, 1024, 1152, 4736]
    w = np.arange(4 * 144, dtype=np.uint8)
    assert np.array_equal(shard.slice_rows(12, w, 4, 256, 2, 1), w[2 * 144 :])
    y_all = np.arange(2 * 5, dtype=np.float32)  # world 2, matrices of 4 and 6 rows
    a, b = shard.split_gathered(y_all, [4, 6], 2)
    assert a.tolist() == [0, 1, 5, 6] and b.tolist() == [2, 3, 4, 7, 8, 9]


def test_prefill_gather_layout_matches_the_unsharded_matmul():
    """Each rank's token-major [tokens, rows/N] products, concatenated per matrix and gathered
    as [rank][matrix][token][rows], must split back into the unsharded [tokens, out] products."""
    world, tokens = 2, 5
    outs, parts = [m[1] for m in MATS], [[] for _ in range(world)]
    refs = []
    for i, (dt, out, cols) in enumerate(MATS):
        gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
        full = gen(out, cols, 300 + i)
        xs = synth.normal(400 + i, tokens * cols)
        refs.append(oracle.matmul_q(oracle.Weight(dt, full, out, cols), xs, tokens))
        for r in range(world):
            mine = shard.slice_rows(dt, full, out, cols, world, r)
            parts[r].append(oracle.matmul_q(oracle.Weight(dt, mine, out // world, cols), xs, tokens).reshape(-1))
    y_all = np.concatenate([np.concatenate(p) for p in parts])
    for got, ref in zip(shard.split_gathered_tokens(y_all, outs, world, tokens), refs):
        assert np.array_equal(got, ref)
