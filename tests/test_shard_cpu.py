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


def _peer_worker(rank, world, port, out_q, silent_rank):
    """The exchange the library's kernels perform, with gloo messages standing in for stores over NVLink: every
    rank writes its rows into the same place of every rank's full-length result vectors (laid out by
    shard.vector_offsets, two regions used by alternate steps), then publishes its step number to every rank;
    a step is complete on a rank when it holds every rank's number.  Messages between two ranks arrive in order,
    like a rank's stores followed by its release store of the number."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        outs = [m[1] for m in MATS]
        offs = shard.vector_offsets(outs, align=16)
        total = offs[-1]
        buf = np.full(2 * total, np.nan, np.float32)  # this rank's gather buffer
        seen = [0] * world                            # this rank's control block: rank r's published step
        ok, timed_out = True, False
        for step in range(1, 4):
            base = shard.step_region(step, total)
            rows, pending = [], []
            if rank != silent_rank:
                for i, (dt, out, cols) in enumerate(MATS):
                    gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
                    mine = shard.slice_rows(dt, gen(out, cols, 100 + i), out, cols, world, rank)
                    x = synth.normal(200 + i + 10 * step, cols)
                    rows.append(oracle.matvec_q(oracle.Weight(dt, mine, out // world, cols), x))
                for peer in range(world):
                    payload = torch.from_numpy(np.concatenate(rows + [np.float32([step])]))
                    if peer == rank:
                        mine_payload = payload
                    else:
                        pending.append(dist.isend(payload, dst=peer))  # posted, not waited for: like a store
            for peer in range(world):
                n_rows = sum(o // world for o in outs)
                if peer == rank:
                    if rank == silent_rank:
                        continue
                    payload = mine_payload
                else:
                    payload = torch.empty(n_rows + 1)
                    try:
                        dist.recv(payload, src=peer)
                    except Exception:  # the bounded wait ran out: the peer never published
                        timed_out = True
                        break
                p, at = payload.numpy(), 0
                for i, o in enumerate(outs):
                    lo, hi = shard.row_range(o, world, peer)
                    buf[base + offs[i] + lo: base + offs[i] + hi] = p[at:at + hi - lo]
                    at += hi - lo
                seen[peer] = int(p[at])
            if timed_out:
                break
            for h in pending:
                h.wait()
            ok = ok and all(v >= step for v in seen)
            for i, (dt, out, cols) in enumerate(MATS):
                gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
                ref = oracle.matvec_q(oracle.Weight(dt, gen(out, cols, 100 + i), out, cols), synth.normal(200 + i + 10 * step, cols))
                ok = ok and np.array_equal(buf[base + offs[i]: base + offs[i] + out], ref)
        out_q.put((rank, ok, timed_out))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run_peers(silent_rank):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, q, silent_rank)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


def test_peer_store_exchange_fills_every_ranks_vectors_step_after_step():
    assert _run_peers(silent_rank=-1) == [(0, True, False), (1, True, False)]


def test_a_rank_that_never_publishes_ends_the_others_wait_with_a_timeout():
    """Failure detection, made on the host: rank 1 computes and sends nothing; rank 0's wait for rank 1's step
    number is bounded and reports the expiry instead of hanging."""
    res = dict((r, (ok, to)) for r, ok, to in _run_peers(silent_rank=1))
    assert res[0][1] is True  # rank 0 saw the time-out


def _tagged_worker(rank, world, port, out_q):
    """The tagged exchange of a waiting launch (``matvec_chain_kernel`` with ``ShardDev::tagged``), gloo messages
    standing in for 8-byte stores over NVLink: a rank's rows reach the others as {value, step} pairs in the half
    of the pair area that ``step`` selects; a rank polls the pairs it is owed for the step's tag and writes the
    values into its own vectors.  Rank 1 is made slow on purpose: before it takes the pairs of step s it has
    already been sent rank 0's pairs of step s + 1 (rank 0 only needed rank 1's rows of step s to go on), which
    land in the other half and must not disturb step s."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        outs = [m[1] for m in MATS]
        offs = shard.vector_offsets(outs, align=16)
        total = offs[-1]
        vec = np.full(total, np.nan, np.float32)       # this rank's result vectors
        pair_val = np.zeros(2 * total, np.float32)     # pair area: values ...
        pair_tag = np.zeros(2 * total, np.int64)       # ... and step tags (0: never written)
        peer, n_rows, last = 1 - rank, sum(o // world for o in outs), 4
        ok, early, applied, pending = True, 0, 0, []

        def apply_one_message():
            msg = torch.empty(n_rows + 1)
            dist.recv(msg, src=peer)
            m, at = msg.numpy(), 0
            step = int(m[-1])
            for i, o in enumerate(outs):
                lo, hi = shard.row_range(o, world, peer)
                for e in range(offs[i] + lo, offs[i] + hi):  # the peer's stores: its own rows, tagged
                    slot = shard.pair_slot(step, total, e)
                    pair_val[slot], pair_tag[slot] = m[at], step
                    at += 1
            return step

        for step in range(1, last + 1):
            rows = []
            for i, (dt, out, cols) in enumerate(MATS):
                gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
                mine = shard.slice_rows(dt, gen(out, cols, 100 + i), out, cols, world, rank)
                y = oracle.matvec_q(oracle.Weight(dt, mine, out // world, cols), synth.normal(200 + i + 10 * step, cols))
                lo, hi = shard.row_range(out, world, rank)
                vec[offs[i] + lo: offs[i] + hi] = y      # own rows: plain stores into the own vector
                rows.append(y)
            pending.append(dist.isend(torch.from_numpy(np.concatenate(rows + [np.float32([step])])), dst=peer))
            # what has arrived when this rank starts polling: the fast rank has exactly its peer's current step,
            # the slow rank has let the peer run ahead by one step
            want = step if rank == 0 else min(step + 1, last)
            while applied < want:
                early += apply_one_message() > step
                applied += 1
            for i, (dt, out, cols) in enumerate(MATS):
                for j in range(out - out // world):
                    e = shard.owed_element(j, offs[i], out, world, rank)
                    slot = shard.pair_slot(step, total, e)
                    ok = ok and pair_tag[slot] == step  # a real kernel polls here, bounded
                    vec[e] = pair_val[slot]
                gen = synth.gen_q4k if dt == oracle.Q4_K else synth.gen_q6k
                ref = oracle.matvec_q(oracle.Weight(dt, gen(out, cols, 100 + i), out, cols), synth.normal(200 + i + 10 * step, cols))
                ok = ok and np.array_equal(vec[offs[i]: offs[i] + out], ref)
        for h in pending:
            h.wait()
        out_q.put((rank, bool(ok), early))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_tagged_exchange_survives_a_rank_that_runs_one_step_ahead():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tagged_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert [(r, ok) for r, ok, _ in res] == [(0, True), (1, True)]
    assert res[1][2] == 3  # rank 1 held rank 0's next step before it took the current one, in three of four steps


def test_owed_elements_and_pair_slots():
    # rank 1 of 4 on a 16-row vector at offset 100 computes rows 4..7 and is owed the other twelve
    got = [shard.owed_element(j, 100, 16, 4, 1) for j in range(12)]
    assert got == [100, 101, 102, 103, 108, 109, 110, 111, 112, 113, 114, 115]
    with pytest.raises(ValueError):
        shard.owed_element(12, 100, 16, 4, 1)
    assert shard.pair_slot(6, 1000, 7) == 7 and shard.pair_slot(7, 1000, 7) == 1007


def test_library_row_split_agrees_with_the_index_math():
    import ctypes as C

    from ullm_b200 import backend

    lib = backend.load_library()
    for out, world in ((28672, 8), (8192, 4), (1024, 2), (7, 1)):
        for rank in range(world):
            r0, n = C.c_size_t(), C.c_size_t()
            assert lib.ullm_cuda_shard_row_range(out, world, rank, C.byref(r0), C.byref(n)) == 0
            assert (r0.value, r0.value + n.value) == shard.row_range(out, world, rank)
    r0, n = C.c_size_t(), C.c_size_t()
    assert lib.ullm_cuda_shard_row_range(10, 4, 0, C.byref(r0), C.byref(n)) == backend.ERR_FORMAT
    assert shard.vector_offsets([8192, 1024, 28672]) == [0, 8192, 9216, 37888]
    assert shard.vector_offsets([100, 7], align=64) == [0, 128, 192]
    assert shard.step_region(4, 1000) == 0 and shard.step_region(5, 1000) == 1000


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
