#!/usr/bin/env python
"""Benchmark of the quantized matvec hot path: achieved HBM GB/s of the dequant-in-kernel matvec,
with decode tokens/s and prefill TFLOP/s as secondary figures.

One JSON line on stdout.  A *step* is one pass of the hot path over one batch of synthetic input.
At every ``--gpus N`` the workload is ``c4_70b_layer_matvec``: the seven matrices of one
Llama-3-70B-shaped block (Q4_K q, k, v, o, gate, up; Q6_K down) as batch-1 matvecs, each with its own
seeded input vector — the largest configuration that fits one GPU and the one that shards.

* N = 1: resident weight objects, one persistent launch per step through
  ``ullm_cuda_weight_matvec_batch_dev`` (``--launch separate``: seven launches).
* N > 1 (one process per GPU under torchrun): output rows split evenly over the ranks
  (``ullm_cuda_shard_*``); each rank runs its slices as one persistent launch that stores its rows
  into every rank's memory over NVLink as {value, step} pairs and takes the pairs the other ranks
  owe it before it ends (no NCCL on the data path).  ``--exchange nccl`` runs the comparison arm instead:
  the same kernels followed by an ``ncclAllGather``.  torch.distributed only carries the set-up
  (handle exchange) and the max-over-ranks of the timings.

The K timed steps are captured in one CUDA graph, replayed ``--replays`` times with CUDA events
between the replays on the launching stream; ``ms_per_step`` is the median replay (max over ranks),
with the minimum and maximum beside it.  ``e2e`` goes through the host-buffer entry points
(``ullm_cuda_weight_matvec_batch`` / ``ullm_cuda_shard_matvec``) with pinned host vectors, copies
inside the timed region.  ``--impl reference`` times the CPU restatement of the reference's path
(OpenMP over rows) on the host cores for the same workload.  At N = 1 the line also carries a
``secondary`` object: the other benchmark configurations measured the same way.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from ullm_b200 import shard, synth  # noqa: E402

C1_UP = (14336, 4096)
C1_DOWN = (4096, 14336)
C1_BYTES_PER_LAUNCH = 48_168_960 + 16_384 + 57_344  # weights + x + y (either launch)

C4_MATS = [  # name, dtype, out, in   (one Llama-3-70B block)
    ("q", synth.Q4_K, 8192, 8192), ("k", synth.Q4_K, 1024, 8192), ("v", synth.Q4_K, 1024, 8192),
    ("o", synth.Q4_K, 8192, 8192), ("gate", synth.Q4_K, 28672, 8192), ("up", synth.Q4_K, 28672, 8192),
    ("down", synth.Q6_K, 8192, 28672),
]
METRIC = "quantized_matvec_hbm_gbs"
DTYPE = "u8 x s16 integer dot products (x as 16-bit fixed point per 32/64 values), f32 scale and accumulate"
# dram__bytes_read.sum + dram__bytes_write.sum of one step's kernels at N = 1, from an ncu capture of this
# workload (None until one has been taken)
NCU_TRAFFIC_PER_STEP = {"c4_70b_layer_matvec": 543_715_328 + 6_088_192}


def weight_bytes(dtype, out, cols):
    return out * (cols // 256) * (144 if dtype == synth.Q4_K else 210)


def c4_step_bytes():
    """Algorithmic bytes of one step: packed weights + 4 bytes per input and per output element."""
    return sum(weight_bytes(dt, o, c) + 4 * (o + c) for _, dt, o, c in C4_MATS)


def measured_peak_tflops():
    """Dense bf16 cuBLAS burst throughput measured on this pool (else the earlier measurement)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.idx)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])), mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU restatement (oracle port) legs
# ---------------------------------------------------------------------------
def cpu_c1_step_factory(frac: float = 1.0):
    """CPU step on the first ``frac`` of the rows of each matrix (bounded sample)."""
    import oracle

    ru, rd = max(8, int(C1_UP[0] * frac)), max(8, int(C1_DOWN[0] * frac))
    up = oracle.Weight(oracle.Q6_K, synth.gen_q6k(ru, C1_UP[1], synth.seed_for(1, 0)), ru, C1_UP[1])
    down = oracle.Weight(oracle.Q6_K, synth.gen_q6k(rd, C1_DOWN[1], synth.seed_for(1, 1)), rd, C1_DOWN[1])
    x = synth.normal(synth.seed_for(1, 2), C1_UP[1])
    h_full = np.zeros(C1_DOWN[1], np.float32)

    def step():
        h_full[:ru] = oracle.matvec_q(up, x)
        return oracle.matvec_q(down, h_full)

    nbytes = weight_bytes(synth.Q6_K, ru, C1_UP[1]) + weight_bytes(synth.Q6_K, rd, C1_DOWN[1]) + 4 * (ru + rd + sum(C1_UP[1:]) + C1_DOWN[1])
    return step, oracle.max_threads(), nbytes, f"rows 0..{ru} of up and 0..{rd} of down"


def cpu_c4_step_factory(frac: float = 1.0):
    import oracle

    ws, xs, nbytes = [], [], 0
    for i, (name, dt, out, cols) in enumerate(C4_MATS):
        r = max(8, int(out * frac))
        ws.append(oracle.Weight(dt, synth.gen_weight(dt, r, cols, synth.seed_for(4, i)), r, cols))
        xs.append(synth.normal(synth.seed_for(4, 8 + i), cols))
        nbytes += weight_bytes(dt, r, cols) + 4 * (r + cols)

    def step():
        return [oracle.matvec_q(w, x) for w, x in zip(ws, xs)]

    return step, oracle.max_threads(), nbytes, f"first {frac:.3f} of the rows of each of the 7 matrices"


def _lift_omp_limit():
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are the reference's path with every host
    # thread it can use, so the setting is lifted before the oracle library (and its OpenMP runtime) is loaded
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)


def run_reference(args):
    """The reference's CPU path (oracle port) on the host cores, same workload and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    _lift_omp_limit()
    # Size the per-step sample so that warmup + steps end within ~2 minutes.
    probe, cores, pbytes, _ = cpu_c4_step_factory(1.0 / 32)
    probe()
    t0 = time.perf_counter()
    probe()
    t_probe = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)
    frac = min(1.0, (1.0 / 32) * budget / max(t_probe, 1e-6))
    step, cores, nbytes, sample = cpu_c4_step_factory(frac)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    gbs = args.steps * nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c4_70b_layer_matvec", "note": "C restatement of ullm-model's CPU path (rayon -> OpenMP over rows); the Rust reference cannot be built here"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": f"{args.steps} steps, each over {sample}"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------
# CUDA arm
# ---------------------------------------------------------------------------
EAGER = False  # --eager: launch the timed steps from the host instead of replaying a graph (for profilers)


def time_graph(torch, step, steps, warmup, replays, before_timing=None):
    """``step(i, stream)`` enqueues step i.  The ``steps`` timed steps are captured in one CUDA graph on a
    non-default stream and replayed ``replays`` times back to back with an event between replays; returns the
    per-replay times in ms.  (A NULL stream handle would mean "the context's own stream" to the library, so the
    default stream is never used.)"""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(warmup):
            step(i, side.cuda_stream)
    side.synchronize()
    if EAGER:
        class _Eager:
            def replay(self):
                for i in range(steps):
                    step(warmup + i, side.cuda_stream)
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(steps):
                step(warmup + i, side.cuda_stream)
    with torch.cuda.stream(side):
        graph.replay()  # one untimed replay
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    if before_timing:
        before_timing()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        evs[0].record()
        for r in range(replays):
            graph.replay()
            evs[r + 1].record()
    torch.cuda.synchronize()
    return [evs[r].elapsed_time(evs[r + 1]) for r in range(replays)]


def spread(ms_list, steps):
    per = sorted(m / steps for m in ms_list)
    return {"median": statistics.median(per), "min": per[0], "max": per[-1], "replays": len(per)}


def oracle_rows(dt, w, cols, r0, n, x):
    """The oracle's product for rows [r0, r0 + n) of a row-major quantized matrix."""
    import oracle

    rb = cols // 256 * (144 if dt == synth.Q4_K else 210)
    blk = np.ascontiguousarray(np.asarray(w).reshape(-1).view(np.uint8)[r0 * rb:(r0 + n) * rb])
    return oracle.matvec_q(oracle.Weight(dt, blk, n, cols), x)


# ---- secondary workloads (N = 1): the other benchmark configurations, GPU legs only ----
def sec_c1(torch, backend, ctx, dev, args, peak):
    w_up_h = synth.gen_q6k(*C1_UP, synth.seed_for(1, 0))
    w_dn_h = synth.gen_q6k(*C1_DOWN, synth.seed_for(1, 1))
    x_h = synth.normal(synth.seed_for(1, 2), C1_UP[1])
    n = 4  # 4 x 96 MB walked round-robin: larger than L2
    ups = [backend.Weight(ctx, backend.Q6_K, w_up_h, *C1_UP) for _ in range(n)]
    dns = [backend.Weight(ctx, backend.Q6_K, w_dn_h, *C1_DOWN) for _ in range(n)]
    x = torch.from_numpy(x_h).to(dev)
    h = torch.empty(C1_UP[0], dtype=torch.float32, device=dev)
    y = torch.empty(C1_DOWN[0], dtype=torch.float32, device=dev)

    def step(i, st):
        ups[i % n].matvec_dev(x.data_ptr(), h.data_ptr(), st)
        dns[i % n].matvec_dev(h.data_ptr(), y.data_ptr(), st)

    sp = spread(time_graph(torch, step, args.steps, args.warmup, args.replays), args.steps)
    ref_h = oracle_rows(synth.Q6_K, w_up_h, C1_UP[1], 0, C1_UP[0], x_h)
    ref = oracle_rows(synth.Q6_K, w_dn_h, C1_DOWN[1], 0, 256, ref_h)
    err = synth.rel_err(y.cpu().numpy()[:256], ref)
    out = {"workload": "c1_q6k_ffn_pair", "us_per_launch": sp["median"] * 1e3 / 2, "gbs": 2 * C1_BYTES_PER_LAUNCH / (sp["median"] * 1e-3) / 1e9,
           "ms_per_step": sp, "rel_err_vs_cpu": err}
    out["frac"] = out["gbs"] / peak
    for w in ups + dns:
        w.free()
    return out


def sec_c0(torch, backend, ctx, dev, args, peak):
    shape = (4096, 4096)
    w = synth.gen_q4k(*shape, synth.seed_for(0, 0))
    x_h = synth.normal(synth.seed_for(0, 1), shape[1])
    n = 40  # 9.4 MB each: 377 MB walked round-robin
    ws = [backend.Weight(ctx, backend.Q4_K, w, *shape) for _ in range(n)]
    x = torch.from_numpy(x_h).to(dev)
    y = torch.empty(shape[0], dtype=torch.float32, device=dev)
    sp = spread(time_graph(torch, lambda i, st: ws[i % n].matvec_dev(x.data_ptr(), y.data_ptr(), st), args.steps, args.warmup, args.replays), args.steps)
    nbytes = weight_bytes(synth.Q4_K, *shape) + 4 * sum(shape)
    err = synth.rel_err(y.cpu().numpy()[:256], oracle_rows(synth.Q4_K, w, shape[1], 0, 256, x_h))
    out = {"workload": "c0_q4k_4096", "us_per_launch": sp["median"] * 1e3, "gbs": nbytes / (sp["median"] * 1e-3) / 1e9, "ms_per_step": sp, "rel_err_vs_cpu": err}
    out["frac"] = out["gbs"] / peak
    for w_ in ws:
        w_.free()
    return out


def sec_c2(torch, backend, ctx, dev, args, peak):
    ne, hid, inter, gs, ntok, k = 128, 2048, 768, 64, 8, 8
    g = synth.gen_mlx4(ne * inter, hid, gs, synth.seed_for(2, 0))
    u = synth.gen_mlx4(ne * inter, hid, gs, synth.seed_for(2, 1))
    d = synth.gen_mlx4(ne * hid, inter, gs, synth.seed_for(2, 2))
    exs = [backend.Experts(ctx, g, u, d, ne, hid, inter, gs) for _ in range(2)]  # 2 x 340 MB
    x = torch.from_numpy(synth.normal(synth.seed_for(2, 4), ntok * hid)).to(dev)
    lgs, dist = [], []
    for j in range(4):
        lg = synth.router_logits(ntok, ne, k, synth.seed_for(2, 5) + 977 * j)
        dist.append(len(np.unique(np.argsort(-lg, axis=1)[:, :k])))
        lgs.append(torch.from_numpy(lg).to(dev))
    y = torch.empty(ntok * hid, dtype=torch.float32, device=dev)
    sp = spread(time_graph(torch, lambda i, st: exs[i % 2].moe_ffn_dev(x.data_ptr(), lgs[i % 4].data_ptr(), ntok, k, y.data_ptr(), stream=st),
                           args.steps, args.warmup, args.replays), args.steps)
    D = sum(dist) / len(dist)
    nbytes = D * 2_654_208 + 131_072
    out = {"workload": "c2_moe_mlx4", "us_per_step": sp["median"] * 1e3, "distinct_experts": D, "gbs": nbytes / (sp["median"] * 1e-3) / 1e9,
           "ms_per_step": sp}
    out["frac"] = out["gbs"] / peak
    for e in exs:
        e.free()
    return out


def sec_c3(torch, backend, ctx, dev, args, peak):
    """Llama-3.2-1B-shaped decode: 16 prompt tokens one by one, then 128 greedy tokens kept on the device; the
    tokens are compared with the oracle's, stored beside the tests."""
    import oracle  # embedding rows of the prompt: host-side lookup, as the reference does (lib.rs:692-710)

    p = dict(synth.LLAMA_1B)
    m = synth.gen_llama_model(p, synth.seed_for(3, 0))
    kk, vv = synth.gen_kv_prefill(p, 1024, synth.seed_for(3, 1))
    gf = backend.GpuForward(ctx, m, kv_f16=True)
    gf.set_kv(0, kk, vv)
    embd = ctx.upload(m["tok_embd"][1])
    prompt = synth.rand_ints(synth.seed_for(3, 2), 16, 0, p["vocab"] - 1)
    rb = p["n_embd"] // 256 * 144
    tab = np.asarray(m["tok_embd"][1]).reshape(-1).view(np.uint8)
    for i, t in enumerate(prompt):
        row = oracle.dequantize(m["tok_embd"][0], tab[int(t) * rb:(int(t) + 1) * rb], p["n_embd"])
        lg = gf.forward(row, 1024 + i)
    tok = int(np.argmax(lg))
    n_gen = 128
    gf.greedy(embd, m["tok_embd"][0], tok, 1040, 8)  # warm the greedy graph
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        toks = gf.greedy(embd, m["tok_embd"][0], tok, 1040, n_gen)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    wbytes = 16 * 38_805_504 + 215_470_080
    kvbytes = 32_768 * (1040 + 64)
    out = {"workload": "c3_llama1b_decode", "tok_per_s": n_gen / dt, "us_per_token": dt / n_gen * 1e6, "tokens": n_gen,
           "gbs": (wbytes + kvbytes + 513_024) * n_gen / dt / 1e9, "runs_s": times,
           "note": "one blocking call generates the 128 tokens on the device (argmax feeds the next embedding lookup); host wall clock"}
    out["frac"] = out["gbs"] / peak
    gold = os.path.join(ROOT, "tests", "golden", "c3_decode_128.npz")
    if os.path.exists(gold):
        g = np.load(gold)
        same = int(np.sum(np.cumprod(toks == g["tokens"])))
        out["check"] = {"first_token_matches": bool(tok == int(g["first"])), "leading_tokens_equal_to_oracle": same, "of": n_gen}
    gf.free()
    return out


def aux_c2decode(torch, backend, ctx, dev, args, peak):
    out = {"workload": "c2decode"}
    if True:
        # Decode step of the Qwen3-30B-A3B shape (MLX 4-bit, 128 experts, 8 per token): the model the reference
        # quotes its MoE decode rate on.  One seeded layer's weights are uploaded once per layer (separate device
        # copies, so every layer streams its own bytes from HBM); tokens are produced by the on-device greedy loop.
        p = dict(synth.QWEN3MOE_30B)
        p["n_layer"] = args.layers or p["n_layer"]
        one = synth.gen_qwen3moe_model(dict(p, n_layer=1), synth.seed_for(2, 8))
        m = dict(one, params=p, layers=[one["layers"][0]] * p["n_layer"])
        gf = backend.GpuForward(ctx, m, kv_f16=True, rope_neox=1, qk_norm=1)
        t = m["tok_embd"]
        embd = backend.Weight(ctx, t[0], t[1], t[2], t[3], t[4], t[5], t[6])
        n_gen = args.steps if args.steps > 20 else 128
        gf.greedy_weight(embd, 11, 0, min(8, n_gen))  # warm the greedy graph
        t0 = time.perf_counter()
        toks = gf.greedy_weight(embd, 11, 0, n_gen)
        dt = time.perf_counter() - t0
        e, hd, g = p["n_embd"], p["head_dim"], p["group"]
        qd, kvd, ne, k, mi = p["n_head"] * hd, p["n_kv_head"] * hd, p["n_experts"], p["n_experts_used"], p["moe_inter"]
        mlx = lambda o, c: o * c // 2 + 2 * 2 * o * (c // g)  # packed words + bf16 scale and bias tables
        layer = mlx(qd, e) + 2 * mlx(kvd, e) + mlx(e, qd) + mlx(ne, e) + k * (2 * mlx(mi, e) + mlx(e, mi))
        nbytes = p["n_layer"] * layer + mlx(p["vocab"], e) + 2 * 2 * kvd * p["n_layer"] * (n_gen // 2)
        out.update(tok_per_s=n_gen / dt, us_per_token=dt / n_gen * 1e6, tokens=n_gen, layers=p["n_layer"], bytes_per_token=nbytes,
                   gbs=nbytes * n_gen / dt / 1e9, first_tokens=toks[:8].tolist(),
                   note="weights of one seeded layer repeated per layer (distinct device copies); greedy loop on the device")
    return out


def aux_c3prefill(torch, backend, ctx, dev, args, peak):
    out = {"workload": "c3prefill"}
    if True:
        # time to first token on the Llama-3.2-1B shape: all prompt tokens in one batched pass
        # (tensor-core GEMMs on the quantized weights), against the same prompt token by token
        p = dict(synth.LLAMA_1B)
        m = synth.gen_llama_model(p, synth.seed_for(3, 0))
        gf = backend.GpuForward(ctx, m, kv_f16=True)
        S = args.tokens
        emb = synth.normal(synth.seed_for(3, 5), S * p["n_embd"]).reshape(S, p["n_embd"]) * np.float32(0.02)
        gf.forward_batch(emb, S)  # allocates the chunk buffers
        reps = max(3, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(reps):
            lg = gf.forward_batch(emb, S)
        dt = (time.perf_counter() - t0) / reps
        n_seq = min(S, 32)
        t0 = time.perf_counter()
        for i in range(n_seq):
            gf.forward(emb[i], i)
        dt_seq = (time.perf_counter() - t0) / n_seq
        params = 16 * (2560 * 2048 + 512 * 2048 + 2048 * 2048 + 2 * 8192 * 2048 + 2048 * 8192)
        flop = 2.0 * S * params
        out.update(tokens=S, ms_prefill=dt * 1e3, prefill_tok_per_s=S / dt, gemm_tflops=flop / dt / 1e12,
                   ms_per_token_stepwise=dt_seq * 1e3, speedup_vs_stepwise=dt_seq * S / dt, last_logit_argmax=int(np.argmax(lg)),
                   note="host embeddings in, last-token logits out; projections as bf16 tensor-core GEMMs, attention f32")
    return out


def run_aux(args):
    """Single-GPU runs of one of the other configurations on its own (the figures the N = 1 line carries in
    `secondary`, plus the Qwen3-MoE decode step and the batched prefill), for profiling one workload at a time."""
    import torch

    from ullm_b200 import backend

    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    ctx = backend.CudaContext(0)
    ctx.set_option(backend.OPT_PDL, 1 if args.pdl else 0)
    for kv in args.knob:
        ctx.debug_set(kv.split("=")[0], int(kv.split("=")[1]))
    peak, _ = measured_peak_gbs()
    if args.workload == "c4gemm":
        mats = [m for m in c4_weights(backend, ctx) if not args.only or m["name"] == args.only]
        out = sec_c4gemm(torch, backend, ctx, dev, args, mats)
    elif args.workload == "readprobe":
        out = read_only_ceiling(ctx, c4_step_bytes())
    else:
        fn = {"c0": sec_c0, "c1": sec_c1, "c2": sec_c2, "c3": sec_c3, "c2decode": aux_c2decode, "c3prefill": aux_c3prefill}[args.workload]
        out = fn(torch, backend, ctx, dev, args, peak)
    if "gbs" in out:
        out["frac_of_measured_peak"] = out["gbs"] / peak
    print(json.dumps(out), flush=True)
    return 0


def c4_weights(backend, ctx):
    mats = []
    for i, (name, dt, o, c) in enumerate(C4_MATS):
        w = synth.gen_weight(dt, o, c, synth.seed_for(4, i))
        mats.append(dict(name=name, dt=dt, out=o, cols=c, host=w, w=backend.Weight(ctx, dt, w, o, c), xh=synth.normal(synth.seed_for(4, 8 + i), c)))
    return mats


def sec_c4gemm(torch, backend, ctx, dev, args, mats):
    """The block as a 512-token prefill GEMM (tcgen05 path) on the weights already resident."""
    S = args.tokens
    tf_peak = measured_peak_tflops()
    per, total_ms, total_flop, worst = {}, 0.0, 0.0, 0.0
    for i, m in enumerate(mats):
        o, c = m["out"], m["cols"]
        xs = torch.randn(S * c, dtype=torch.float32, device=dev, generator=torch.Generator(device=dev).manual_seed(40 + i))
        xs = xs.to(torch.bfloat16).to(torch.float32)  # bf16-representable activations, as the configuration states
        ys = torch.empty(S * o, dtype=torch.float32, device=dev)
        sp = spread(time_graph(torch, lambda _i, st: m["w"].matmul_dev(xs.data_ptr(), ys.data_ptr(), S, st), max(4, args.steps // 4), 3, args.replays),
                    max(4, args.steps // 4))
        assert ctx.last_plan()["grid"] == -1, "tensor-core GEMM did not run"
        flop = 2.0 * S * o * c
        per[m["name"]] = {"us": round(sp["median"] * 1e3, 2), "tflops": round(flop / sp["median"] / 1e9, 1)}
        total_ms += sp["median"]
        total_flop += flop
        # 64 rows of the result against the oracle's f32 product of the same inputs (the 2e-2 bf16 bar)
        import oracle
        r0 = (o // 2) // 64 * 64
        rb = c // 256 * (144 if m["dt"] == synth.Q4_K else 210)
        blk = np.ascontiguousarray(np.asarray(m["host"]).reshape(-1).view(np.uint8)[r0 * rb:(r0 + 64) * rb])
        xs_h = xs[:8 * c].cpu().numpy().reshape(8, c)
        ref = oracle.matmul_q(oracle.Weight(m["dt"], blk, 64, c), xs_h, 8).reshape(8, 64)
        got = ys.view(S, o)[:8, r0:r0 + 64].cpu().numpy()
        worst = max(worst, synth.rel_err(got, ref))
        del xs, ys
    return {"workload": "c4_70b_layer_gemm", "tokens": S, "us_per_step": total_ms * 1e3, "tflops": total_flop / total_ms / 1e9, "peak_tflops": tf_peak,
            "frac": total_flop / total_ms / 1e9 / tf_peak, "per_matrix": per, "rel_err_vs_cpu_64_rows_8_tokens": worst,
            "note": "includes the f32->bf16 activation cast kernel of every call; frac of the measured cuBLAS bf16 burst"}


def run_c4(args):
    """The headline arm at every N."""
    import torch

    from ullm_b200 import backend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    ctx = backend.CudaContext(local)
    ctx.set_option(backend.OPT_PDL, 1 if args.pdl else 0)
    for kv in args.knob:
        ctx.debug_set(kv.split("=")[0], int(kv.split("=")[1]))
    peak, peak_kind = measured_peak_gbs()
    total_bytes = c4_step_bytes()

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(vals):
        if dist is None:
            return list(vals)
        t = torch.tensor(list(vals), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    check = {}
    secondary = None
    if world == 1:
        mats = c4_weights(backend, ctx)
        for m in mats:
            m["x"] = torch.from_numpy(m["xh"]).to(dev)
            m["y"] = torch.empty(m["out"], dtype=torch.float32, device=dev)
        batch = backend.WeightBatch(ctx, [m["w"] for m in mats], [m["x"].data_ptr() for m in mats], [m["y"].data_ptr() for m in mats])

        def step(_i, st):
            if args.launch == "separate":
                for m in mats:
                    m["w"].matvec_dev(m["x"].data_ptr(), m["y"].data_ptr(), st)
            else:
                batch.launch(st)  # one persistent launch: the CTAs are dealt out to the seven matrices

        sampler = ClockSampler(local)
        sampler.start()
        time.sleep(0.2)
        ms = time_graph(torch, step, args.steps, args.warmup, args.replays)
        ctx.synchronize()  # surfaces a device-side time-out status
        launches_per_step = 1 if ctx.last_plan()["grid"] == -2 else len(mats)
        # end to end: pinned host vectors through the blocking batch call
        xs_p = [torch.from_numpy(m["xh"]).pin_memory().numpy() for m in mats]
        ys_p = [torch.empty(m["out"], dtype=torch.float32).pin_memory().numpy() for m in mats]
        hb = backend.HostBatch(ctx, [m["w"] for m in mats], xs_p, ys_p)
        for _ in range(max(3, args.warmup)):
            hb.run()
        n_e2e = max(args.steps, 20)
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            hb.run()
        e2e_s = (time.perf_counter() - t0) / n_e2e
        clocks = sampler.stop()
        # parity of what was timed: 64 rows per matrix (the last ones: the ragged end of the row walk) against the oracle
        worst = 0.0
        for m, yp in zip(mats, ys_p):
            r0 = m["out"] - 64
            ref = oracle_rows(m["dt"], m["host"], m["cols"], r0, 64, m["xh"])
            worst = max(worst, synth.rel_err(m["y"].cpu().numpy()[r0:], ref), synth.rel_err(yp[r0:], ref))
        check["rel_err_vs_cpu_64_rows_per_matrix"] = worst
        e2e_api = "ullm_cuda_weight_matvec_batch (7 resident weights, pinned host x / y, one blocking call per step)"
        h2d, d2h = 4 * sum(m["cols"] for m in mats), 4 * sum(m["out"] for m in mats)
        l2 = "every step streams 542 MB of weights once: inputs larger than L2"
        launch = "one CUDA graph of the K timed steps, replayed; seven launches per step" if launches_per_step > 1 else "one CUDA graph of the K timed steps, replayed; one persistent launch per step"
        kernel = "matvec_stream_kernel<Q4_K | Q6_K prepared>" if launches_per_step > 1 else "matvec_chain_kernel"
        parallelism = "single GPU"
        cpu = None
        if not args.no_cpu:
            cpu = cpu_leg(check, [m["y"].cpu().numpy() for m in mats])
        fp32_path = read_ceiling = None
        if not args.no_secondary:
            secondary = {}
            for name, fn in (("c4gemm", lambda: sec_c4gemm(torch, backend, ctx, dev, args, mats)),):
                secondary[name] = fn()
            # The same step through the plain fp32-FMA kernel (one warp per row, f32 x, no fixed-point image): what the
            # integer formulation buys.  Test knobs select it (raw Q6_K rows, generic kernel); nothing timed above uses them.
            ctx.debug_set("no_prepare", 1)
            plain = [backend.Weight(ctx, m["dt"], m["host"], m["out"], m["cols"]) for m in mats]
            ctx.debug_set("no_prepare", 0)
            ctx.debug_set("force_generic", 1)

            def fstep(_i, st):
                for w_, m in zip(plain, mats):
                    w_.matvec_dev(m["x"].data_ptr(), m["y"].data_ptr(), st)

            fsp = spread(time_graph(torch, fstep, 4, 3, 3), 4)
            ctx.debug_set("force_generic", 0)
            ferr = max(synth.rel_err(m["y"].cpu().numpy()[m["out"] - 64:], oracle_rows(m["dt"], m["host"], m["cols"], m["out"] - 64, 64, m["xh"])) for m in mats)
            fp32_path = {"gbs": total_bytes / (fsp["median"] * 1e-3) / 1e9, "us_per_step": fsp["median"] * 1e3, "rel_err_vs_cpu": ferr}
            for w_ in plain:
                w_.free()
            for m in mats:
                m["w"].free()
            torch.cuda.empty_cache()
            read_ceiling = read_only_ceiling(ctx, total_bytes)
            for name, fn in (("c1", sec_c1), ("c0", sec_c0), ("c2", sec_c2), ("c3", sec_c3)):
                secondary[name] = fn(torch, backend, ctx, dev, args, peak)
    else:
        # ---- N > 1: rows / N of every matrix per rank ----
        outs = [o for _, _, o, _ in C4_MATS]
        offs = shard.vector_offsets(outs)  # where each full-length result starts in the gather buffer
        total = offs[-1]
        slice_bytes = sum(weight_bytes(dt, o // world, c) for _, dt, o, c in C4_MATS)
        ncopies = max(1, -(-400_000_000 // slice_bytes))  # distinct device copies walked round-robin: more than L2
        sh = backend.Shard(ctx, world, rank, 2 * total)  # two regions, used by alternate steps
        handles = [None] * world
        dist.all_gather_object(handles, sh.export())
        sh.connect(handles)
        mats = []
        for i, (name, dt, out, cols) in enumerate(C4_MATS):
            r0, rows = sh.row_range(out)
            w = synth.gen_weight(dt, rows, cols, synth.seed_for(4, i) + 0x100000 * (rank + 1))  # each rank generates only its rows
            xv = synth.normal(synth.seed_for(4, 8 + i), cols)
            mats.append(dict(name=name, dt=dt, out=out, cols=cols, row0=r0, rows=rows, host=w, xh=xv, x=torch.from_numpy(xv).to(dev),
                             ws=[backend.Weight(ctx, dt, w, rows, cols) for _ in range(ncopies)]))
        ops = [[sh.ops([dict(w=m["ws"][c], x=m["x"].data_ptr(), y_offset=par * total + o, row0=m["row0"]) for m, o in zip(mats, offs)])
                for par in range(2)] for c in range(ncopies)]
        launches_per_step = 1
        if args.exchange == "nccl":
            ident = [sh.nccl_id() if rank == 0 else None]
            dist.broadcast_object_list(ident, src=0)
            sh.nccl_init(ident[0])
            rows_total = sum(m["rows"] for m in mats)
            y_cat = torch.empty(rows_total, dtype=torch.float32, device=dev)
            y_all = torch.empty(world * rows_total, dtype=torch.float32, device=dev)
            loff = shard.local_offsets(outs, world)
            batches = [backend.WeightBatch(ctx, [m["ws"][c] for m in mats], [m["x"].data_ptr() for m in mats],
                                           [y_cat.data_ptr() + 4 * o for o in loff[:-1]]) for c in range(ncopies)]
            launches_per_step = 2

        def step(i, st):
            if args.exchange == "nccl":
                batches[i % ncopies].launch(st)
                sh.allgather_nccl_dev(y_cat.data_ptr(), y_all.data_ptr(), rows_total, st)
            else:
                sh.matvec_dev(ops[i % ncopies][i & 1], st)

        barrier()  # every rank is connected before any rank runs a step
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
            time.sleep(0.2)
        if args.exchange == "nccl":  # comparison arm: host launches, as NCCL is not captured here
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for i in range(max(args.warmup, 3)):
                    step(i, side.cuda_stream)
            torch.cuda.synchronize()
            barrier()
            ms = []
            for r in range(args.replays):
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(side):
                    ev0.record()
                    for i in range(args.steps):
                        step(args.warmup + i, side.cuda_stream)
                    ev1.record()
                torch.cuda.synchronize()
                ms.append(ev0.elapsed_time(ev1))
            sh.nccl_check()
        else:
            ms = time_graph(torch, step, args.steps, args.warmup, args.replays, before_timing=barrier)
        ctx.synchronize()
        ms = max_over_ranks(ms)
        barrier()
        # end to end: pinned host x in, the gathered vectors back to pinned host memory, one blocking call per step
        xs_p = [torch.from_numpy(m["xh"]).pin_memory().numpy() for m in mats]
        y_p = torch.empty(total, dtype=torch.float32).pin_memory().numpy()
        e2e_api = "ullm_cuda_shard_matvec (pinned host x -> this rank's row slices -> rows to all ranks as tagged pairs -> pinned host y of all 7 full vectors)"
        if args.exchange == "nccl":
            e2e_s = float("nan")
        else:
            for i in range(4):
                sh.matvec_host(ops[i % ncopies][i & 1], xs_p, y_p, (i & 1) * total)
            barrier()
            n_e2e = max(args.steps, 20) // 2 * 2
            t0 = time.perf_counter()
            for i in range(n_e2e):
                sh.matvec_host(ops[i % ncopies][i & 1], xs_p, y_p, (i & 1) * total)
            e2e_s = max_over_ranks([(time.perf_counter() - t0) / n_e2e])[0]
        clocks = sampler.stop() if rank == 0 else None
        # parity on every rank's copy: each rank computes 64 rows of its own slice of every matrix with the oracle,
        # the values travel to all ranks, and every rank compares them with what lies in ITS gather buffer at those rows
        _lift_omp_limit()
        mine = []
        for m in mats:
            l0 = max(0, m["rows"] - 64)
            mine.append((m["row0"] + l0, oracle_rows(m["dt"], m["host"], m["cols"], l0, m["rows"] - l0, m["xh"])))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        if args.exchange == "nccl":
            got_all = shard.split_gathered(y_all.cpu().numpy(), outs, world)
        else:
            last = (args.warmup + args.steps - 1) & 1 if n_e2e == 0 else (n_e2e - 1) & 1
            got = sh.read_y(last * total, total)
            got_all = [got[o:o + n] for o, n in zip(offs, outs)]
        worst = 0.0
        for r in range(world):
            for i, (g0, ref) in enumerate(everyone[r]):
                worst = max(worst, synth.rel_err(got_all[i][g0:g0 + len(ref)], ref))
        check["rel_err_vs_cpu_64_rows_per_matrix_per_rank"] = max_over_ranks([worst])[0]
        h2d, d2h = 4 * sum(m["cols"] for m in mats), 4 * total
        l2 = f"{ncopies} distinct copies of the per-rank slice set ({slice_bytes // 1000000} MB each) walked round-robin: inputs larger than L2"
        if args.exchange == "nccl":
            launch, kernel = "host launches: one persistent launch + ncclAllGather per step (comparison arm)", "matvec_chain_kernel + ncclAllGather"
            parallelism = f"rows/{world} per matrix; NCCL all-gather of the ranks' output rows"
        else:
            launch, kernel = "one CUDA graph of the K timed steps, replayed; one persistent launch per step", "matvec_chain_kernel (rows to all ranks as {value, step} pairs)"
            parallelism = f"rows/{world} per matrix; every rank's kernel stores its rows into all ranks' memory over NVLink as tagged pairs and takes the pairs it is owed: no all-gather"
        cpu = None  # the CPU baseline is an N = 1 figure: one process then has the host's cores to itself
        barrier()

    sp = spread(ms, args.steps)
    step_ms = sp["median"]
    if world > 1:
        fp32_path = read_ceiling = None
    if rank == 0:
        value = total_bytes / (step_ms * 1e-3) / 1e9
        per_rank = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "ms_per_step_spread": sp, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": "c4_70b_layer_matvec", "shapes": "Q4_K q,o [8192,8192] k,v [1024,8192] gate,up [28672,8192]; Q6_K down [8192,28672]; batch 1",
                       "parallelism": parallelism, "l2": l2, "launch": launch, "pdl": bool(args.pdl), "frac_of_8000": per_rank / 8000.0},
            "roofline": {"bound": "hbm", "achieved": per_rank, "peak": peak, "unit": "GB/s", "frac": per_rank / peak,
                         "traffic": NCU_TRAFFIC_PER_STEP["c4_70b_layer_matvec"] if world == 1 else None, "peak_kind": f"of {peak_kind}", "kernel": kernel,
                         "launch_us": step_ms * 1e3 / launches_per_step, "launches_per_step": launches_per_step,
                         "algorithmic_bytes_per_step_per_gpu": total_bytes / world,
                         "note": "per GPU: algorithmic bytes of a rank's share of the step / step time (N > 1: the exchange is inside the step)"},
            "cpu_baseline": cpu,
            "e2e": {"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_step": e2e_s * 1e6, "api": e2e_api},
            "gpu_launches": launches_per_step * args.steps * len(ms),
            "clocks": clocks,
            "check": check,
        }
        if fp32_path is not None:
            line["roofline"]["fp32_path_gbs"] = fp32_path["gbs"]
            line["roofline"]["fp32_path"] = fp32_path
        if read_ceiling is not None:
            line["roofline"]["read_only_ceiling"] = read_ceiling
        if secondary is not None:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def read_only_ceiling(ctx, nbytes):
    """What a kernel that only READS `nbytes` (one launch, L2 flushed before it) reaches on this GPU: plain
    16-byte loads, and a bulk-copy ring with nothing consuming it (the streaming side of the matvec kernels
    alone, two stages of 92 KB as the Q4_K matrices use).  `peak` in the roofline stays the copy bandwidth;
    these two rates say how much of the gap to it a pure reader can close at all."""
    nbytes = nbytes // (1 << 20) * (1 << 20)
    ld = ctx.read_probe(0, nbytes)
    ring = ctx.read_probe(1, nbytes, 94208, 2, 16384)
    return {"bytes": nbytes, "plain_loads_gbs": ld["gbs"], "plain_loads_us": ld["us"], "bulk_copy_ring_gbs": ring["gbs"], "bulk_copy_ring_us": ring["us"],
            "note": "one launch over the same number of bytes as a step, 256 MB written before each launch; median of 8"}


def cpu_leg(check, gpu_outputs):
    """The oracle port on the same workload, on the host cores: full steps for about ten seconds."""
    _lift_omp_limit()
    cstep, cores, nbytes, _ = cpu_c4_step_factory()
    refs = cstep()
    t0 = time.perf_counter()
    n = 0
    while n < 3 or (time.perf_counter() - t0 < 10.0 and n < 400):
        refs = cstep()
        n += 1
    cdt = (time.perf_counter() - t0) / n
    if gpu_outputs is not None:
        check["rel_err_vs_cpu_full_vectors"] = max(synth.rel_err(g, r) for g, r in zip(gpu_outputs, refs))
    return {"value": nbytes / cdt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{n} full steps of c4_70b_layer_matvec, {cdt * 1e3:.1f} ms each"}


def run_slice(args):
    """Single-GPU diagnostic: what ONE rank of a `--slice-of W` group computes per step (rows / W of every matrix),
    without any peer: the sharded entry point on a group of one (the kernel and its epilogue, no exchange), and the
    same slices through the ordinary batch call.  The difference to the N = W line is what the exchange costs."""
    import torch

    from ullm_b200 import backend

    W = args.slice_of
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    ctx = backend.CudaContext(0)
    ctx.set_option(backend.OPT_PDL, 1 if args.pdl else 0)
    for kv in args.knob:
        ctx.debug_set(kv.split("=")[0], int(kv.split("=")[1]))
    outs = [o for _, _, o, _ in C4_MATS]
    offs = shard.vector_offsets(outs)
    total = offs[-1]
    slice_bytes = sum(weight_bytes(dt, o // W, c) for _, dt, o, c in C4_MATS)
    ncopies = max(1, -(-400_000_000 // slice_bytes))
    sh = backend.Shard(ctx, 1, 0, 2 * total)
    mats = []
    for i, (name, dt, out, cols) in enumerate(C4_MATS):
        rows = out // W
        w = synth.gen_weight(dt, rows, cols, synth.seed_for(4, i))
        mats.append(dict(rows=rows, cols=cols, x=torch.from_numpy(synth.normal(synth.seed_for(4, 8 + i), cols)).to(dev),
                         y=torch.empty(rows, dtype=torch.float32, device=dev), ws=[backend.Weight(ctx, dt, w, rows, cols) for _ in range(ncopies)]))
    ops = [[sh.ops([dict(w=m["ws"][c], x=m["x"].data_ptr(), y_offset=par * total + o, row0=0) for m, o in zip(mats, offs)]) for par in range(2)]
           for c in range(ncopies)]
    batches = [backend.WeightBatch(ctx, [m["ws"][c] for m in mats], [m["x"].data_ptr() for m in mats], [m["y"].data_ptr() for m in mats])
               for c in range(ncopies)]
    res = {"workload": f"one rank's share of c4 split {W} ways, on one GPU", "slice_mb": slice_bytes / 1e6, "copies": ncopies}
    sp = spread(time_graph(torch, lambda i, st: sh.matvec_dev(ops[i % ncopies][i & 1], st), args.steps, args.warmup, args.replays), args.steps)
    res["sharded_entry_us"] = sp["median"] * 1e3
    for name, pc in (("batch_chain_us", 1), ("batch_separate_us", 0)):
        ctx.debug_set("no_chain", 0 if pc else 1)
        sp = spread(time_graph(torch, lambda i, st: batches[i % ncopies].launch(st), args.steps, args.warmup, args.replays), args.steps)
        res[name] = sp["median"] * 1e3
    # every matrix alone (its own launches, copies walked round-robin)
    ctx.debug_set("no_chain", 0)
    per = {}
    for (name, dt, out, cols), m in zip(C4_MATS, mats):
        sp = spread(time_graph(torch, lambda i, st: m["ws"][i % ncopies].matvec_dev(m["x"].data_ptr(), m["y"].data_ptr(), st), args.steps, args.warmup, 5), args.steps)
        nb = weight_bytes(dt, m["rows"], cols)
        per[name] = {"us": round(sp["median"] * 1e3, 2), "gbs": round(nb / sp["median"] / 1e6, 1)}
    res["per_matrix_alone"] = per
    if args.tokens:
        # the same slices as a prefill GEMM: plain calls, and the sharded entry point on a group of one
        S = args.tokens
        goffs = [S * o for o in shard.vector_offsets(outs)]
        shg = backend.Shard(ctx, 1, 0, goffs[-1])
        xs = [torch.randn(S * m["cols"], dtype=torch.float32, device=dev) for m in mats]
        ys = [torch.empty(S * m["rows"], dtype=torch.float32, device=dev) for m in mats]
        gper = {}
        for (name, dt, out, cols), m, x_, y_ in zip(C4_MATS, mats, xs, ys):
            sp = spread(time_graph(torch, lambda i, st: m["ws"][0].matmul_dev(x_.data_ptr(), y_.data_ptr(), S, st), 4, 3, 5), 4)
            gper[name] = round(sp["median"] * 1e3, 1)
        res["gemm_plain_us_per_matrix"] = gper
        res["gemm_plain_us"] = sum(gper.values())

        def gstep(_i, st):
            for k, (m, off, x_) in enumerate(zip(mats, goffs, xs)):
                shg.matmul_dev(m["ws"][0], x_.data_ptr(), S, off, 0, m["rows"] * 1, st, 0 if k + 1 == len(mats) else backend.SHARD_NO_WAIT)

        sp = spread(time_graph(torch, gstep, 4, 3, 5), 4)
        res["gemm_sharded_entry_us"] = sp["median"] * 1e3
    if args.q6k_cost:
        ctx.debug_set("q6k_cost_permille", args.q6k_cost)
        sp = spread(time_graph(torch, lambda i, st: batches[i % ncopies].launch(st), args.steps, args.warmup, args.replays), args.steps)
        res[f"batch_chain_us_q6k_cost_{args.q6k_cost}"] = sp["median"] * 1e3
    ctx.synchronize()
    res["gbs_sharded_entry"] = (slice_bytes + 4 * sum(m["rows"] + m["cols"] for m in mats)) / res["sharded_entry_us"] / 1e3
    print(json.dumps(res), flush=True)
    return 0


def run_c4gemm_multi(args):
    """N > 1, --workload c4gemm: the block as a 512-token prefill GEMM, rows / N of every matrix per rank; the
    GEMM's epilogue stores each rank's [tokens, rows / N] block into its columns of [tokens, out] on every rank."""
    import torch
    import torch.distributed as dist

    from ullm_b200 import backend

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    ctx = backend.CudaContext(local)
    S = args.tokens
    outs = [o for _, _, o, _ in C4_MATS]
    offs = [S * o for o in shard.vector_offsets(outs)]  # [tokens, out] matrices one after the other
    sh = backend.Shard(ctx, world, rank, offs[-1])
    handles = [None] * world
    dist.all_gather_object(handles, sh.export())
    sh.connect(handles)
    mats = []
    for i, (name, dt, out, cols) in enumerate(C4_MATS):
        r0, rows = sh.row_range(out)
        w = synth.gen_weight(dt, rows, cols, synth.seed_for(4, i) + 0x100000 * (rank + 1))
        xs = torch.randn(S * cols, dtype=torch.float32, device=dev, generator=torch.Generator(device=dev).manual_seed(40 + i))
        xs = xs.to(torch.bfloat16).to(torch.float32)
        mats.append(dict(dt=dt, out=out, cols=cols, row0=r0, rows=rows, host=w, w=backend.Weight(ctx, dt, w, rows, cols), xs=xs))

    fused = {"fused": backend.SHARD_FUSED_STORES, "push": backend.SHARD_SM_PUSH, "copy": 0, "auto": 0}[args.gemm_exchange]
    if args.gemm_exchange == "copy":
        ctx.debug_set("shard_gemm_exchange", 1)  # comparison: copy engines whatever the block's shape

    def step(_i, st):
        for k, (m, off) in enumerate(zip(mats, offs)):
            last = k + 1 == len(mats)  # the step waits for the other ranks once, after its last matrix
            sh.matmul_dev(m["w"], m["xs"].data_ptr(), S, off, m["row0"], m["out"], st, (0 if last else backend.SHARD_NO_WAIT) | fused)

    dist.barrier()
    ms = time_graph(torch, step, max(2, args.steps // 4), 3, args.replays, before_timing=dist.barrier)
    ctx.synchronize()
    t = torch.tensor(ms, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sp = spread(t.tolist(), max(2, args.steps // 4))
    # parity: 64 rows x 8 tokens of every rank's block, read from this rank's copy of the full result
    import oracle

    _lift_omp_limit()
    mine = []
    for m in mats:
        l0 = max(0, m["rows"] - 64)
        rb = m["cols"] // 256 * (144 if m["dt"] == synth.Q4_K else 210)
        blk = np.ascontiguousarray(np.asarray(m["host"]).reshape(-1).view(np.uint8)[l0 * rb:m["rows"] * rb])
        xs_h = m["xs"][:8 * m["cols"]].cpu().numpy().reshape(8, m["cols"])
        mine.append((m["row0"] + l0, oracle.matmul_q(oracle.Weight(m["dt"], blk, m["rows"] - l0, m["cols"]), xs_h, 8).reshape(8, -1)))
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    worst = 0.0
    for i, (m, off) in enumerate(zip(mats, offs)):
        got = sh.read_y(off, 8 * m["out"]).reshape(8, m["out"])
        for r in range(world):
            g0, ref = everyone[r][i]
            worst = max(worst, synth.rel_err(got[:, g0:g0 + ref.shape[1]], ref))
    wt = torch.tensor([worst], dtype=torch.float64, device=dev)
    dist.all_reduce(wt, op=dist.ReduceOp.MAX)
    if rank == 0:
        flop = 2.0 * S * sum(o * c for _, _, o, c in C4_MATS)
        tf = flop / sp["median"] / 1e9
        print(json.dumps({"workload": "c4_70b_layer_gemm", "n_gpus": world, "tokens": S, "us_per_step": sp["median"] * 1e3, "ms_per_step_spread": sp,
                          "tflops": tf, "tflops_per_gpu": tf / world, "peak_tflops": measured_peak_tflops(),
                          "frac_per_gpu": tf / world / measured_peak_tflops(), "scaling": "strong",
                          "peer_store_bytes_per_rank_per_step": 4 * S * sum(outs) // world * (world - 1),
                          "exchange": args.gemm_exchange,
                          "parallelism": {"fused": f"rows/{world} per matrix; the GEMM epilogue stores each tile into all ranks' [tokens, out] over NVLink",
                                          "push": f"rows/{world} per matrix; each finished [tokens, rows/{world}] block is pushed to all ranks' [tokens, out] by a copy kernel on a side stream while the next matrix is multiplied; step flags instead of an all-gather",
                                          "auto": f"rows/{world} per matrix; each finished [tokens, rows/{world}] block is pushed to all ranks' [tokens, out] on a side stream while the next matrix is multiplied (copy kernel for narrow blocks or more than four ranks, else copy engines); step flags instead of an all-gather",
                                          "copy": f"rows/{world} per matrix; each finished [tokens, rows/{world}] block is pushed to all ranks' [tokens, out] by the copy engines (one stream per peer) while the next matrix is multiplied; step flags instead of an all-gather"}[args.gemm_exchange],
                          "launch": "one CUDA graph of the timed steps, replayed", "check": {"rel_err_vs_cpu_64_rows_8_tokens_per_rank": float(wt.item())}}), flush=True)
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--replays", type=int, default=15, help="timed replays of the K-step graph (median / min / max reported)")
    ap.add_argument("--tokens", type=int, default=512, help="prefill length of the GEMM workloads")
    ap.add_argument("--pdl", type=int, default=1, help="ULLM_OPT_PDL: launch kernels programmatically dependent on their predecessor")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true", help="N = 1: skip the other configurations")
    ap.add_argument("--launch", default="auto", choices=["auto", "separate"],
                    help="N = 1: the batch call (one persistent launch for the seven matrices) or seven launches per step")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="N > 1: fused peer stores (default) or the NCCL all-gather comparison arm")
    ap.add_argument("--workload", default="c4", choices=["c4", "c4gemm", "c0", "c1", "c2", "c3", "c2decode", "c3prefill", "readprobe"],
                    help="c4 is the benchmark.  N > 1: c4gemm runs the block as a sharded prefill GEMM.  N = 1: any other choice runs that "
                         "configuration alone and prints its figures (what `secondary` holds, plus the MoE decode step and the batched prefill)")
    ap.add_argument("--layers", type=int, default=0, help="c2decode: number of layers (default: the model's 48)")
    ap.add_argument("--only", default="", help="c4gemm at N = 1: just this matrix of the block (q, k, v, o, gate, up, down)")
    ap.add_argument("--q6k-cost", type=int, default=0, help="--slice-of diagnostic: also time the persistent launch with this per-byte cost (permille) of Q6_K rows")
    ap.add_argument("--gemm-exchange", default="auto", choices=["auto", "copy", "fused", "push"],
                    help="c4gemm at N > 1: the library's choice per block (default), or forced: copy engines on side streams, stores from the GEMM epilogue, a copy kernel on the side stream")
    ap.add_argument("--slice-of", type=int, default=0, help="N = 1 diagnostic: time one rank's share of a W-way split without peers")
    ap.add_argument("--knob", action="append", default=[], help="test knob key=value passed to the library (sweeps; not used by any default run)")
    ap.add_argument("--eager", action="store_true", help="launch the timed steps from the host instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global EAGER
    EAGER = args.eager
    if args.impl == "reference":
        return run_reference(args)
    if args.slice_of:
        return run_slice(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and args.workload == "c4gemm":
        return run_c4gemm_multi(args)
    if args.workload != "c4":
        return run_aux(args)
    return run_c4(args)


if __name__ == "__main__":
    sys.exit(main())
