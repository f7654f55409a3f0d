#!/usr/bin/env python
"""Benchmark of the quantized matvec hot path (BASELINE.json's metric: achieved
HBM GB/s of the dequant-in-kernel matvec).

One JSON line on stdout.  A *step* is one pass of the hot path over one batch of
synthetic input:

* ``--gpus 1`` — workload ``c1_q6k_ffn_pair``: the Q6_K matvec [14336, 4096]
  followed by the companion Q6_K down-projection [4096, 14336] on its result.
  Weights are resident; successive steps walk distinct device copies of the two
  matrices whose total exceeds L2 several times over, so every step reads HBM.
* ``--gpus N`` (N > 1, under torchrun) — workload ``c4_70b_layer_matvec``: the
  seven matrices of one Llama-3-70B-shaped block, output rows split evenly over
  the ranks, followed by an NCCL all-gather of each output vector.

``value`` is device-timed (CUDA events on the launching stream, max over ranks);
``e2e`` goes through the host-buffer entry point ``ullm_cuda_weight_matvec`` with
pinned host activations (host<->device copies inside the timed region).
``--impl reference`` times the CPU restatement of the reference's path (the
oracle port, OpenMP over rows) on the host cores for the same workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel,
# from the ncu capture summarised in profiles/ (None until captured).
NCU_TRAFFIC_PER_LAUNCH = {"c1_q6k_ffn_pair": (48_236_032 + 48_276_992) // 2}  # dram read + write of the two launches, ncu capture under profiles/

C4_MATS = [  # name, dtype, out, in   (one Llama-3-70B block)
    ("q", synth.Q4_K, 8192, 8192), ("k", synth.Q4_K, 1024, 8192), ("v", synth.Q4_K, 1024, 8192),
    ("o", synth.Q4_K, 8192, 8192), ("gate", synth.Q4_K, 28672, 8192), ("up", synth.Q4_K, 28672, 8192),
    ("down", synth.Q6_K, 8192, 28672),
]


def weight_bytes(dtype, out, cols):
    return out * (cols // 256) * (144 if dtype == synth.Q4_K else 210)


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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.idx)],
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


def run_reference(args):
    """The reference's CPU path (oracle port) on the host cores, same workload and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is the CPU path with every host thread it can
    # use, so the setting is lifted before the oracle library (and with it the OpenMP runtime) is loaded
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    factory = cpu_c1_step_factory if args.gpus == 1 else cpu_c4_step_factory
    workload = "c1_q6k_ffn_pair" if args.gpus == 1 else "c4_70b_layer_matvec"
    # Size the per-step sample so that warmup + steps end within ~2 minutes.
    probe, cores, pbytes, _ = factory(1.0 / 16)
    probe()
    t0 = time.perf_counter()
    probe()
    t_probe = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)
    frac = min(1.0, (1.0 / 16) * budget / max(t_probe, 1e-6))
    step, cores, nbytes, sample = factory(frac)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    gbs = args.steps * nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": "quantized_matvec_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "note": "C restatement of ullm-model's CPU path (rayon -> OpenMP over rows); the Rust reference cannot be built here"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": f"{args.steps} steps, each over {sample}"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------
# CUDA arm
# ---------------------------------------------------------------------------
def run_single(args):
    import torch

    from ullm_b200 import backend

    torch.cuda.set_device(0)
    ctx = backend.CudaContext(0)
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.device("cuda:0")

    w_up_h = synth.gen_q6k(*C1_UP, synth.seed_for(1, 0))
    w_dn_h = synth.gen_q6k(*C1_DOWN, synth.seed_for(1, 1))
    x_h = synth.normal(synth.seed_for(1, 2), C1_UP[1])
    ncopies = args.copies  # 2 * 48 MB per copy; the walk must exceed L2 (126 MB) several times
    # resident weight objects (what GpuForward::new builds from a GpuWeight): one device copy each
    ups = [backend.Weight(ctx, backend.Q6_K, w_up_h, *C1_UP) for _ in range(ncopies)]
    dns = [backend.Weight(ctx, backend.Q6_K, w_dn_h, *C1_DOWN) for _ in range(ncopies)]
    x = torch.from_numpy(x_h).to(dev)
    h = torch.empty(C1_UP[0], dtype=torch.float32, device=dev)
    y = torch.empty(C1_DOWN[0], dtype=torch.float32, device=dev)

    # the pair as one persistent launch (up, then down behind a grid barrier) or as two launches
    chains = [backend.WeightChain(ctx, [dict(w=ups[c], x=x.data_ptr(), y=h.data_ptr()),
                                        dict(w=dns[c], x=h.data_ptr(), y=y.data_ptr(), dep=True)]) for c in range(ncopies)]

    def step(i):
        c = i % ncopies
        if args.chain:
            chains[c].launch(stream)
        else:
            ups[c].matvec_dev(x.data_ptr(), h.data_ptr(), stream)
            dns[c].matvec_dev(h.data_ptr(), y.data_ptr(), stream)

    if args.pdl:
        ctx.debug_set("pdl", 1)
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    plan = ctx.last_plan()

    # The K timed steps are captured into one CUDA graph and replayed, so the host's
    # launch rate (a few microseconds per call from Python) is not what is measured.
    side = torch.cuda.Stream()
    graph = None
    if not args.eager:
        stream = side.cuda_stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.steps):
                step(args.warmup + i)
        graph.replay()  # one untimed replay
        torch.cuda.synchronize()

    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        ev0.record()
        if graph is not None:
            graph.replay()
        else:
            stream = side.cuda_stream
            for i in range(args.steps):
                step(args.warmup + i)
        ev1.record()
    torch.cuda.synchronize()
    ctx.synchronize()  # surfaces a device-side timeout status
    ms = ev0.elapsed_time(ev1)

    # end to end: host buffers in, host buffers out, through matvec_resident
    xp = torch.from_numpy(x_h).pin_memory().numpy()
    hp = torch.empty(C1_UP[0], dtype=torch.float32).pin_memory().numpy()
    yp = torch.empty(C1_DOWN[0], dtype=torch.float32).pin_memory().numpy()

    def e2e_step(i):
        c = i % ncopies
        ups[c].matvec(xp, out=hp)
        dns[c].matvec(hp, out=yp)

    for i in range(args.warmup):
        e2e_step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(args.warmup + i)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()

    # parity spot check of what was timed (64 rows of the final output)
    y_host = y.cpu().numpy()
    check = {"rel_err_vs_e2e": synth.rel_err(y_host, yp)}

    step_bytes = 2 * C1_BYTES_PER_LAUNCH
    value = args.steps * step_bytes / (ms * 1e-3) / 1e9
    per_launch = 2 if args.chain else 1  # matrices streamed by one launch
    launch_us = ms * 1e3 / (2 * args.steps) * per_launch
    peak, peak_kind = measured_peak_gbs()
    achieved = per_launch * C1_BYTES_PER_LAUNCH / (launch_us * 1e-6) / 1e9

    cpu = None
    if not args.no_cpu:
        cstep, cores, _, _ = cpu_c1_step_factory()
        cstep()
        t0 = time.perf_counter()
        n = 0
        while n < 3 or (time.perf_counter() - t0 < 10.0 and n < 200):
            ref = cstep()
            n += 1
        cdt = (time.perf_counter() - t0) / n
        check["rel_err_vs_cpu"] = synth.rel_err(y_host, ref)
        cpu = {"value": step_bytes / cdt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
               "sample": f"{n} full steps of c1_q6k_ffn_pair, {cdt * 1e3:.1f} ms each"}

    line = {
        "metric": "quantized_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 dot products (16-bit fixed-point x) + f32 accumulate", "data": "synthetic",
        "config": {"workload": "c1_q6k_ffn_pair", "shapes": "Q6_K [14336,4096] then Q6_K [4096,14336], batch 1",
                   "l2": f"{ncopies} distinct weight copies ({ncopies * 96} MB) walked round-robin: inputs larger than L2",
                   "plan": plan, "pdl": bool(args.pdl), "launch": "eager" if args.eager else "one CUDA graph of all timed steps",
                   "frac_of_8000": value / 8000.0},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": per_launch * NCU_TRAFFIC_PER_LAUNCH["c1_q6k_ffn_pair"], "peak_kind": f"of {peak_kind}",
                     "kernel": "matvec_chain_kernel (both matrices, one persistent launch)" if args.chain else "matvec_stream_kernel<Q6_K prepared>",
                     "launch_us": launch_us, "algorithmic_bytes_per_launch": per_launch * C1_BYTES_PER_LAUNCH},
        "cpu_baseline": cpu,
        "e2e": {"value": args.steps * step_bytes / e2e_s / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": 4 * (C1_UP[1] + C1_DOWN[1]), "d2h_bytes_per_step": 4 * (C1_UP[0] + C1_DOWN[0]),
                "us_per_step": e2e_s / args.steps * 1e6, "api": "ullm_cuda_weight_matvec (resident weight, pinned host x / y)"},
        "gpu_launches": (1 if args.chain else 2) * args.steps,
        "clocks": clocks,
        "check": check,
    }
    print(json.dumps(line), flush=True)
    return 0


def _time_steps(torch, step, steps, warmup):
    """step(i, stream) enqueues step i; the timed steps run as one CUDA graph."""
    cur = torch.cuda.current_stream().cuda_stream
    for i in range(warmup):
        step(i, cur)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(steps):
            step(warmup + i, side.cuda_stream)
    graph.replay()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        ev0.record()
        graph.replay()
        ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1)


def run_other(args):
    """Single-GPU measurements of the other benchmark configurations (parity-test
    cases; reported for the design notes, not the headline line)."""
    import torch

    from ullm_b200 import backend

    torch.cuda.set_device(0)
    ctx = backend.CudaContext(0)
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.device("cuda:0")
    peak, peak_kind = measured_peak_gbs()
    if args.pdl:
        ctx.debug_set("pdl", 1)
    out = {"workload": args.workload, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "pdl": bool(args.pdl)}

    if args.workload == "c0":
        shape = (4096, 4096)
        w = synth.gen_q4k(*shape, synth.seed_for(0, 0))
        n = 40  # 9.4 MB each: 377 MB walked round-robin
        ws = [backend.Weight(ctx, backend.Q4_K, w, *shape) for _ in range(n)]
        x = torch.from_numpy(synth.normal(synth.seed_for(0, 1), shape[1])).to(dev)
        y = torch.empty(shape[0], dtype=torch.float32, device=dev)
        ms = _time_steps(torch, lambda i, st: ws[i % n].matvec_dev(x.data_ptr(), y.data_ptr(), st), args.steps, args.warmup)
        nbytes = weight_bytes(synth.Q4_K, *shape) + 4 * sum(shape)
        out.update(us_per_launch=ms * 1e3 / args.steps, gbs=args.steps * nbytes / ms / 1e6, bytes_per_launch=nbytes, plan=ctx.last_plan())
    elif args.workload == "c4":
        mats = []
        for i, (name, dt, o, c) in enumerate(C4_MATS):
            w = synth.gen_weight(dt, o, c, synth.seed_for(4, i))
            mats.append((backend.Weight(ctx, dt, w, o, c), torch.from_numpy(synth.normal(synth.seed_for(4, 8 + i), c)).to(dev),
                         torch.empty(o, dtype=torch.float32, device=dev)))

        def step(_i, st):
            for w, xv, yv in mats:
                w.matvec_dev(xv.data_ptr(), yv.data_ptr(), st)

        ms = _time_steps(torch, step, args.steps, args.warmup)
        nbytes = sum(weight_bytes(dt, o, c) + 4 * (o + c) for _, dt, o, c in C4_MATS)
        out.update(us_per_step=ms * 1e3 / args.steps, gbs=args.steps * nbytes / ms / 1e6, bytes_per_step=nbytes)
    elif args.workload == "c4gemm":
        # the same block as a prefill GEMM: 512 tokens through every matrix (tcgen05 path)
        S = args.tokens
        tf_peak = measured_peak_tflops()
        per, total_ms, total_flop = {}, 0.0, 0.0
        for i, (name, dt, o, c) in enumerate(C4_MATS):
            if args.only and name != args.only:
                continue
            w = backend.Weight(ctx, dt, synth.gen_weight(dt, o, c, synth.seed_for(4, i)), o, c)
            xs = torch.randn(S * c, dtype=torch.float32, device=dev, generator=torch.Generator(device=dev).manual_seed(40 + i))
            ys = torch.empty(S * o, dtype=torch.float32, device=dev)
            ms = _time_steps(torch, lambda _i, st: w.matmul_dev(xs.data_ptr(), ys.data_ptr(), S, st), args.steps, args.warmup)
            flop = 2.0 * S * o * c
            per[name] = {"us": round(ms * 1e3 / args.steps, 2), "tflops": round(args.steps * flop / ms / 1e9, 1)}
            total_ms += ms / args.steps
            total_flop += flop
            assert ctx.last_plan()["grid"] == -1, "tensor-core GEMM did not run"
            w.free()
            del xs, ys
        out.update(tokens=S, us_per_step=total_ms * 1e3, tflops=total_flop / total_ms / 1e9, peak_tflops=tf_peak,
                   frac=total_flop / total_ms / 1e9 / tf_peak, per_matrix=per,
                   note="includes the f32->bf16 activation cast kernel of every call")
    elif args.workload == "c2":
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
        ms = _time_steps(torch, lambda i, st: exs[i % 2].moe_ffn_dev(x.data_ptr(), lgs[i % 4].data_ptr(), ntok, k, y.data_ptr(), stream=st), args.steps, args.warmup)
        D = sum(dist) / len(dist)
        nbytes = D * 2_654_208 + 131_072
        out.update(us_per_step=ms * 1e3 / args.steps, distinct_experts=D, gbs=args.steps * nbytes / ms / 1e6,
                   bytes_per_step=nbytes, launches_per_step=4)
    elif args.workload == "c3":
        p = dict(synth.LLAMA_1B)
        m = synth.gen_llama_model(p, synth.seed_for(3, 0))
        kk, vv = synth.gen_kv_prefill(p, 1024, synth.seed_for(3, 1))
        gf = backend.GpuForward(ctx, m, kv_f16=True)
        gf.set_kv(0, kk, vv)
        embd = ctx.upload(m["tok_embd"][1])
        prompt = synth.rand_ints(synth.seed_for(3, 2), 16, 0, p["vocab"] - 1)
        import oracle  # embedding rows for the prompt (host-side lookup, as the reference does)

        emb_w = oracle.Weight(m["tok_embd"][0], m["tok_embd"][1], p["vocab"], p["n_embd"])
        t0 = time.perf_counter()
        for i, t in enumerate(prompt):
            row = oracle.dequantize(m["tok_embd"][0], m["tok_embd"][1][int(t)], p["n_embd"])
            lg = gf.forward(row, 1024 + i)
        t_prompt = time.perf_counter() - t0
        tok = int(np.argmax(lg))
        n_gen = 128 if args.steps == 500 else args.steps  # 128 tokens unless --steps is given
        gf.greedy(embd, m["tok_embd"][0], tok, 1040, min(8, n_gen))  # warm the greedy graph
        t0 = time.perf_counter()
        toks = gf.greedy(embd, m["tok_embd"][0], tok, 1040, n_gen)
        dt = time.perf_counter() - t0
        wbytes = 16 * 38_805_504 + 215_470_080
        kvbytes = 32_768 * (1040 + 64)
        out.update(tok_per_s=n_gen / dt, us_per_token=dt / n_gen * 1e6, prompt_ms_per_token=t_prompt / 16 * 1e3, tokens=n_gen,
                   bytes_per_token=wbytes + kvbytes + 513_024, gbs=(wbytes + kvbytes + 513_024) * n_gen / dt / 1e9,
                   first_tokens=toks[:8].tolist())
    elif args.workload == "c2decode":
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
        n_gen = 128 if args.steps == 500 else args.steps
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
    elif args.workload == "c3prefill":
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
    if "gbs" in out:
        out["frac_of_measured_peak"] = out["gbs"] / peak
    out["peak_kind"] = peak_kind
    print(json.dumps(out), flush=True)
    return 0


def run_multi_gemm(args):
    """N>1, --workload c4gemm: the 70B block as a 512-token prefill GEMM, rows/N of every matrix per
    rank (tcgen05 kernel on the slice), one all-gather of the ranks' [tokens, rows/N] outputs per step."""
    import torch
    import torch.distributed as dist

    from ullm_b200 import backend

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ctx = backend.CudaContext(local)
    dev = torch.device(f"cuda:{local}")
    S = args.tokens
    rows_total = shard.local_offsets([o for _, _, o, _ in C4_MATS], world)[-1]
    mats = []
    for i, (name, dt, out, cols) in enumerate(C4_MATS):
        rows = out // world
        w = backend.Weight(ctx, dt, synth.gen_weight(dt, rows, cols, synth.seed_for(4, i) + 0x100000 * (rank + 1)), rows, cols)
        xs = torch.randn(S * cols, dtype=torch.float32, device=dev, generator=torch.Generator(device=dev).manual_seed(40 + i))
        y_r = torch.empty(S * rows, dtype=torch.float32, device=dev)             # this rank's [token][rows/N]
        y_g = torch.empty(world * S * rows, dtype=torch.float32, device=dev)     # [rank][token][rows/N]
        mats.append((w, xs, y_r, y_g))
    side = torch.cuda.Stream()
    ctx.debug_set("pdl", 0)

    def step():
        # the gather of one matrix' output overlaps the GEMM of the next (NCCL runs on its own stream)
        works = []
        for w, xs, y_r, y_g in mats:
            w.matmul_dev(xs.data_ptr(), y_r.data_ptr(), S, side.cuda_stream)
            works.append(dist.all_gather_into_tensor(y_g, y_r, async_op=True))
        for wk in works:
            wk.wait()

    with torch.cuda.stream(side):
        for _ in range(max(args.warmup, 3)):
            step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms_t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = float(ms_t.item()) / args.steps
    if rank == 0:
        flop = 2.0 * S * sum(o * c for _, _, o, c in C4_MATS)
        tf = flop / ms / 1e9
        print(json.dumps({"workload": "c4gemm", "n_gpus": world, "tokens": S, "steps": args.steps, "us_per_step": ms * 1e3,
                          "tflops": tf, "tflops_per_gpu": tf / world, "peak_tflops": measured_peak_tflops(),
                          "frac_per_gpu": tf / world / measured_peak_tflops(), "scaling": "strong",
                          "gather_bytes_per_step": 4 * world * S * rows_total,
                          "parallelism": f"rows/{world} per matrix; each matrix' [token][rows/N] output is all-gathered while the next matrix is multiplied",
                          "launch": "host launches + NCCL"}), flush=True)
    dist.destroy_process_group()
    return 0


def run_multi(args):
    import torch
    import torch.distributed as dist

    from ullm_b200 import backend

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ctx = backend.CudaContext(local)
    dev = torch.device(f"cuda:{local}")
    stream = torch.cuda.current_stream().cuda_stream

    # Row slices: rank r owns rows [r*out/N, (r+1)*out/N) of every matrix and generates
    # only those (rows are self-contained byte ranges).  Enough distinct device copies of
    # the slice set are walked round-robin that a step never finds its weights in L2.
    slice_bytes = sum(weight_bytes(dt, o // world, c) for _, dt, o, c in C4_MATS)
    ncopies = max(1, -(-400_000_000 // slice_bytes))
    rows_total = shard.local_offsets([o for _, _, o, _ in C4_MATS], world)[-1]
    y_cat = torch.empty(rows_total, dtype=torch.float32, device=dev)       # this rank's rows of all 7 outputs
    y_all = torch.empty(world * rows_total, dtype=torch.float32, device=dev)  # [rank][matrix][rows]
    mats, off = [], 0
    for i, (name, dt, out, cols) in enumerate(C4_MATS):
        assert out % world == 0
        rows = out // world
        w = synth.gen_weight(dt, rows, cols, synth.seed_for(4, i) + 0x100000 * (rank + 1))
        xv = synth.normal(synth.seed_for(4, 8 + i), cols)
        mats.append(dict(rows=rows, cols=cols, off=off, ws=[backend.Weight(ctx, dt, w, rows, cols) for _ in range(ncopies)],
                         x=torch.from_numpy(xv).to(dev), xh=torch.from_numpy(xv).pin_memory()))
        off += rows
    y_host = torch.empty(world * rows_total, dtype=torch.float32).pin_memory()

    # Kernels and the NCCL collective share one non-default stream (a NULL handle would
    # send the kernels to the context's own stream, unordered with NCCL).
    side = torch.cuda.Stream()
    stream = side.cuda_stream
    use_pdl = bool(args.pdl) and args.multi_graph
    ctx.debug_set("pdl", 1 if use_pdl else 0)
    batches = [backend.WeightBatch(ctx, [m["ws"][c] for m in mats], [m["x"].data_ptr() for m in mats],
                                   [y_cat.data_ptr() + 4 * m["off"] for m in mats]) for c in range(ncopies)]

    def step(i):
        batches[i % ncopies].launch(stream)  # the seven matvecs of this rank, one host call
        # the one exchange of the path: every rank's output rows to every rank
        dist.all_gather_into_tensor(y_all, y_cat)

    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for i in range(max(args.warmup, 3)):
            step(i)
    torch.cuda.synchronize()
    # the batch call is one persistent launch when the chain kernel takes the list, else one launch per matrix
    launches_per_step = 1 if ctx.last_plan()["grid"] == -2 else len(mats)
    graph = None
    if args.multi_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    step(args.warmup + i)
            graph.replay()
            torch.cuda.synchronize()
        except Exception as e:  # fall back to host launches, say so in the line
            graph = None
            print(f"graph capture failed on rank {rank}: {e}", file=sys.stderr)
            torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        ev0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(args.steps):
                step(args.warmup + i)
        ev1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ctx.synchronize()

    # end to end: x vectors from pinned host memory, gathered outputs back to the host
    def e2e_step(i):
        with torch.cuda.stream(side):
            for m in mats:
                m["x"].copy_(m["xh"], non_blocking=True)
            step(i)
            y_host.copy_(y_all, non_blocking=True)
        side.synchronize()

    for i in range(3):
        e2e_step(i)
    dist.barrier()
    t0 = time.perf_counter()
    n_e2e = min(args.steps, 200)
    for i in range(n_e2e):
        e2e_step(i)
    e2e_t = torch.tensor([time.perf_counter() - t0], device=dev)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_t.item()) / n_e2e
    ms_t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = float(ms_t.item())
    clocks = sampler.stop() if rank == 0 else None

    total_bytes = sum(weight_bytes(dt, o, c) + 4 * (o + c) for _, dt, o, c in C4_MATS)
    if rank == 0:
        value = args.steps * total_bytes / (ms * 1e-3) / 1e9
        peak, peak_kind = measured_peak_gbs()
        line = {
            "metric": "quantized_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 dot products (16-bit fixed-point x) + f32 accumulate", "data": "synthetic",
            "config": {"workload": "c4_70b_layer_matvec", "shapes": "Q4_K q,o [8192,8192] k,v [1024,8192] gate,up [28672,8192]; Q6_K down [8192,28672]",
                       "parallelism": f"rows/{world} per matrix, one NCCL all-gather of the ranks' output rows per step",
                       "l2": f"{ncopies} distinct copies of the per-rank slice set ({slice_bytes // 1000000} MB each) walked round-robin: inputs larger than L2",
                       "launch": "one CUDA graph of all timed steps" if graph is not None else "host launches (one C call per step) + NCCL", "pdl": use_pdl},
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                         "traffic": None, "peak_kind": f"of {peak_kind}", "kernel": "matvec_stream_kernel (per rank, incl. all-gather time)"},
            "cpu_baseline": None,
            "e2e": {"value": total_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * sum(c for _, _, _, c in C4_MATS),
                    "d2h_bytes_per_step": 4 * world * rows_total, "us_per_step": e2e_s * 1e6,
                    "api": "pinned host x -> ullm_cuda_weight_matvec_dev x7 -> NCCL all-gather -> pinned host y"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=512, help="prefill length of the c4gemm workload")
    ap.add_argument("--layers", type=int, default=0, help="c2decode: number of layers (default: the model's 48)")
    ap.add_argument("--only", default="", help="c4gemm: run just this matrix of the block (q, k, v, o, gate, up, down)")
    ap.add_argument("--pdl", type=int, default=1, help="launch the kernels with programmatic dependent launch (weight prefetch of the next kernel overlaps the tail of the previous one)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--chain", type=int, default=0,
                    help="c1: run the pair as one persistent launch (ullm_cuda_weight_matvec_chain_dev); measured slower than "
                         "two programmatically chained launches for this pair, so off by default")
    ap.add_argument("--multi-graph", action="store_true", help="N>1: capture kernels + NCCL in a CUDA graph (off by default)")
    ap.add_argument("--eager", action="store_true", help="launch the timed steps from the host instead of replaying a CUDA graph")
    ap.add_argument("--workload", default="c1", choices=["c0", "c1", "c2", "c2decode", "c3", "c3prefill", "c4", "c4gemm"],
                    help="single-GPU only: c1 is the headline workload, the others are auxiliary measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_multi_gemm(args) if args.workload == "c4gemm" else run_multi(args)
    if args.workload != "c1":
        return run_other(args)
    return run_single(args)


if __name__ == "__main__":
    sys.exit(main())
