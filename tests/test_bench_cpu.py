"""CPU tests of bench.py's reference arm (``--impl reference``: the oracle port on the host cores) and of the
helpers every arm uses: the JSON line has the keys the measurement contract names, rank 0 alone prints under a
multi-process launch, and the byte counts behind GB/s are the algorithmic ones."""
import argparse
import json

import numpy as np

import bench
import oracle
from ullm_b200 import synth


def _tiny_factory(frac: float = 1.0):
    """Eight rows of every matrix of the block: the same code path as the full sample, in milliseconds."""
    ws, xs, nbytes = [], [], 0
    for i, (_name, dt, _out, cols) in enumerate(bench.C4_MATS):
        ws.append(oracle.Weight(dt, synth.gen_weight(dt, 8, cols, 1000 + i), 8, cols))
        xs.append(synth.normal(2000 + i, cols))
        nbytes += bench.weight_bytes(dt, 8, cols) + 4 * (8 + cols)
    return (lambda: [oracle.matvec_q(w, x) for w, x in zip(ws, xs)]), oracle.max_threads(), nbytes, "8 rows of each of the 7 matrices"


def test_reference_arm_prints_one_contract_line(monkeypatch, capsys):
    monkeypatch.setattr(bench, "cpu_c4_step_factory", _tiny_factory)
    monkeypatch.delenv("RANK", raising=False)
    assert bench.run_reference(argparse.Namespace(steps=3, warmup=1, gpus=1)) == 0
    out = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(out) == 1
    line = json.loads(out[0])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == "GB/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert (line["n_gpus"], line["steps"], line["warmup"]) == (1, 3, 1) and line["ms_per_step"] > 0
    assert line["config"]["workload"] == "c4_70b_layer_matvec"
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "sample" in cb
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_exit_quietly(monkeypatch, capsys):
    monkeypatch.setenv("RANK", "3")
    assert bench.run_reference(argparse.Namespace(steps=3, warmup=1, gpus=8)) == 0
    assert capsys.readouterr().out == ""


def test_algorithmic_bytes_of_the_step():
    """542,498,816 bytes: packed weights of the seven matrices plus 4 bytes per input and output element."""
    q4 = lambda out, cols: out * cols // 256 * 144
    q6 = lambda out, cols: out * cols // 256 * 210
    weights = 2 * q4(8192, 8192) + 2 * q4(1024, 8192) + 2 * q4(28672, 8192) + q6(8192, 28672)
    vectors = 4 * sum(out + cols for _n, _dt, out, cols in bench.C4_MATS)
    assert bench.c4_step_bytes() == weights + vectors == 542_498_816
    assert bench.weight_bytes(synth.Q4_K, 1024, 8192) == q4(1024, 8192)


def test_spread_reports_median_min_max_per_step():
    sp = bench.spread([2.0, 1.0, 4.0], 2)
    assert sp == {"median": 1.0, "min": 0.5, "max": 2.0, "replays": 3}
    assert np.isclose(bench.spread([3.0], 3)["median"], 1.0)


def test_roofline_denominators_come_from_the_measured_file_or_the_stated_fallback(monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.measured_peak_gbs() == (6650.0, "fallback") and bench.measured_peak_tflops() == 1590.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6545.0, "bf16_tflops": 1699.0}))
    assert bench.measured_peak_gbs() == (6545.0, "measured") and bench.measured_peak_tflops() == 1699.0
