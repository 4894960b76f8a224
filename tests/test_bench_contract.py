"""bench.py's arithmetic and the reference arm's JSON line (CPU only)."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_workload_arithmetic_matches_published_figures():
    n = bench.workload_numbers(bench.WORKLOADS["c3"])
    assert n["flops"] == pytest.approx(59.190e9, rel=1e-4) and n["bytes"] == pytest.approx(52.56e6, rel=1e-3)
    n = bench.workload_numbers(bench.WORKLOADS["c2"])
    assert n["flops"] == pytest.approx(26.307e9, rel=1e-4) and n["bytes"] == pytest.approx(513.84e6, rel=1e-3)
    n = bench.workload_numbers(bench.WORKLOADS["c4"])
    assert n["oh"] == 112 and n["flops"] == pytest.approx(60.423e9, rel=1e-4)
    assert n["bytes"] == pytest.approx(488.13e6, rel=1e-3)
    n = bench.workload_numbers(bench.WORKLOADS["c1"])
    assert n["flops"] == pytest.approx(0.9248e9, rel=1e-3) and n["bytes"] == pytest.approx(6.570e6, rel=1e-3)


def test_peaks_fall_back_when_file_is_missing(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    peaks, source = bench.load_peaks()
    assert source == "fallback" and peaks["hbm_gbs"] == 6650.0 and peaks["bf16_tflops"] == 1590.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 6517.6, "bf16_tflops": 1630.7, "bf16_tflops_sustained": 1369.7}))
    peaks, source = bench.load_peaks()
    assert source == "measured" and peaks["bf16_tflops"] == 1630.7


@pytest.mark.parametrize("workload", ["c3", "c1"])
def test_reference_arm_prints_one_contract_line(workload):
    env = dict(os.environ, RANK="0", WORLD_SIZE="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", workload,
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, env=env, timeout=600)  # ~3 s of warm-up
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fused_conv2d_tflops" and d["unit"] == "TFLOP/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["config"]["workload"] == workload
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["steps"] == 2 and d["warmup"] == 1, "the arm times exactly the steps it was asked for"
    assert d["ms_per_step"] <= d["ms_per_step_mean"] * 1.5 and d["value_from_mean"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_cpu_timer_warms_up_until_steady_then_times_exactly_the_requested_calls():
    calls = []
    durations = iter([0.030, 0.012, 0.004, 0.0041] + [0.004] * 50)   # slow first calls, then steady

    def fn():
        d = next(durations)
        calls.append(d)
        import time
        time.sleep(d)

    times = bench.time_cpu_calls(fn, warmup=1, steps=5, min_warm_seconds=0.0)
    assert len(times) == 5 and len(calls) == 4 + 5, "warm-up ends at the first two calls that agree within 5 %"
    assert max(times) < 0.012
    t0 = __import__("time").perf_counter()
    times = bench.time_cpu_calls(lambda: None, warmup=3, min_seconds=0.05, min_warm_seconds=0.2)
    assert len(times) >= 3 and __import__("time").perf_counter() - t0 >= 0.2, "the warm-up lasts its minimum time"
