"""The parts of bench.py that run without a GPU: the reference arm's line, the bandwidth and
roofline arithmetic, the clock sampler's degraded mode, and the GPU tests' bench run (gpu mark)."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_reference_arm_prints_one_unavailable_line_and_exits_zero():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "8",
                           "--steps", "5", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and "CUDA 13.1" in line["unavailable"]


def test_reference_arm_under_a_per_gpu_launcher_prints_once_per_job():
    outputs = []
    for rank in range(3):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="3", LOCAL_RANK=str(rank))
        done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "3"],
                              capture_output=True, text=True, timeout=120, env=env)
        assert done.returncode == 0
        outputs.append([line for line in done.stdout.splitlines() if line.strip()])
    assert [len(o) for o in outputs] == [1, 0, 0]


def test_bus_bandwidth_and_roofline_arithmetic():
    bench = load_bench()
    gib = 1 << 30
    assert bench.busbw(gib, 1.0, 1) == pytest.approx(gib / 1e6)  # one rank: plain pass bandwidth
    assert bench.busbw(gib, 2.0, 8) == pytest.approx(gib / 2e6 * 14 / 8)
    r = bench.roofline(gib, 2.233, 8)
    assert r["bound_ms"] == pytest.approx(gib * 1.125 / 770e6, abs=1e-3)
    assert r["bound_busbw_gb_s"] == pytest.approx(770 * 14 / 9, abs=0.1)
    assert 0.69 < r["fraction_of_measured"] < 0.71
    assert "note" in bench.roofline(gib, 1.0, 1)


def test_clock_sampler_without_nvml_reports_nothing_instead_of_failing():
    bench = load_bench()
    sampler = bench.ClockSampler(0)
    sampler.start()
    out = sampler.stop()
    assert set(out) >= {"sm_mhz", "sm_max_mhz", "reasons", "samples"}
    if not sampler.ok:
        assert out["sm_mhz"] is None and out["samples"] == 0


def test_default_arguments_are_the_contract():
    bench = load_bench()
    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        args = bench.parse_args()
    finally:
        sys.argv = old
    assert (args.gpus, args.warmup, args.impl, args.bytes) == (1, 3, "ours", 1 << 30) and args.steps >= 1


@pytest.mark.gpu
def test_bench_line_has_every_key_of_the_contract():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "3", "--warmup", "3",
                           "--bytes", str(256 << 20)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    line = json.loads([x for x in done.stdout.splitlines() if x.startswith("{")][-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["gpu_launches"] == 3 and line["value"] > 0
    assert set(line["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert line["e2e"]["h2d_bytes_per_step"] == 256 << 20 and line["e2e"]["d2h_bytes_per_step"] == 8
