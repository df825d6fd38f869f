"""The benchmark's reference arm needs no GPU (it times the CPU oracle), so its JSON line can be checked here:
one line, the keys the benchmark contract names, values of the right kind."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*flags, env=None):
    e = dict(os.environ)
    e.update(env or {})
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True,
                         timeout=600, env=e, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line():
    d = run_bench("--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "0", "--workload", "c3n8")
    assert d["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["steps"] == 1 and d["warmup"] == 0 and d["n_gpus"] == 1
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert isinstance(d["config"]["workload"], str) and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and isinstance(cb["sample"], str)
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["value"] > 0 and d["ms_per_step"] > 0


def test_reference_arm_other_ranks_print_nothing():
    e = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0", "--workload", "c3n8"], capture_output=True, text=True, timeout=600, env=e, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert not [l for l in out.stdout.splitlines() if l.startswith("{")]


def test_roofline_and_sustained_entries_are_self_consistent():
    """The roofline arithmetic of the benchmark line: achieved = algorithmic units / time, fractions against the
    measured and the nominal peak, FP8 peak = twice the BF16 figure."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class W:
        units = 962.072674304e9
    pk = {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0, "source": "measured"}
    r = bench.roofline("c2", W, 0.35, pk)
    assert r["bound"] == "tensor" and r["peak"] == 3200.0 and r["nominal_peak"] == 4500.0
    assert abs(r["achieved"] - 962.072674304 / 0.35) < 1e-6 and abs(r["frac"] - r["achieved"] / 3200.0) < 1e-12
    assert r["traffic"] == bench.NCU_TRAFFIC_BYTES["c2"] and r["algorithmic_units_per_launch"] == W.units
    s = bench.sustained_entry("c2", W, 0.4, {"sm_mhz": 1450, "reasons": ["sw_power_cap"]}, 5000, pk)
    assert s["peak"] == 2800.0 and abs(s["ms_times_mhz"] - 580.0) < 1e-9 and abs(s["frac"] - s["achieved"] / 2800.0) < 1e-12
    W.units = 67.1e6
    g = bench.roofline("c3n1", W, 0.016, pk)
    assert g["bound"] == "hbm" and g["peak"] == 6500.0 and g["nominal_peak"] == 8000.0 and g["unit"] == "GB/s"
    c4 = bench.roofline("c4", W, 1.0, pk)
    assert c4["peak"] == 1600.0 and c4["nominal_peak"] == 2250.0
