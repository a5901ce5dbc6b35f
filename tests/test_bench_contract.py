"""bench.py's output contract, as far as it can be checked without a GPU: the reference arm (CPU
statement of the product) prints one JSON line with the agreed keys, and the helpers of the GPU arm
(clock sampling, algorithmic bytes, workload table) behave."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_workloads_match_the_baseline_configurations():
    w = bench.WORKLOADS
    assert (w["gemm8192"]["M"], w["gemm8192"]["transA"], w["gemm8192"]["alpha"], w["gemm8192"]["beta"], w["gemm8192"]["seed"]) == (8192, True, 2.0, 0.5, 2)
    assert (w["gemm4096"]["M"], w["gemm4096"]["transA"], w["gemm4096"]["beta"], w["gemm4096"]["seed"]) == (4096, False, 1.0, 1)
    assert (w["skinny"]["M"], w["skinny"]["N"], w["skinny"]["K"], w["skinny"]["beta"], w["skinny"]["seed"]) == (16384, 128, 8192, 0.0, 3)
    assert (w["sharded"]["M"], w["sharded"]["N"], w["sharded"]["K"], w["sharded"]["seed"]) == (32768, 32768, 16384, 4)
    # algorithmic bytes: 2MK + 2KN + 4MN written (+ 4MN read when beta != 0)
    assert bench.algorithmic_bytes(w["gemm8192"]) == 805306368
    assert bench.algorithmic_bytes(w["gemm4096"]) == 201326592
    assert bench.algorithmic_bytes(w["skinny"]) == 278921216


def test_clock_sampler_parses_nvidia_smi_lines():
    s = bench.ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0, "kill": lambda self: None})()
    s.lines = [(10.0, "0, 1965, 1965, 200.1, Not Active, Not Active, Not Active, Not Active"),   # before the region
               (11.0, "0, 1410, 1965, 998.0, Not Active, Not Active, Not Active, Active"),
               (11.1, "0, 1380, 1965, 1001.2, Not Active, Not Active, Not Active, Active"),
               (11.2, "0, 1395, 1965, 1000.0, Not Active, Not Active, Not Active, Not Active"),
               (11.3, "garbage"),
               (20.0, "0, 1965, 1965, 210.0, Not Active, Not Active, Not Active, Not Active")]    # after it
    out = s.stop(10.9, 11.25)
    assert out == {"sm_mhz": 1395.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}


def test_measured_peaks_fall_back_when_the_file_is_missing(monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    p = bench.measured_peaks()
    assert p["source"] == "fallback" and p["hbm_gbs"] == 6650.0 and p["tf_burst"] == 1590.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6460.5, "bf16_tflops": 1632.1, "bf16_tflops_sustained": 1371.4}))
    p = bench.measured_peaks()
    assert p == {"hbm_gbs": 6460.5, "tf_burst": 1632.1, "tf_sustained": 1371.4, "source": "measured"}


def test_reference_arm_prints_one_contract_line():
    """`bench.py --impl reference` on the smallest workload: one JSON line, metric keys as agreed,
    e2e equal to the line's own value with zero copy bytes, a cpu_baseline that names the port."""
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "gemm4096", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"] == "gemm4096" and d["data"] == "synthetic"
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and "sgemm" in d["cpu_baseline"]["sample"]
