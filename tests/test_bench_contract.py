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


def test_sampled_tile_check_accepts_a_right_slab_and_names_a_wrong_one():
    """bench.check_slab_tiles (the parity leg of every sharded run) on the CPU: a slab computed by the
    oracle passes with all ten tiles looked at; one spoiled element in the slab's last column, or a
    spoiled column of A, fails with the place in the message."""
    import numpy as np
    import torch

    import __graft_entry__ as entry

    oracle, rng = entry.load_oracle(), entry.load_package().rng
    w = dict(M=256, N=384, K=128, transA=False, transB=False, alpha=1.0, beta=1.0, seed=4, b_rsqrt=True, c_dist="normal")
    n0, ns = 128, 256  # the middle of three slabs
    a = rng.matrix(w["seed"], 0, w["M"], w["K"], rng.NORMAL, w["K"] ** -0.5, np.float16)
    b = rng.window(w["seed"], 1, w["K"], 0, w["K"], n0, n0 + ns, rng.NORMAL, w["K"] ** -0.5, np.float16)
    c = rng.window(w["seed"], 2, w["M"], 0, w["M"], n0, n0 + ns, rng.NORMAL, 1.0, np.float32)
    d = oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c)
    D = torch.from_numpy(np.ascontiguousarray(d.T)).reshape(-1)      # column-major slab, as the device holds it
    A = torch.from_numpy(np.ascontiguousarray(a.T)).reshape(-1)
    ok = bench.check_slab_tiles(w, D, n0, ns, A=A)
    assert ok["ok"] and ok["tiles"] == 10 and ok["a_columns"] >= 2 and ok["rel_fro_max"] < 1e-5
    bad = D.clone()
    bad.view(ns, w["M"])[ns - 1, :] += 1.0                           # the slab's last column
    out = bench.check_slab_tiles(w, bad, n0, ns)
    assert not out["ok"] and "tile rows" in out["why"]
    bad_a = A.clone()
    bad_a.view(w["K"], w["M"])[w["K"] - 1, 5] = 0.25
    out = bench.check_slab_tiles(w, D, n0, ns, A=bad_a)
    assert not out["ok"] and "column 127 of A" in out["why"]
    assert bench.check_slab_tiles(w, D, n0, 0)["tiles"] == 0         # a rank without columns has nothing to check


def test_host_threads_are_raised_past_a_one_thread_environment(monkeypatch):
    """torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm sets the BLAS pool itself and reports it."""
    import os

    monkeypatch.setenv("OMP_NUM_THREADS", "1")
    assert bench.use_all_host_threads() == (os.cpu_count() or 1)
