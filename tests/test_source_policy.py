"""Guards on the sources that need no GPU: rules of the shared B200 pool that a later edit could break
without any test noticing until a run is refused or a GPU is lost."""
import re
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SOURCES = [p for pat in ("cudanative.jl_b200/**/*.cu", "cudanative.jl_b200/**/*.cuh", "cudanative.jl_b200/**/*.h",
                         "cudanative.jl_b200/**/*.py", "tests/*.cu", "tests/*.py", "include/*.h", "oracle/*.c", "oracle/*.py",
                         "bench.py", "__graft_entry__.py") for p in ROOT.glob(pat) if p.name != Path(__file__).name]


def test_no_load_carries_a_cluster_multicast_qualifier():
    """One library serves 1 to 8 GPUs, and a multicast TMA load that reaches a peer's memory takes the GPU
    down: the qualifier is allowed on tcgen05.commit's barrier signal only."""
    for path in SOURCES:
        for n, line in enumerate(path.read_text().splitlines(), 1):
            if "multicast::cluster" in line and not line.lstrip().startswith(("//", "*", "#")):
                assert "tcgen05.commit" in line, f"{path.relative_to(ROOT)}:{n}: {line.strip()}"


def test_batched_memcpy_entry_points_are_not_named():
    """Four driver / runtime calls for batches of copies raised GPU faults on this driver; copies are issued one
    cudaMemcpyAsync each.  The names are assembled here so that this file does not contain them either."""
    banned = [a + "Memcpy" + b + "BatchAsync" for a in ("cuda", "cu") for b in ("", "3D")]
    for path in SOURCES:
        text = path.read_text()
        for name in banned:
            assert name not in text, f"{path.relative_to(ROOT)} names {name}"


def test_kernel_waits_are_bounded():
    """Every spin in device code goes through the bounded helpers (mbar_wait / flag_wait with a WaitCtx) or
    carries its own deadline: no `while (true)` / `for (;;)` without a clock in the kernels' sources."""
    for path in ROOT.glob("cudanative.jl_b200/csrc/*.cu*"):
        text = re.sub(r"//.*", "", path.read_text())
        for m in re.finditer(r"(while\s*\(\s*(?:true|1)\s*\)|for\s*\(\s*;\s*;\s*\))", text):
            body = text[m.end():m.end() + 600]
            assert re.search(r"clock64|global_timer_ns|budget", body), f"{path.name}: unbounded loop near offset {m.start()}"
    assert "__trap" not in "".join(p.read_text() for p in ROOT.glob("cudanative.jl_b200/csrc/*.cu*"))


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure: only tests/, the smoke entry and bench.py's CPU legs may touch it."""
    for path in ROOT.glob("cudanative.jl_b200/**/*.py"):
        text = path.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), path
        assert "load_oracle" not in text and "liboracle" not in text, path


def test_fixtures_are_reproducible(tmp_path):
    """tests/golden/make_golden.py regenerates exactly the committed arrays (run on a copy of the script's
    directory so that the committed files are not touched)."""
    import shutil

    work = tmp_path / "tests" / "golden"
    work.mkdir(parents=True)
    shutil.copy(ROOT / "tests" / "golden" / "make_golden.py", work / "make_golden.py")
    script = (work / "make_golden.py").read_text().replace("ROOT = Path(__file__).resolve().parent.parent.parent",
                                                           f"ROOT = Path({str(ROOT)!r})")
    (work / "make_golden.py").write_text(script)
    r = subprocess.run([sys.executable, str(work / "make_golden.py")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    committed = sorted((ROOT / "tests" / "golden").glob("*.npz"))
    assert committed and sorted(p.name for p in work.glob("*.npz")) == [p.name for p in committed]
    for p in committed:
        old, new = np.load(p), np.load(work / p.name)
        assert sorted(old.files) == sorted(new.files), p.name
        for k in old.files:
            # results of the BLAS-backed statement may differ in the last bits between hosts; everything else is exact
            if p.name == "config3_small.npz" and k == "d":
                assert np.allclose(old[k], new[k], rtol=1e-5, atol=1e-6), f"{p.name}:{k}"
            else:
                assert np.array_equal(old[k], new[k]), f"{p.name}:{k}"
