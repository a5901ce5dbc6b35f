"""The counter-based generator: numpy statement == C statement == committed known answers;
the device statement is compared in the GPU test below."""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_known_answers(pkg):
    rng = pkg.rng
    kat = np.load(GOLDEN / "rng_kat.npz")
    idx = np.arange(16, dtype=np.uint64) * np.uint64(1000003)
    for key in kat.files:
        s, m, d = key.split("_")
        got = rng.synth_values(int(s[1:]), int(m[1:]), idx, rng.UNIFORM if d == "u" else rng.NORMAL)
        assert np.array_equal(got, kat[key]), key


@pytest.mark.parametrize("dist", [0, 1, 2])
def test_numpy_and_c_generators_agree(pkg, oracle, dist):
    rng = pkg.rng
    for f16 in (False, True):
        a = oracle.fill(33, 21, 7, 3, dist, 0.37, f16, col0=5)
        b = rng.window(7, 3, 33, 0, 33, 5, 26, dist, 0.37, np.float16 if f16 else np.float32).astype(np.float32)
        assert np.array_equal(a, b)


def test_distributions_and_windows(pkg):
    rng = pkg.rng
    u = rng.matrix(11, 0, 512, 512, rng.UNIFORM)
    n = rng.matrix(11, 1, 512, 512, rng.NORMAL)
    assert -1.0 <= u.min() and u.max() < 1.0 and abs(u.mean()) < 0.01 and abs(u.std() - 3 ** -0.5) < 0.01
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01 and np.all(np.isfinite(n))
    w = rng.window(11, 1, 512, 100, 140, 300, 333, rng.NORMAL, 1.0)
    assert np.array_equal(w, n[100:140, 300:333])  # any window is recomputable in isolation
    assert not np.array_equal(rng.matrix(11, 2, 8, 8, rng.UNIFORM), rng.matrix(12, 2, 8, 8, rng.UNIFORM))


@pytest.mark.gpu
@pytest.mark.parametrize("dist", [0, 1, 2])
def test_device_fill_matches_numpy(pkg, lib, dist):
    from cudanative_jl_b200.array import Array, CuHostArray

    rng = pkg.rng
    rows, cols, ld, col0 = 1000, 300, 1008, 17
    for f16, dt in ((True, np.float16), (False, np.float32)):
        dev = CuHostArray(dt, shape=(ld, cols))
        pkg._lib.check(lib.b200_memset(dev.ptr, 0, dev.nbytes, None), "memset")
        rng.fill_device(dev.ptr, rows, cols, ld, 3, 1, dist, 0.125, f16, col0=col0)
        got = Array(dev)
        want = rng.window(3, 1, rows, 0, rows, col0, col0 + cols, dist, 0.125, dt)
        assert np.array_equal(got[:rows], want)
        assert not got[rows:].any()  # padding rows untouched
