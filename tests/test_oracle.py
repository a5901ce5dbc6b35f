"""The CPU oracle against itself and against the committed fixtures (no GPU).

The reference has no golden vectors for this path (its tests recompute a CPU product from unseeded
rand(), test/device/wmma.jl:102-151 of CUDAnative.jl), so what is pinned here is that the three
statements of the arithmetic -- oracle.c, numpy/OpenBLAS sgemm, and a float64 triple loop -- agree,
and that they still produce the committed outputs for the benchmark configurations' seeds."""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_f16_rounding_is_ieee_round_to_nearest_even(oracle):
    L = oracle.clib()
    rs = np.random.RandomState(0)
    xs = np.concatenate([rs.randn(4000).astype(np.float32) * s for s in (1, 1e-3, 1e-5, 6e-8, 3e-8, 1e3, 7e4)]
                        + [np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                                     1.00048828125, 1.0009765625 + 2.0 ** -12, np.inf, -np.inf], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16)
    got = np.array([L.oracle_f32_to_f16_bits(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, want.view(np.uint16))
    back = np.array([L.oracle_f16_bits_to_f32(int(v)) for v in got], dtype=np.float32)
    assert np.array_equal(back, want.astype(np.float32))


def test_every_f16_bit_pattern_round_trips(oracle):
    L = oracle.clib()
    bits = np.arange(0, 65536, dtype=np.uint32)
    vals = bits.astype(np.uint16).view(np.float16).astype(np.float32)
    finite = np.isfinite(vals)
    for bpat, v in zip(bits[finite][::17], vals[finite][::17]):
        assert L.oracle_f32_to_f16_bits(float(v)) == int(bpat) or (v == 0.0)
        assert L.oracle_f16_bits_to_f32(int(bpat)) == v


@pytest.mark.parametrize("tA,tB", [(False, False), (True, False), (False, True), (True, True)])
def test_sgemm_statement_matches_triple_loop(oracle, pkg, tA, tB):
    rng = pkg.rng
    M, N, K = 37, 29, 111
    a = rng.matrix(5, 0, *((K, M) if tA else (M, K)), rng.NORMAL, K ** -0.5, np.float16)
    b = rng.matrix(5, 1, *((N, K) if tB else (K, N)), rng.NORMAL, 1.0, np.float16)
    c = rng.matrix(5, 2, M, N, rng.UNIFORM, 1.0, np.float32)
    blas = oracle.gemm_ref(tA, tB, 1.5, a, b, -0.25, c)
    loop32 = oracle.gemm_c(tA, tB, 1.5, a.astype(np.float32), b.astype(np.float32), -0.25, c, False)
    loop64 = oracle.gemm_c(tA, tB, 1.5, a.astype(np.float32), b.astype(np.float32), -0.25, c, True)
    for other in (loop32, loop64):
        rel, elem = oracle.errors(blas, other)
        assert rel < 1e-6 and elem < 1e-5
    # beta == 0 ignores C entirely
    d0 = oracle.gemm_ref(tA, tB, 1.0, a, b, 0.0, np.full_like(c, np.nan))
    assert np.all(np.isfinite(d0))


@pytest.mark.parametrize("tA,tB", [(False, False), (True, True)])
def test_float16_accumulating_statements_agree(oracle, pkg, tA, tB):
    """The two statements of the product with a binary16 accumulator (numpy per 16-wide block, C triple
    loop) differ only where the sum inside a block lands within rounding distance of a binary16 tie:
    at most one binary16 ulp on a handful of elements, and both are measurably further from the binary32
    product than one rounding of it is (so they do state binary16 accumulation)."""
    rng = pkg.rng
    M, N, K = 40, 24, 1000  # K is not a multiple of the block
    a = np.abs(rng.matrix(6, 0, *((K, M) if tA else (M, K)), rng.NORMAL, 1.0, np.float16)) * np.float16(0.25)
    b = np.abs(rng.matrix(6, 1, *((N, K) if tB else (K, N)), rng.NORMAL, 1.0, np.float16)) * np.float16(0.25)
    c = rng.matrix(6, 2, M, N, rng.UNIFORM, 1.0, np.float16)
    blocked = oracle.gemm_ref_f16acc(tA, tB, 1.0, a, b, 0.5, c).astype(np.float32)
    loop = oracle.gemm_c_f16acc(tA, tB, 1.0, a.astype(np.float32), b.astype(np.float32), 0.5, c.astype(np.float32))
    ulp = np.spacing(np.abs(loop).astype(np.float16)).astype(np.float32)
    assert np.all(np.abs(blocked - loop) <= ulp) and np.mean(blocked != loop) < 0.05
    ref32 = oracle.gemm_ref(tA, tB, 1.0, a, b, 0.5, c.astype(np.float32))
    once = ref32.astype(np.float16).astype(np.float32)
    assert oracle.errors(loop, ref32)[0] > 1.5 * oracle.errors(once, ref32)[0]
    assert oracle.errors(loop, ref32)[0] < 5e-3


def test_unit_oracle_follows_the_reference_formula(oracle, pkg):
    """alpha * new_a * new_b + beta * new_c with row-major meaning transpose
    (test/device/wmma.jl:233-246), alpha folded into Float16 A, beta into C in C's type."""
    rng = pkg.rng
    a = rng.matrix(9, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
    b = rng.matrix(9, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
    c = rng.matrix(9, 2, 16, 16, rng.UNIFORM, 1.0, np.float16)
    alpha, beta = np.float16(0.3), np.float16(0.7)
    d = oracle.wmma_unit_ref(a, b, c, a_layout=1, b_layout=0, c_layout=1, d_layout=1, d_type=np.float32, alpha=alpha, beta=beta)
    new_a = (alpha * a.T).astype(np.float16).astype(np.float64)   # Float16 product, rounded once
    new_c = (beta * c.T).astype(np.float16).astype(np.float64)
    want = (new_a @ b.astype(np.float64) + new_c).T               # d stored row-major
    assert oracle.unit_close(d, want.astype(np.float32))
    assert np.max(np.abs(d - want)) < 1e-5
    assert not oracle.unit_close(d + 0.1, want.astype(np.float32))  # the tolerance check can fail
    # fill_c(0) case
    d0 = oracle.wmma_unit_ref(a, b, None, d_type=np.float16)
    assert d0.dtype == np.float16 and oracle.unit_close(d0, a.astype(np.float64) @ b.astype(np.float64))


def test_golden_config1_unit(oracle):
    g = np.load(GOLDEN / "config1_unit.npz")
    assert np.array_equal(oracle.wmma_unit_ref(g["a"], g["b"], g["c"]), g["d"])
    assert np.array_equal(oracle.wmma_unit_ref(g["a"], g["b"], g["c"], beta=0.5), g["d_half_c"])
    got = oracle.wmma_unit_ref(g["a"], g["b"], g["c"].astype(np.float16), a_layout=1, b_layout=1, c_layout=1, d_layout=1,
                               d_type=np.float16, alpha=np.float16(0.75), beta=np.float16(0.25))
    assert np.array_equal(got, g["d_rowmajor_f16"])
    # the example's check: a*b + 0.5*c within rtol 0.01 (examples/wmma/high-level.jl:49)
    ref = g["a"].astype(np.float32) @ g["b"].astype(np.float32) + 0.5 * g["c"]
    assert np.allclose(g["d_half_c"], ref, rtol=0.01, atol=1e-6)


def test_golden_config3_small(oracle):
    g = np.load(GOLDEN / "config3_small.npz")
    d = oracle.gemm_ref(True, False, 2.0, g["a"], g["b"], 0.5, g["c"])
    oracle.assert_close(d, g["d"], "sgemm statement vs fixture")   # BLAS blocking may differ between hosts
    oracle.assert_close(d, g["d64"], "sgemm statement vs float64 fixture")
    d64 = oracle.gemm_c(True, False, 2.0, g["a"].astype(np.float32), g["b"].astype(np.float32), 0.5, g["c"], True)
    assert np.array_equal(d64, g["d64"])                            # the C loop is deterministic


def test_golden_bf16_batch(oracle, pkg):
    """bfloat16 operands: the stored results are the C loop with double accumulation on the widened inputs;
    the sgemm statement agrees within the acceptance, both roundings to bfloat16 (oracle and library helper)
    reproduce the stored bits."""
    from cudanative_jl_b200.bfloat16 import round_to_bf16, widen_bf16
    g = np.load(GOLDEN / "bf16_batch_small.npz")
    for i in range(2):
        a, b, c = g[f"a{i}"], g[f"b{i}"], g[f"c{i}"]
        assert a.dtype == np.uint16 and np.array_equal(oracle.bf16_round(oracle.bf16_widen(a)), a)
        d64 = oracle.gemm_c(False, False, 1.25, oracle.bf16_widen(a), oracle.bf16_widen(b), 0.5, c, True)
        assert np.array_equal(d64, g[f"d{i}"])
        oracle.assert_close(oracle.gemm_ref(False, False, 1.25, oracle.bf16_widen(a), oracle.bf16_widen(b), 0.5, c), g[f"d{i}"])
        assert np.array_equal(oracle.bf16_round(g[f"d{i}"]), g[f"d{i}_bf16"])
        assert np.array_equal(round_to_bf16(g[f"d{i}"]), g[f"d{i}_bf16"])
        assert np.array_equal(widen_bf16(a), oracle.bf16_widen(a))


def test_acceptance_thresholds_reject_wrong_answers(oracle):
    g = np.load(GOLDEN / "config3_small.npz")
    bad = g["d"].copy()
    bad[3, 4] += 0.5
    with pytest.raises(AssertionError):
        oracle.assert_close(bad, g["d"])
    with pytest.raises(AssertionError):
        oracle.assert_close(g["d"] * 1.01, g["d"])
