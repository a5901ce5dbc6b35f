"""The 16x16x16 WMMA unit against the CPU oracle: the reference's own test plan
(test/device/wmma.jl of CUDAnative.jl) through this library's entry points."""
import itertools

import numpy as np
import pytest

from cudanative_jl_b200 import rng, wmma
from cudanative_jl_b200.array import Array, CuArray, CuHostArray, pointer
from cudanative_jl_b200.wmma import ColMajor, Config, RowMajor

pytestmark = pytest.mark.gpu

LAYOUTS = [ColMajor, RowMajor]
TYPES = [np.float16, np.float32]


def code(layout):
    return 1 if layout is RowMajor else 0


@pytest.mark.parametrize("mat", ["a", "b", "c"])
@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("ty", TYPES)
def test_load_all_42(mat, layout, ty):
    """test/device/wmma.jl:13-59: load a tile of 42s, every fragment element must be 42."""
    if ty == np.float32 and mat != "c":
        pytest.skip("Float32 is only supported for C")
    conf = Config(16, 16, 16, np.float32)
    dev = CuArray(np.full((16, 16), 42, dtype=ty, order="F"))
    frag = {"a": wmma.load_a, "b": wmma.load_b, "c": wmma.load_c}[mat](pointer(dev), 16, layout, conf)
    x = frag.x
    assert x.shape == (32, 16 if mat != "c" else 8) and np.all(x == ty(42))


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("ty", TYPES)
def test_store_all_42(layout, ty):
    """test/device/wmma.jl:61-100: store a fragment of 42s, all 256 outputs must be 42."""
    conf = Config(16, 16, 16, ty)
    out = CuArray(np.zeros((16, 16), dtype=ty, order="F"))
    frag = wmma.mma(wmma.load_a(pointer(CuArray(np.zeros((16, 16), np.float16, order="F"))), 16, ColMajor, conf),
                    wmma.load_b(pointer(CuArray(np.zeros((16, 16), np.float16, order="F"))), 16, ColMajor, conf),
                    wmma.fill_c(ty(42), conf), conf)  # 0*0 + 42
    wmma.store_d(pointer(out), frag, 16, layout, conf)
    wmma.synchronize()
    assert np.all(Array(out) == ty(42))


def _case(seed, c_type):
    a = rng.matrix(seed, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
    b = rng.matrix(seed, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
    c = rng.matrix(seed, 2, 16, 16, rng.UNIFORM, 1.0, c_type)
    # alpha, beta in [0, 1) like rand(Float16) / rand(c_type) in the reference's test
    alpha = np.float16(abs(float(rng.matrix(seed, 3, 1, 1, rng.UNIFORM, 1.0)[0, 0])))
    beta = c_type(abs(float(rng.matrix(seed, 4, 1, 1, rng.UNIFORM, 1.0)[0, 0])))
    return a, b, c, alpha, beta


SWEEP = list(itertools.product(LAYOUTS, LAYOUTS, LAYOUTS, LAYOUTS, TYPES, TYPES, [True, False]))


@pytest.mark.parametrize("lowering", [wmma.LOWER_WARP, wmma.LOWER_TCGEN05])
def test_fused_unit_128_case_sweep(oracle, lowering):
    """test/device/wmma.jl:188-248: 2^4 layouts x C type x D type x {MAC, MUL}, alpha on the A
    fragment (Float16), beta on the C fragment, rtol = sqrt(eps(Float16))."""
    for i, (al, bl, cl, dl, ct, dt, mac) in enumerate(SWEEP):
        a, b, c, alpha, beta = _case(100 + i, ct)
        d_dev = CuArray(np.zeros((16, 16), dtype=dt, order="F"))
        wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(c) if mac else None, d_dev, a_layout=al, b_layout=bl,
                           c_layout=cl, d_layout=dl, alpha=alpha, beta=beta if mac else None, lowering=lowering)
        wmma.synchronize()
        ref = oracle.wmma_unit_ref(a, b, c if mac else None, a_layout=code(al), b_layout=code(bl), c_layout=code(cl),
                                   d_layout=code(dl), d_type=dt, alpha=alpha, beta=beta if mac else None)
        assert oracle.unit_close(Array(d_dev), ref), f"case {i}: {al.__name__} {bl.__name__} {cl.__name__} {dl.__name__} {ct} {dt} mac={mac}"


def test_fragment_api_128_case_sweep(oracle):
    """The same sweep through load_a / load_b / load_c / fill_c / broadcast / mma / store_d."""
    for i, (al, bl, cl, dl, ct, dt, mac) in enumerate(SWEEP):
        a, b, c, alpha, beta = _case(300 + i, ct)
        conf = Config(16, 16, 16, dt)
        a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
        d_dev = CuArray(np.zeros((16, 16), dtype=dt, order="F"))
        a_frag = wmma.load_a(pointer(a_dev), 16, al, conf)
        b_frag = wmma.load_b(pointer(b_dev), 16, bl, conf)
        c_frag = wmma.load_c(pointer(c_dev), 16, cl, conf) if mac else wmma.fill_c(ct(0), conf)
        a_frag = alpha * a_frag
        c_frag = beta * c_frag
        d_frag = wmma.mma(a_frag, b_frag, c_frag, conf)
        wmma.store_d(pointer(d_dev), d_frag, 16, dl, conf)
        wmma.synchronize()
        ref = oracle.wmma_unit_ref(a, b, c if mac else None, a_layout=code(al), b_layout=code(bl), c_layout=code(cl),
                                   d_layout=code(dl), d_type=dt, alpha=alpha, beta=beta if mac else None)
        assert oracle.unit_close(Array(d_dev), ref), f"case {i}"
        assert a_frag.FS == 16 and c_frag.FS == 8 and d_frag.T == np.dtype(dt)


@pytest.mark.parametrize("lowering", [wmma.LOWER_WARP, wmma.LOWER_TCGEN05])
def test_config1_and_example(oracle, lowering):
    """Benchmark config 1 (uniform[-1,1), seed 0, D = A*B + C) and the reference's example
    (examples/wmma/high-level.jl:49: a*b + 0.5*c with rtol 0.01)."""
    a = rng.matrix(0, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
    b = rng.matrix(0, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
    c = rng.matrix(0, 2, 16, 16, rng.UNIFORM, 1.0, np.float32)
    d_dev = CuHostArray(np.float32, shape=(16, 16))
    wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(c), d_dev, lowering=lowering)
    wmma.synchronize()
    d = Array(d_dev)
    assert oracle.unit_close(d, oracle.wmma_unit_ref(a, b, c))
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "config 1")
    # example: 0.5f0 .* c_frag
    wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(c), d_dev, beta=0.5, lowering=lowering)
    wmma.synchronize()
    ref = a.astype(np.float32) @ b.astype(np.float32) + np.float32(0.5) * c
    assert np.all(np.abs(Array(d_dev) - ref) <= 0.01 * np.maximum(np.abs(ref), np.abs(Array(d_dev))) + 1e-6)


def test_strided_tiles_inside_a_larger_matrix(oracle):
    """load/store with stride > 16: a 16x16 window of a 48x40 matrix."""
    big_a = rng.matrix(7, 0, 48, 40, rng.UNIFORM, 1.0, np.float16)
    big_b = rng.matrix(7, 1, 48, 40, rng.UNIFORM, 1.0, np.float16)
    big_d = np.zeros((48, 40), np.float32, order="F")
    a_dev, b_dev, d_dev = CuArray(big_a), CuArray(big_b), CuArray(big_d)
    conf = Config(16, 16, 16, np.float32)
    a_frag = wmma.load_a(pointer(a_dev) + (16 + 8 * 48), 48, ColMajor, conf)   # rows 16.., cols 8..
    b_frag = wmma.load_b(pointer(b_dev) + (32 + 16 * 48), 48, ColMajor, conf)  # rows 32.., cols 16..
    d_frag = wmma.mma(a_frag, b_frag, wmma.fill_c(np.float32(0), conf), conf)
    wmma.store_d(pointer(d_dev) + (8 + 24 * 48), d_frag, 48, ColMajor, conf)
    wmma.synchronize()
    out = Array(d_dev)
    ref = big_a[16:32, 8:24].astype(np.float32) @ big_b[32:48, 16:32].astype(np.float32)
    assert oracle.unit_close(out[8:24, 24:40], ref)
    out[8:24, 24:40] = 0
    assert not out.any(), "store_d wrote outside its 16x16 window"
