"""Parity of the tiled GEMM (through the C ABI) with the CPU oracle.

Tolerances are the benchmark specification's: relative Frobenius error <= 1e-3 and |D - ref| <= 1e-2 * (|ref| + 1)
elementwise, against float32 sgemm on the Float16-rounded inputs (oracle.assert_close)."""
import numpy as np
import pytest

from cudanative_jl_b200 import _lib, rng
from cudanative_jl_b200.array import Array, CuArray, CuHostArray
from helpers import operands, padded, run_gemm

pytestmark = pytest.mark.gpu

LAYOUTS = [(False, False), (True, False), (False, True), (True, True)]


def force(handle, kernel=_lib.KERNEL_TCGEN05, tile_n=0, pair=0, split_k=0, max_ctas=0):
    handle.set_option(_lib.OPT_FORCE_KERNEL, kernel)
    handle.set_option(_lib.OPT_TILE_N, tile_n)
    handle.set_option(_lib.OPT_CTA_PAIR, pair)
    handle.set_option(_lib.OPT_SPLIT_K, split_k)
    handle.set_option(_lib.OPT_MAX_CTAS, max_ctas)


def test_simple_kernel_matches_oracle(handle, oracle):
    """The plain kernel is the on-device yardstick for the big cases below: pin it first."""
    force(handle, _lib.KERNEL_SIMPLE)
    for (tA, tB) in LAYOUTS:
        M, N, K = 150, 70, 99
        a, b, c = operands(M, N, K, tA, tB, seed=11)
        d = run_gemm(handle, tA, tB, M, N, K, 1.5, a, b, -0.5, c)
        oracle.assert_close(d, oracle.gemm_ref(tA, tB, 1.5, a, b, -0.5, c), f"simple tA={tA} tB={tB}")
        ref64 = oracle.gemm_c(tA, tB, 1.5, a.astype(np.float32), b.astype(np.float32), -0.5, c, True)
        oracle.assert_close(d, ref64, "simple vs double accumulation")


@pytest.mark.parametrize("tA,tB", LAYOUTS)
@pytest.mark.parametrize("tile_n,pair", [(256, 1), (128, 1), (64, 1), (256, 2), (128, 2)])
def test_one_tile_one_kblock(handle, oracle, tA, tB, tile_n, pair):
    """Smallest case that exercises descriptors and TMEM layout: one tile, K = 64."""
    if tB and (tile_n // pair) % 64:
        pytest.skip("row-major B needs 64 tile columns per CTA")
    force(handle, tile_n=tile_n, pair=pair)
    M, N, K = 128 * pair, tile_n, 64
    a, b, c = operands(M, N, K, tA, tB, seed=21)
    d = run_gemm(handle, tA, tB, M, N, K, 1.0, a, b, 1.0, c)
    oracle.assert_close(d, oracle.gemm_ref(tA, tB, 1.0, a, b, 1.0, c), f"one tile {tile_n}x{pair}")
    info = handle.last_launch()
    assert info["kernel"] == _lib.KERNEL_TCGEN05 and info["tile_n"] == tile_n and info["cta_pair"] == pair


@pytest.mark.parametrize("tA,tB", LAYOUTS)
@pytest.mark.parametrize("tile_n,pair", [(256, 1), (128, 1), (64, 1), (256, 2), (128, 2)])
def test_ragged_multi_tile(handle, oracle, tA, tB, tile_n, pair):
    """Several tiles per CTA pipeline, ragged M / N / K edges, alpha and beta both active."""
    if tB and (tile_n // pair) % 64:
        pytest.skip("row-major B needs 64 tile columns per CTA")
    force(handle, tile_n=tile_n, pair=pair, max_ctas=6)  # few CTAs: each walks many tiles
    M, N, K = 712, 664, 1000
    a, b, c = operands(M, N, K, tA, tB, seed=31)
    d = run_gemm(handle, tA, tB, M, N, K, 2.0, a, b, 0.5, c)
    oracle.assert_close(d, oracle.gemm_ref(tA, tB, 2.0, a, b, 0.5, c), f"ragged {tile_n}x{pair}")


@pytest.mark.parametrize("M,N,K,tile_n,pair", [(300, 300, 192, 256, 2), (300, 300, 192, 128, 2), (64, 48, 64, 64, 1),
                                               (8, 8, 8, 64, 1), (132, 257, 65 * 8, 256, 1)])
def test_edge_tiles(handle, oracle, M, N, K, tile_n, pair):
    """Tiles that hang over the bottom / right edge: in 2-CTA tiles the second CTA may own no valid
    row at all (M = 300: rows 384..511 of the second tile do not exist)."""
    force(handle, tile_n=tile_n, pair=pair)
    for (tA, tB) in LAYOUTS:
        if tB and (tile_n // pair) % 64:
            continue
        # leading dimensions rounded up to what TMA can address, plus canary rows below D
        a, b, c = operands(M, N, K, tA, tB, seed=77)
        lda = -(-a.shape[0] // 8) * 8
        ldb = -(-b.shape[0] // 8) * 8
        d = run_gemm(handle, tA, tB, M, N, K, 0.5, padded(a, lda, 0), padded(b, ldb, 0), 2.0, padded(c, M + 4, 0), ldd=M + 8)
        oracle.assert_close(d[:M], oracle.gemm_ref(tA, tB, 0.5, a, b, 2.0, c), f"edge {M}x{N}x{K} tA={tA} tB={tB}")
        assert np.all(d[M:] == np.float32(-7.25)), "rows beyond M were written"


@pytest.mark.parametrize("M", [129, 130, 135, 5, 3])
def test_row_counts_that_are_not_multiples_of_four(handle, oracle, M):
    """Bulk stores are 16-byte granular, so the tensor-core kernel takes M - M % 4 rows and the plain
    kernel the rest: the result is complete and nothing below row M is touched."""
    force(handle, _lib.KERNEL_AUTO)
    N, K = 200, 136
    for (tA, tB) in LAYOUTS:
        a, b, c = operands(M, N, K, tA, tB, seed=78)
        lda = -(-a.shape[0] // 8) * 8
        ldb = -(-b.shape[0] // 8) * 8
        ld = -(-M // 4) * 4 + 4
        d = run_gemm(handle, tA, tB, M, N, K, 1.5, padded(a, lda, 0), padded(b, ldb, 0), -1.0, padded(c, ld, 9.0), ldd=ld)
        oracle.assert_close(d[:M], oracle.gemm_ref(tA, tB, 1.5, a, b, -1.0, c), f"M={M} tA={tA} tB={tB}")
        assert np.all(d[M:] == np.float32(-7.25)), "rows beyond M were written"
        if M > 4:
            assert handle.last_launch()["kernel"] == _lib.KERNEL_TCGEN05
    force(handle, _lib.KERNEL_TCGEN05)
    with pytest.raises(Exception, match="multiple of 4"):
        a, b, c = operands(130, N, K, False, False, seed=78)
        run_gemm(handle, False, False, 130, N, K, 1.0, padded(a, 136, 0), b, 0.0, None, ldd=136)


@pytest.mark.parametrize("K", [100, 101, 65, 7])
def test_k_tail_is_zero_filled_not_read(handle, oracle, K):
    """K need not be a multiple of anything: the loads fill elements beyond K with zeros one element at
    a time, so NaNs sitting in the leading-dimension padding right behind the last k never reach D."""
    force(handle)
    M, N = 128, 192
    for (tA, tB) in LAYOUTS:
        a, b, c = operands(M, N, K, tA, tB, seed=79)
        lda = -(-a.shape[0] // 8) * 8 + 8
        ldb = -(-b.shape[0] // 8) * 8 + 8
        d = run_gemm(handle, tA, tB, M, N, K, 1.0, padded(a, lda, np.nan), padded(b, ldb, np.nan), 0.0, None)
        oracle.assert_close(d, oracle.gemm_ref(tA, tB, 1.0, a, b, 0.0, None), f"K={K} tA={tA} tB={tB}")


@pytest.mark.parametrize("tile_n", [128, 256])
def test_pair_many_stage_wraps(handle, oracle, tile_n):
    """2-CTA tiles with a K loop far longer than the stage ring and several tiles per pair."""
    force(handle, tile_n=tile_n, pair=2, max_ctas=4)
    M, N, K = 1024, 768, 2048
    a, b, c = operands(M, N, K, True, False, seed=41)
    d = run_gemm(handle, True, False, M, N, K, 1.0, a, b, 1.0, c)
    oracle.assert_close(d, oracle.gemm_ref(True, False, 1.0, a, b, 1.0, c), f"pair tile_n={tile_n}")


def test_beta_zero_never_reads_c(handle, oracle):
    """beta == 0: C may be NULL (fill_c(0) case) and NaNs in a passed C must not leak."""
    force(handle)
    M, N, K = 256, 384, 320
    a, b, c = operands(M, N, K, False, False, seed=51)
    ref = oracle.gemm_ref(False, False, 3.0, a, b, 0.0, None)
    oracle.assert_close(run_gemm(handle, False, False, M, N, K, 3.0, a, b, 0.0, None), ref, "C = NULL")
    poison = np.full_like(c, np.nan)
    oracle.assert_close(run_gemm(handle, False, False, M, N, K, 3.0, a, b, 0.0, poison), ref, "C = NaN")


def test_d_aliases_c_and_padding_untouched(handle, oracle):
    """In-place update (D is C) with ldd > M: rows M..ldd-1 must keep their canary values."""
    force(handle)
    M, N, K, ld = 200, 136, 192, 208
    a, b, c = operands(M, N, K, False, False, seed=61)
    cd = padded(c, ld, fill=np.float32(123.5))
    cd_dev = CuArray(cd)
    a_dev, b_dev = CuArray(a), CuArray(b)
    handle.gemm(False, False, M, N, K, 1.0, a_dev, M, b_dev, K, 1.0, cd_dev, ld, cd_dev, ld)
    out = Array(cd_dev)
    assert handle.device_status()[0] == 0
    oracle.assert_close(out[:M], oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "in place")
    assert np.all(out[M:] == np.float32(123.5)), "padding rows were overwritten"


@pytest.mark.parametrize("split_k", [2, 3, 8])
def test_split_k(handle, oracle, split_k):
    force(handle, tile_n=128, pair=1, split_k=split_k)
    M, N, K = 384, 128, 1536 + 40
    a, b, c = operands(M, N, K, False, False, seed=71)
    d = run_gemm(handle, False, False, M, N, K, 1.25, a, b, 0.75, c)
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.25, a, b, 0.75, c), f"split_k={split_k}")
    # slices are whole 64-wide k-blocks and none may be empty: 25 k-blocks split 8 ways gives 7
    assert handle.last_launch()["split_k"] == {2: 2, 3: 3, 8: 7}[split_k]


@pytest.mark.parametrize("tA,tB", LAYOUTS)
def test_split_k_with_two_cta_tiles(handle, oracle, tA, tB):
    """k-slices on 2-CTA 256-wide tiles, ragged in every dimension, several tiles per cluster."""
    force(handle, tile_n=256, pair=2, split_k=4, max_ctas=8)
    M, N, K = 520, 600, 1100
    a, b, c = operands(M, N, K, tA, tB, seed=72)
    lda, ldb = -(-a.shape[0] // 8) * 8, -(-b.shape[0] // 8) * 8
    d = run_gemm(handle, tA, tB, M, N, K, 0.5, padded(a, lda, 0), padded(b, ldb, 0), 1.5, c)
    oracle.assert_close(d, oracle.gemm_ref(tA, tB, 0.5, a, b, 1.5, c), f"pair split-K tA={tA} tB={tB}")
    info = handle.last_launch()
    assert info["split_k"] == 4 and info["cta_pair"] == 2


def test_unaligned_and_empty_shapes_take_the_simple_kernel(handle, oracle):
    force(handle, _lib.KERNEL_AUTO)
    # lda = 45 is not a multiple of 8: TMA cannot address it
    M, N, K = 45, 37, 29
    a, b, c = operands(M, N, K, False, False, seed=81)
    d = run_gemm(handle, False, False, M, N, K, 1.0, a, b, 1.0, c)
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "unaligned")
    assert handle.last_launch()["kernel"] == _lib.KERNEL_SIMPLE
    # K == 0: D = beta * C
    c0 = rng.matrix(82, 2, 64, 32, rng.UNIFORM, 1.0, np.float32)
    a0 = np.zeros((64, 0), np.float16, order="F")
    b0 = np.zeros((0, 32), np.float16, order="F")
    d0_dev, c0_dev = CuHostArray(np.float32, shape=(64, 32)), CuArray(c0)
    handle.gemm(False, False, 64, 32, 0, 1.0, CuArray(np.zeros((1, 1), np.float16)), 64, CuArray(np.zeros((1, 1), np.float16)), 1,
                0.5, c0_dev, 64, d0_dev, 64)
    assert np.array_equal(Array(d0_dev), np.float32(0.5) * c0)
    # M == 0 or N == 0: nothing to do, no error
    handle.gemm(False, False, 0, 32, 16, 1.0, None, 1, None, 16, 0.0, None, 1, None, 1)
    # forcing the tcgen05 kernel on an unaligned problem is refused loudly
    force(handle, _lib.KERNEL_TCGEN05)
    with pytest.raises(Exception, match="not eligible"):
        run_gemm(handle, False, False, M, N, K, 1.0, a, b, 1.0, c)


def test_argument_validation(handle):
    with pytest.raises(Exception, match="lda smaller"):
        handle.gemm(False, False, 64, 64, 64, 1.0, 256, 8, 256, 64, 0.0, None, 64, 256, 64)
    with pytest.raises(Exception, match="C is null"):
        handle.gemm(False, False, 64, 64, 64, 1.0, 256, 64, 256, 64, 1.0, None, 64, 256, 64)
    with pytest.raises(Exception, match="negative"):
        handle.gemm(False, False, -1, 64, 64, 1.0, 256, 64, 256, 64, 0.0, None, 64, 256, 64)


def test_deterministic(handle):
    force(handle, _lib.KERNEL_AUTO)
    M, N, K = 1024, 1024, 1024
    a, b, c = operands(M, N, K, False, False, seed=91)
    d1 = run_gemm(handle, False, False, M, N, K, 1.0, a, b, 1.0, c)
    d2 = run_gemm(handle, False, False, M, N, K, 1.0, a, b, 1.0, c)
    assert np.array_equal(d1, d2)


def test_back_to_back_launches_with_and_without_programmatic_launch(handle, oracle):
    """B200_OPT_PDL: the kernel's set-up may overlap the tail of the kernel before it; its global accesses
    may not.  Ten dependent launches in a row (each reads the D of the one before as its C) give the same
    bits with the option on (default) and off, and the right numbers."""
    force(handle, _lib.KERNEL_TCGEN05)
    M, N, K = 512, 768, 256
    a, b, c = operands(M, N, K, True, False, seed=92)
    a_dev, b_dev = CuArray(a), CuArray(b)
    assert handle.get_option(_lib.OPT_PDL) == 1
    out = {}
    for pdl in (1, 0):
        handle.set_option(_lib.OPT_PDL, pdl)
        d_dev = CuArray(c)
        for _ in range(10):  # D <- 0.5 * A B + 0.5 * D, in place
            handle.gemm(True, False, M, N, K, 0.5, a_dev, K, b_dev, K, 0.5, d_dev, M, d_dev, M)
        _lib.check(_lib.lib().b200_stream_sync(None), "sync")
        assert handle.device_status()[0] == 0
        out[pdl] = Array(d_dev)
    handle.set_option(_lib.OPT_PDL, 1)
    assert np.array_equal(out[0], out[1])
    ref = c
    for _ in range(10):
        ref = oracle.gemm_ref(True, False, 0.5, a, b, 0.5, ref)
    oracle.assert_close(out[1], ref, "ten dependent launches")


def test_config2_4096_cubed(handle, oracle):
    """Benchmark config 2: M=N=K=4096, A, B column-major normal/sqrt(K), C normal, alpha=beta=1, seed 1."""
    force(handle, _lib.KERNEL_AUTO)
    n = 4096
    a = rng.matrix(1, 0, n, n, rng.NORMAL, n ** -0.5, np.float16)
    b = rng.matrix(1, 1, n, n, rng.NORMAL, n ** -0.5, np.float16)
    c = rng.matrix(1, 2, n, n, rng.NORMAL, 1.0, np.float32)
    d = run_gemm(handle, False, False, n, n, n, 1.0, a, b, 1.0, c)
    assert handle.last_launch()["kernel"] == _lib.KERNEL_TCGEN05
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "config 2")


def test_config4_skinny(handle, oracle):
    """Benchmark config 4: M=16384, N=128, K=8192, A column-major normal/sqrt(K), B normal, C zeros, beta=0, seed 3."""
    force(handle, _lib.KERNEL_AUTO)
    M, N, K = 16384, 128, 8192
    a = rng.matrix(3, 0, M, K, rng.NORMAL, K ** -0.5, np.float16)
    b = rng.matrix(3, 1, K, N, rng.NORMAL, 1.0, np.float16)
    d = run_gemm(handle, False, False, M, N, K, 1.0, a, b, 0.0, None)
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.0, a, b, 0.0, None), "config 4")


def _device_problem(handle, M, N, K, seed, transA, c_dist):
    """Operands generated on the device (too big to build on the host quickly)."""
    L = _lib.lib()
    a = CuHostArray(np.float16, shape=((K, M) if transA else (M, K)))
    b = CuHostArray(np.float16, shape=(K, N))
    c = CuHostArray(np.float32, shape=(M, N))
    rng.fill_device(a.ptr, a.shape[0], a.shape[1], a.shape[0], seed, 0, rng.NORMAL, K ** -0.5, True)
    rng.fill_device(b.ptr, K, N, K, seed, 1, rng.NORMAL, K ** -0.5, True)
    rng.fill_device(c.ptr, M, N, M, seed, 2, c_dist, 1.0, False)
    return a, b, c


def test_config3_8192_cubed_properties(handle, oracle):
    """Benchmark config 3 at full size: A row-major, B column-major, alpha=2, beta=0.5, seed 2.
    Checked three ways without a full CPU product: (1) against the independent plain kernel on
    the device, elementwise over the whole matrix; (2) sampled 128x128 tiles against the CPU
    oracle with operands regenerated from the counter-based generator; (3) linearity in alpha."""
    n = 8192
    a, b, c = _device_problem(handle, n, n, n, 2, True, rng.UNIFORM)
    d = CuHostArray(np.float32, shape=(n, n))
    force(handle, _lib.KERNEL_AUTO)
    handle.gemm(True, False, n, n, n, 2.0, a, n, b, n, 0.5, c, n, d, n)
    d_host = Array(d)
    assert handle.device_status()[0] == 0
    assert handle.last_launch()["kernel"] == _lib.KERNEL_TCGEN05
    # (2) sampled tiles vs CPU oracle
    picks = [(0, 0), (n - 128, n - 128), (3968, 4224), (128 * 17, 128 * 45), (128 * 63, 0)]
    for (m0, n0) in picks:
        a_win = rng.window(2, 0, n, 0, n, m0, m0 + 128, rng.NORMAL, n ** -0.5, np.float16)  # stored K x M
        b_win = rng.window(2, 1, n, 0, n, n0, n0 + 128, rng.NORMAL, n ** -0.5, np.float16)
        c_win = rng.window(2, 2, n, m0, m0 + 128, n0, n0 + 128, rng.UNIFORM, 1.0, np.float32)
        ref = oracle.gemm_ref(True, False, 2.0, a_win, b_win, 0.5, c_win)
        oracle.assert_close(d_host[m0:m0 + 128, n0:n0 + 128], ref, f"config 3 tile ({m0},{n0})")
    # (1) whole matrix vs the plain kernel
    d2 = CuHostArray(np.float32, shape=(n, n))
    force(handle, _lib.KERNEL_SIMPLE)
    handle.gemm(True, False, n, n, n, 2.0, a, n, b, n, 0.5, c, n, d2, n)
    oracle.assert_close(d_host, Array(d2), "config 3 vs plain kernel")
    # (3) linearity: D(alpha=4, beta=0) == 2 * D(alpha=2, beta=0) exactly (powers of two)
    force(handle, _lib.KERNEL_AUTO)
    handle.gemm(True, False, n, n, n, 2.0, a, n, b, n, 0.0, None, n, d, n)
    handle.gemm(True, False, n, n, n, 4.0, a, n, b, n, 0.0, None, n, d2, n)
    assert np.array_equal(Array(d2), np.float32(2.0) * Array(d))


@pytest.mark.parametrize("c_type,d_type", [(np.float16, np.float16), (np.float16, np.float32), (np.float32, np.float16)])
@pytest.mark.parametrize("kernel,split_k", [(_lib.KERNEL_TCGEN05, 0), (_lib.KERNEL_TCGEN05, 3), (_lib.KERNEL_SIMPLE, 0)])
def test_float16_c_and_d(handle, oracle, c_type, d_type, kernel, split_k):
    """The reference's other three accumulator / result type combinations (wmma.jl:23-30; swept by
    test/device/wmma.jl:188-248) on whole matrices: Float16 C is widened on load, Float16 D rounded once."""
    from cudanative_jl_b200.gemm import gemm_f16f32
    force(handle, kernel, split_k=split_k)
    M, N, K = 392, 264, 520
    for (tA, tB) in LAYOUTS:
        a, b, c32 = operands(M, N, K, tA, tB, seed=88)
        c = c32.astype(c_type)
        d_dev = CuArray(np.full((M, N), -3.0, dtype=d_type, order="F"))
        gemm_f16f32(handle, d_dev, CuArray(a), CuArray(b), CuArray(c), alpha=1.5, beta=0.5, transA=tA, transB=tB)
        d = Array(d_dev)
        assert handle.device_status()[0] == 0 and d.dtype == d_type
        ref = oracle.gemm_ref(tA, tB, 1.5, a, b, 0.5, c.astype(np.float32))
        if d_type == np.float16:  # one rounding to nearest even on the way out, nothing more
            assert np.max(np.abs(d.astype(np.float32) - ref.astype(np.float16).astype(np.float32))
                          / (np.abs(ref) + 1)) <= 2.0 ** -10
        oracle.assert_close(d.astype(np.float32), ref, f"C {c_type.__name__} D {d_type.__name__} tA={tA} tB={tB}")
    assert handle.last_launch()["kernel"] == kernel
    # beta == 0 with a Float16 D and no C
    a, b, _ = operands(M, N, K, False, False, seed=89)
    d_dev = CuArray(np.zeros((M, N), dtype=np.float16, order="F"))
    gemm_f16f32(handle, d_dev, CuArray(a), CuArray(b), alpha=1.0)
    oracle.assert_close(Array(d_dev).astype(np.float32), oracle.gemm_ref(False, False, 1.0, a, b, 0.0, None), "f16 D, no C")


def test_float16_d_with_ragged_rows(handle, oracle):
    """Float16 D: 16-byte store chunks hold 8 rows; M % 8 rows go to the plain kernel and the rows
    below M stay untouched."""
    force(handle, _lib.KERNEL_AUTO)
    M, N, K, ld = 267, 136, 128, 280
    a, b, c32 = operands(M, N, K, False, False, seed=90)
    c = padded(c32.astype(np.float16), ld, 0)
    d_dev = CuArray(np.full((ld, N), 7.5, dtype=np.float16, order="F"))
    handle.gemm_typed(False, False, M, N, K, 1.0, CuArray(padded(a, 272, 0)), 272, CuArray(b), K, 1.0, CuArray(c), ld, np.float16,
                      d_dev, ld, np.float16)
    d = Array(d_dev)
    oracle.assert_close(d[:M].astype(np.float32), oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c32.astype(np.float16).astype(np.float32)),
                        "ragged f16 D")
    assert np.all(d[M:] == np.float16(7.5))


def _streams(lib, n):
    import ctypes as C
    out = []
    for _ in range(n):
        s = C.c_void_p()
        _lib.check(lib.b200_stream_create(C.byref(s)), "stream_create")
        out.append(s)
    return out


def test_gated_gemm_waits_for_panel_flags(handle, oracle, lib):
    """The gated GEMM reads a K panel of A only after its flag word is set.  Here the flags are
    written from a second stream by stream memory operations while the kernel is already running,
    with the panel's data uploaded just before its flag: a panel read early would see zeros."""
    import time
    M, N, K, panel_k = 512, 768, 1024, 256
    a, b, c = operands(M, N, K, False, False, seed=111)
    a_dev = CuArray(np.zeros_like(a))              # A starts empty on the device
    b_dev, c_dev = CuArray(b), CuArray(c)
    d_dev = CuHostArray(np.float32, shape=(M, N))
    flags = CuArray(np.zeros(32, dtype=np.float32))  # 32 zero words
    s_gemm, s_copy = _streams(lib, 2)
    force(handle, _lib.KERNEL_AUTO)
    handle.set_option(_lib.OPT_WAIT_BUDGET_NS, 1_000_000_000)
    handle.gemm_gated(False, False, M, N, K, 1.5, a_dev, M, b_dev, K, 0.5, c_dev, M, d_dev, M, flags, panel_k, stream=s_gemm)
    for j in range(K // panel_k):                  # the kernel is spinning on flag j by now
        time.sleep(0.002)
        cols = np.ascontiguousarray(a[:, j * panel_k:(j + 1) * panel_k].T).T  # Fortran slice, contiguous
        _lib.check(lib.b200_memcpy_h2d(a_dev.ptr + 2 * j * panel_k * M, cols.ctypes.data, cols.nbytes, s_copy), "upload panel")
        _lib.check(lib.b200_stream_write_u32(s_copy, flags.ptr + 4 * j, 1), "open gate")
        _lib.check(lib.b200_stream_sync(s_copy), "sync")  # `cols` must outlive the copy
    _lib.check(lib.b200_stream_sync(s_gemm), "sync")
    assert handle.device_status()[0] == 0
    oracle.assert_close(Array(d_dev), oracle.gemm_ref(False, False, 1.5, a, b, 0.5, c), "gated gemm")
    # flags already set: behaves like the plain entry point (bit-identical)
    d2 = CuHostArray(np.float32, shape=(M, N))
    handle.gemm_gated(False, False, M, N, K, 1.5, a_dev, M, b_dev, K, 0.5, c_dev, M, d2, M, flags, panel_k, stream=s_gemm)
    _lib.check(lib.b200_stream_sync(s_gemm), "sync")
    assert np.array_equal(Array(d2), Array(d_dev))
    # a gate that never opens: the wait runs out, is reported, and the context stays usable
    _lib.check(lib.b200_memset(flags.ptr, 0, 128, s_copy), "memset")
    _lib.check(lib.b200_stream_sync(s_copy), "sync")
    handle.set_option(_lib.OPT_WAIT_BUDGET_NS, 5_000_000)
    handle.gemm_gated(False, False, M, N, K, 1.5, a_dev, M, b_dev, K, 0.5, c_dev, M, d2, M, flags, panel_k, stream=s_gemm)
    _lib.check(lib.b200_stream_sync(s_gemm), "sync")
    code, _, _ = handle.device_status()
    # the producer's gate wait (108) and the waits of the roles it starves (MMA 102, epilogue 104)
    # run out together; whichever reports first wins the status word
    assert code in (108, 102, 104)
    handle.set_option(_lib.OPT_WAIT_BUDGET_NS, 200_000_000)
    d3 = run_gemm(handle, False, False, M, N, K, 1.5, a, b, 0.5, c)
    oracle.assert_close(d3, oracle.gemm_ref(False, False, 1.5, a, b, 0.5, c), "after a closed gate")
    for s in (s_gemm, s_copy):
        lib.b200_stream_destroy(s)
    with pytest.raises(Exception, match="multiple of 64"):
        handle.gemm_gated(False, False, M, N, K, 1.0, a_dev, M, b_dev, K, 0.0, None, M, d2, M, flags, 100)


def test_bounded_wait_reports_and_context_survives(handle, oracle):
    """A wait nothing satisfies runs out after its budget, the status word names it, and the
    context is still usable afterwards."""
    L = _lib.lib()
    _lib.check(L.b200_selftest_bounded_wait(handle._h, None, 2_000_000), "selftest")
    _lib.check(L.b200_stream_sync(None), "sync")
    code, block, _ = handle.device_status()
    assert code == 107 and block == 0
    assert handle.device_status()[0] == 0  # reading clears it
    force(handle, _lib.KERNEL_AUTO)
    a, b, c = operands(128, 128, 128, False, False, seed=5)
    d = run_gemm(handle, False, False, 128, 128, 128, 1.0, a, b, 1.0, c)
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "after timeout")


@pytest.mark.parametrize("tA,tB,M,N,K", [(False, False, 256, 256, 512), (True, False, 512, 384, 2048), (False, True, 384, 512, 1000)])
def test_float16_accumulation_for_whole_matrices(handle, oracle, tA, tB, M, N, K):
    """B200_OPT_F16_ACCUMULATE: Config{16,16,16,Float16} with a Float16 accumulator (the .f16.f16 mma
    variants, src/device/cuda/wmma.jl:222-257) for whole matrices -- the tensor cores accumulate in
    binary16.  Inputs are non-negative so that the running sums grow and binary16 accumulation shows.
    Tolerances, written out: against the binary32 product every element within sqrt(eps(Float16)) (the
    reference's rtol, test/device/wmma.jl:243-246) of |ref| + rms(ref); against the blockwise binary16
    statement of the oracle a relative Frobenius error of at most 5e-3; and the result must be further
    from the binary32 product than the default (binary32 accumulation, rounded once) is."""
    force(handle, _lib.KERNEL_TCGEN05)
    a, b, c32 = operands(M, N, K, tA, tB, seed=77, a_scale=1.0)
    a, b = np.abs(a) * np.float16(0.25), np.abs(b) * np.float16(0.25)
    c = np.asfortranarray(c32.astype(np.float16))
    a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
    ref32 = oracle.gemm_ref(tA, tB, 1.0, a, b, 0.5, c)
    out = {}
    for mode in (0, 1):
        handle.set_option(_lib.OPT_F16_ACCUMULATE, mode)
        d_dev = CuHostArray(np.float16, shape=(M, N))
        handle.gemm_typed(tA, tB, M, N, K, 1.0, a_dev, a.shape[0], b_dev, b.shape[0], 0.5, c_dev, M, np.float16, d_dev, M, np.float16)
        _lib.check(_lib.lib().b200_stream_sync(None), "sync")
        assert handle.device_status()[0] == 0
        out[mode] = Array(d_dev).astype(np.float32)
    handle.set_option(_lib.OPT_F16_ACCUMULATE, 0)
    rms = float(np.sqrt(np.mean(ref32.astype(np.float64) ** 2)))
    assert np.all(np.abs(out[1] - ref32) <= oracle.UNIT_RTOL * (np.abs(ref32) + rms)), "outside the reference's rtol"
    ref16 = oracle.gemm_ref_f16acc(tA, tB, 1.0, a, b, 0.5, c).astype(np.float32)
    rel16, _ = oracle.errors(out[1], ref16)
    assert rel16 <= 5e-3, f"relative Frobenius error {rel16:.2e} against the binary16-accumulating oracle"
    err_f32acc, _ = oracle.errors(out[0], ref32)
    err_f16acc, _ = oracle.errors(out[1], ref32)
    assert err_f32acc <= 4e-4 and err_f16acc > 1.5 * err_f32acc, (err_f32acc, err_f16acc)
    # a Float32 C or D keeps binary32 accumulation whatever the option says; shapes the TMA kernel cannot take are refused
    from cudanative_jl_b200 import B200Error
    handle.set_option(_lib.OPT_F16_ACCUMULATE, 1)
    force(handle, _lib.KERNEL_AUTO)
    with pytest.raises(B200Error, match="Float16 accumulation needs the tcgen05 kernel"):
        handle.gemm_typed(tA, tB, M - 3, N, K, 1.0, a_dev, a.shape[0], b_dev, b.shape[0], 0.5, c_dev, M, np.float16,
                          CuHostArray(np.float16, shape=(M, N)), M, np.float16)
    handle.set_option(_lib.OPT_F16_ACCUMULATE, 0)


def test_check_on_call_finds_an_earlier_failure_at_the_next_call(handle, oracle):
    """B200_OPT_CHECK_ON_CALL: like the reference's exception flag, polled at every API call
    (src/init.jl:37, src/exceptions.jl:76-89 of CUDAnative.jl), a wait that ran out in an earlier,
    finished launch makes the NEXT GEMM call return B200_DEVICE_TIMEOUT without launching; the call
    after that works.  Off by default: the same sequence then stays silent until device_status."""
    from cudanative_jl_b200 import B200Error

    L = _lib.lib()
    force(handle, _lib.KERNEL_AUTO)
    a, b, c = operands(128, 128, 128, False, False, seed=6)
    want = oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c)
    handle.set_option(_lib.OPT_CHECK_ON_CALL, 1)
    assert handle.get_option(_lib.OPT_CHECK_ON_CALL) == 1
    d = run_gemm(handle, False, False, 128, 128, 128, 1.0, a, b, 1.0, c)  # a clean launch leaves nothing to find
    oracle.assert_close(d, want, "clean launch")
    oracle.assert_close(run_gemm(handle, False, False, 128, 128, 128, 1.0, a, b, 1.0, c), want, "second clean launch")
    _lib.check(L.b200_selftest_bounded_wait(handle._h, None, 1_000_000), "selftest")  # stands in for a launch whose wait ran out
    _lib.check(L.b200_stream_sync(None), "sync")
    with pytest.raises(B200Error) as e:
        run_gemm(handle, False, False, 128, 128, 128, 1.0, a, b, 1.0, c)
    assert e.value.status == _lib.DEVICE_TIMEOUT and "wait id 107" in str(e.value) and "enqueued nothing" in str(e.value)
    oracle.assert_close(run_gemm(handle, False, False, 128, 128, 128, 1.0, a, b, 1.0, c), want, "call after the report")
    handle.set_option(_lib.OPT_CHECK_ON_CALL, 0)
    _lib.check(L.b200_selftest_bounded_wait(handle._h, None, 1_000_000), "selftest")
    _lib.check(L.b200_stream_sync(None), "sync")
    handle.gemm(False, False, 128, 128, 128, 1.0, CuArray(a), 128, CuArray(b), 128, 0.0, None, 128, CuArray(d), 128)  # silent
    _lib.check(L.b200_stream_sync(None), "sync")
    assert handle.device_status()[0] == 107


def test_host_windows_that_end_with_their_buffer(handle, oracle):
    """Operands with ld > rows only own ld * (cols - 1) + rows elements: windows cut from the bottom of a
    taller host matrix (big[8:, :]) end exactly where the allocation ends.  The host-buffer entry point
    must copy them window by window, never ld * cols elements."""
    import ctypes as C

    force(handle, _lib.KERNEL_AUTO)
    M, N, K, pad = 256, 384, 128, 8
    a, b, c = operands(M, N, K, False, False, seed=96)

    def bottom_window(x):
        """x as the last rows of a taller Fortran matrix held in a buffer with not one element to spare"""
        rows, cols = x.shape
        ld = rows + pad
        flat = np.full(ld * (cols - 1) + rows + pad, np.nan, dtype=x.dtype)  # the view below starts `pad` elements in
        view = np.lib.stride_tricks.as_strided(flat[pad:], shape=(rows, cols), strides=(x.itemsize, ld * x.itemsize))
        view[...] = x
        return flat, view, ld

    fa, va, lda = bottom_window(a)
    fb, vb, ldb = bottom_window(b)
    fc, vc, ldc = bottom_window(c)
    d = np.zeros((M, N), dtype=np.float32, order="F")
    L = _lib.lib()
    _lib.check(L.b200_gemm_f16f32_host(handle._h, 0, 0, M, N, K, 1.5, va.ctypes.data, lda, vb.ctypes.data, ldb, 0.5, vc.ctypes.data, ldc,
                                       d.ctypes.data, M), "gemm_host")
    assert fa.size == lda * (K - 1) + M + pad  # the buffers really end with their windows
    oracle.assert_close(d, oracle.gemm_ref(False, False, 1.5, a, b, 0.5, c), "host windows")


@pytest.mark.parametrize("tA,tB,N", [(True, False, 384), (False, True, 1300), (False, False, 2600)])
def test_host_buffer_entry_point(handle, oracle, tA, tB, N):
    """b200_gemm_f16f32_host: host in, host out; wide N is cut into column slabs whose uploads,
    products and downloads overlap; D has padding rows that must stay untouched."""
    force(handle, _lib.KERNEL_AUTO)
    M, K = 512, 256
    a, b, c = operands(M, N, K, tA, tB, seed=95)
    d = np.full((M + 8, N), np.float32(9.0), dtype=np.float32, order="F")
    cp = padded(c, M + 8, fill=np.float32(0.0))
    handle.gemm_host(tA, tB, M, N, K, 2.0, a, a.shape[0], b, b.shape[0], 0.5, cp, M + 8, d, M + 8)
    oracle.assert_close(d[:M], oracle.gemm_ref(tA, tB, 2.0, a, b, 0.5, c), "host path")
    assert np.all(d[M:] == np.float32(9.0))
    # beta == 0 with no C at all
    d2 = np.zeros((M, N), dtype=np.float32, order="F")
    handle.gemm_host(tA, tB, M, N, K, 1.0, a, a.shape[0], b, b.shape[0], 0.0, None, M, d2, M)
    oracle.assert_close(d2, oracle.gemm_ref(tA, tB, 1.0, a, b, 0.0, None), "host path, beta = 0")
