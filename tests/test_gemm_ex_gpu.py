"""bfloat16 operands and strided batches through the C ABI (b200_gemm_ex, b200_gemm_strided_batched)
against the CPU oracle.

Neither exists in the reference (its WMMA types are Float16 / Float32 and its kernels one tile,
src/device/cuda/wmma.jl:11-37, examples/wmma/high-level.jl:30-46); the acceptance is the same as for
the Float16 GEMM: float32 sgemm on the rounded inputs, relative Frobenius error <= 1e-3 and
|D - ref| <= 1e-2 * (|ref| + 1) elementwise (oracle.assert_close)."""
import numpy as np
import pytest

from cudanative_jl_b200 import B200Error, _lib, rng
from cudanative_jl_b200.array import Array, CuArray
from cudanative_jl_b200.bfloat16 import BFloat16, round_to_bf16, widen_bf16

pytestmark = pytest.mark.gpu

LAYOUTS = [(False, False), (True, False), (False, True), (True, True)]
BF16_NAN = np.uint16(0x7FC0)


def force(handle, kernel=_lib.KERNEL_AUTO, tile_n=0, pair=0, split_k=0):
    handle.set_option(_lib.OPT_FORCE_KERNEL, kernel)
    handle.set_option(_lib.OPT_TILE_N, tile_n)
    handle.set_option(_lib.OPT_CTA_PAIR, pair)
    handle.set_option(_lib.OPT_SPLIT_K, split_k)


def store(values32: np.ndarray, elem) -> np.ndarray:
    """float32 values -> the array as it lies in memory for element type `elem`."""
    if elem is BFloat16:
        return round_to_bf16(values32)
    return values32.astype(elem)


def value(stored: np.ndarray, elem, oracle) -> np.ndarray:
    """stored array -> the float32 values it stands for (bfloat16 through the oracle's own conversion,
    not the library's host helper that prepared the inputs)."""
    if elem is BFloat16:
        return oracle.bf16_widen(stored)
    return stored.astype(np.float32)


def storage_dtype(elem):
    return np.uint16 if elem is BFloat16 else np.dtype(elem)


def nan_of(elem):
    return BF16_NAN if elem is BFloat16 else storage_dtype(elem).type(np.nan)


def sentinel_of(elem):
    """A recognisable finite value (-7.25 is exact in every type used here)."""
    return round_to_bf16(np.float32(-7.25)).reshape(())[()] if elem is BFloat16 else storage_dtype(elem).type(-7.25)


def one_problem(seed, M, N, K, tA, tB, ab, c_type):
    """Stored A, B, C of one matrix of a batch (column-major 2-D arrays)."""
    a_shape = (K, M) if tA else (M, K)
    b_shape = (N, K) if tB else (K, N)
    a = store(rng.matrix(seed, 0, *a_shape, rng.NORMAL, K ** -0.5, np.float32), ab)
    b = store(rng.matrix(seed, 1, *b_shape, rng.NORMAL, 1.0, np.float32), ab)
    c = store(rng.matrix(seed, 2, M, N, rng.UNIFORM, 1.0, np.float32), c_type)
    return a, b, c


def pack(mats, ld, stride, elem, fill):
    """Lay 2-D matrices out as a batch: matrix i starts at element i * stride, columns ld apart;
    everything between holds `fill`."""
    rows, cols = mats[0].shape
    span = ld * (cols - 1) + rows
    flat = np.full(stride * (len(mats) - 1) + span if stride else span, fill, dtype=storage_dtype(elem))
    for i, m in enumerate(mats if stride else mats[:1]):
        for j in range(cols):
            flat[i * stride + j * ld: i * stride + j * ld + rows] = m[:, j]
    return flat


def unpack(flat, rows, cols, ld, stride, batch):
    out = []
    for i in range(batch):
        out.append(np.stack([flat[i * stride + j * ld: i * stride + j * ld + rows] for j in range(cols)], axis=1))
    return out


def run_batch(handle, oracle, tA, tB, M, N, K, batch, *, ab=np.float16, c_type=np.float32, d_type=np.float32, alpha=1.25,
              beta=0.5, ld_pad=8, gap=64, repeat_a=False, repeat_b=False, odd_stride=False, seed=300, expect_kernel=None):
    probs = [one_problem(seed + i, M, N, K, tA, tB, ab, c_type) for i in range(batch)]
    if repeat_a:
        probs = [(probs[0][0], p[1], p[2]) for p in probs]
    if repeat_b:
        probs = [(p[0], probs[0][1], p[2]) for p in probs]
    a_rows, a_cols = probs[0][0].shape
    b_rows, b_cols = probs[0][1].shape

    def ld_of(rows):  # a padding that is a multiple of 8 keeps every leading dimension TMA-addressable
        return (rows + 7) // 8 * 8 + ld_pad if ld_pad % 8 == 0 else rows + ld_pad

    lda, ldb = ld_of(a_rows), ld_of(b_rows)
    ldc = ldd = ld_of(M)
    sa = 0 if repeat_a else lda * a_cols + gap + (3 if odd_stride else 0)
    sb = 0 if repeat_b else ldb * b_cols + gap
    sc, sd = ldc * N + gap, ldd * N + gap
    A = pack([p[0] for p in probs], lda, sa, ab, nan_of(ab))
    B = pack([p[1] for p in probs], ldb, sb, ab, nan_of(ab))
    Cm = pack([p[2] for p in probs], ldc, sc, c_type, nan_of(c_type)) if beta != 0.0 else None
    sent = sentinel_of(d_type)
    D0 = np.full(sd * (batch - 1) + ldd * N, sent, dtype=storage_dtype(d_type))
    d_dev = CuArray(D0)
    handle.gemm_strided_batched(tA, tB, M, N, K, alpha, CuArray(A), lda, sa, CuArray(B), ldb, sb, ab, beta,
                                CuArray(Cm) if Cm is not None else None, ldc, sc, c_type, d_dev, ldd, sd, d_type, batch)
    _lib.check(_lib.lib().b200_stream_sync(None), "sync")
    code, block, detail = handle.device_status()
    assert code == 0, f"device wait {code} ran out in block {block} (detail {detail})"
    if expect_kernel is not None:
        assert handle.last_launch()["kernel"] == expect_kernel
    flat = Array(d_dev)
    got = unpack(flat, M, N, ldd, sd, batch)
    written = np.zeros(flat.shape, dtype=bool)
    for i in range(batch):
        for j in range(N):
            written[i * sd + j * ldd: i * sd + j * ldd + M] = True
    assert np.all(flat[~written] == sent), "wrote outside the D matrices"
    for i, (a, b, c) in enumerate(probs):
        ref = oracle.gemm_ref(tA, tB, alpha, value(a, ab, oracle), value(b, ab, oracle), beta,
                              value(c, c_type, oracle) if beta != 0.0 else None)
        d = value(got[i], d_type, oracle)
        if d_type is BFloat16:
            # One rounding to nearest even on the way out.  Half an ulp of 8 significant bits is 2e-3
            # of the value, more than the acceptance allows in the Frobenius norm, so the yardstick is
            # the oracle's result rounded the same way: equal except where the two binary32 results
            # straddle a rounding boundary (one ulp).
            ref_rounded = oracle.bf16_widen(oracle.bf16_round(ref))
            assert np.max(np.abs(d - ref_rounded) / (np.abs(ref) + 1)) <= 2.0 ** -7
            ref = ref_rounded
        oracle.assert_close(d, ref, f"matrix {i} of {batch}: tA={tA} tB={tB} {M}x{N}x{K}")
    return handle.last_launch()


# ------------------------------------------------------------------------------------------- bfloat16

@pytest.mark.parametrize("kernel", [_lib.KERNEL_TCGEN05, _lib.KERNEL_SIMPLE])
@pytest.mark.parametrize("tA,tB", LAYOUTS)
def test_bfloat16_operands(handle, oracle, kernel, tA, tB):
    """bfloat16 A and B (range of binary32, 8 significant bits), binary32 C and D.  The inputs span
    magnitudes binary16 cannot hold, so reading them as binary16 would not pass."""
    force(handle, kernel)
    M, N, K = 392, 264, 520
    a, b, c = one_problem(41, M, N, K, tA, tB, BFloat16, np.float32)
    a = round_to_bf16(widen_bf16(a) * np.float32(2.0 ** 20))  # exact rescaling: far beyond binary16's 65504
    d_dev = CuArray(np.full((M, N), -3.0, dtype=np.float32, order="F"))
    handle.gemm_ex(tA, tB, M, N, K, 2.0 ** -20, CuArray(a), a.shape[0], CuArray(b), b.shape[0], BFloat16, 0.5, CuArray(c), M,
                   np.float32, d_dev, M, np.float32)
    d = Array(d_dev)
    assert handle.device_status()[0] == 0
    assert handle.last_launch()["kernel"] == kernel
    oracle.assert_close(d, oracle.gemm_ref(tA, tB, 2.0 ** -20, oracle.bf16_widen(a), oracle.bf16_widen(b), 0.5, c),
                        f"bf16 tA={tA} tB={tB}")


@pytest.mark.parametrize("tile_n,pair,split_k", [(256, 2, 0), (128, 1, 0), (64, 1, 0), (256, 1, 3), (128, 2, 2)])
def test_bfloat16_tiles_and_split_k(handle, oracle, tile_n, pair, split_k):
    force(handle, _lib.KERNEL_TCGEN05, tile_n=tile_n, pair=pair, split_k=split_k)
    info = run_batch(handle, oracle, True, False, 520, 392, 456, 1, ab=BFloat16, c_type=BFloat16, d_type=BFloat16,
                     expect_kernel=_lib.KERNEL_TCGEN05)
    assert info["tile_n"] == tile_n and info["cta_pair"] == pair and info["split_k"] == max(split_k, 1)


@pytest.mark.parametrize("c_type,d_type", [(np.float32, BFloat16), (BFloat16, np.float32), (BFloat16, np.float16),
                                           (np.float16, BFloat16), (BFloat16, BFloat16)])
@pytest.mark.parametrize("kernel", [_lib.KERNEL_TCGEN05, _lib.KERNEL_SIMPLE])
def test_bfloat16_c_and_d(handle, oracle, c_type, d_type, kernel):
    """Every mix of 16-bit and 32-bit C / D with bfloat16 among them: same-size pairs update the
    staged tile in place, mixed sizes take the read-all / write-all epilogue."""
    force(handle, kernel)
    run_batch(handle, oracle, False, False, 264, 200, 136, 1, ab=np.float16, c_type=c_type, d_type=d_type,
              expect_kernel=kernel)


def test_bfloat16_fill_matches_host_generator(handle):
    """b200_fill_bf16 rounds the counter-based values exactly as the host helper does."""
    rows, cols, ld = 70, 9, 72
    dev = CuArray(np.zeros((ld, cols), dtype=np.uint16, order="F"))
    _lib.check(_lib.lib().b200_fill_bf16(None, dev.ptr, rows, cols, ld, 5, 1, 0, rng.NORMAL, 0.25), "fill")
    _lib.check(_lib.lib().b200_stream_sync(None), "sync")
    got = Array(dev)
    want = round_to_bf16(rng.matrix(5, 1, rows, cols, rng.NORMAL, 0.25, np.float32))
    assert np.array_equal(got[:rows], want) and np.all(got[rows:] == 0)


# ------------------------------------------------------------------------------------------- batches

@pytest.mark.parametrize("tA,tB", LAYOUTS)
def test_batch_one_launch(handle, oracle, tA, tB):
    """Aligned strides: the whole batch is one tensor-core launch; gaps between matrices and the rows
    behind each leading dimension hold NaN on the input side and must stay untouched on the output side."""
    force(handle)
    info = run_batch(handle, oracle, tA, tB, 264, 200, 136, 5, expect_kernel=_lib.KERNEL_TCGEN05)
    assert info["split_k"] == 1


@pytest.mark.parametrize("tile_n,pair", [(256, 2), (128, 2), (256, 1), (64, 1)])
def test_batch_tile_shapes(handle, oracle, tile_n, pair):
    force(handle, _lib.KERNEL_TCGEN05, tile_n=tile_n, pair=pair)
    info = run_batch(handle, oracle, True, False, 520, 328, 200, 3, expect_kernel=_lib.KERNEL_TCGEN05)
    assert info["tile_n"] == tile_n and info["cta_pair"] == pair


def test_batch_more_units_than_ctas(handle, oracle):
    """Many small matrices: every CTA walks through several matrices, so the C prefetch and the
    accumulator hand-over cross matrix boundaries."""
    force(handle)
    handle.set_option(_lib.OPT_MAX_CTAS, 24)
    try:
        info = run_batch(handle, oracle, False, False, 128, 64, 192, 150, gap=0, ld_pad=0,
                         expect_kernel=_lib.KERNEL_TCGEN05)
        assert info["ctas"] == 24
    finally:
        handle.set_option(_lib.OPT_MAX_CTAS, 0)


def test_batch_types(handle, oracle):
    force(handle)
    run_batch(handle, oracle, True, False, 264, 136, 200, 4, ab=BFloat16, c_type=np.float32, d_type=BFloat16,
              expect_kernel=_lib.KERNEL_TCGEN05)
    run_batch(handle, oracle, False, True, 264, 136, 200, 4, ab=np.float16, c_type=np.float16, d_type=np.float16,
              expect_kernel=_lib.KERNEL_TCGEN05)


def test_batch_without_c(handle, oracle):
    force(handle)
    run_batch(handle, oracle, False, False, 200, 72, 64, 6, beta=0.0, expect_kernel=_lib.KERNEL_TCGEN05)


def test_batch_ragged_rows(handle, oracle):
    """M % 4 != 0: the last rows of every matrix go to the plain kernel (one batched launch), the
    rest to the tensor-core kernel."""
    force(handle)
    run_batch(handle, oracle, False, False, 267, 136, 128, 4, expect_kernel=_lib.KERNEL_TCGEN05)
    run_batch(handle, oracle, True, True, 267, 136, 128, 4, d_type=np.float16, c_type=np.float16,
              expect_kernel=_lib.KERNEL_TCGEN05)


def test_batch_repeated_operand(handle, oracle):
    """Stride 0 repeats a matrix for the whole batch (one B for many A): no third tensor-map
    dimension can say that, so the matrices are multiplied one launch each."""
    force(handle)
    run_batch(handle, oracle, False, False, 264, 200, 136, 3, repeat_b=True, expect_kernel=_lib.KERNEL_TCGEN05)
    run_batch(handle, oracle, True, False, 264, 200, 136, 3, repeat_a=True, expect_kernel=_lib.KERNEL_TCGEN05)


def test_batch_unaligned_stride(handle, oracle):
    """A stride that is no multiple of 16 bytes: matrices 1, 3, ... of A are not TMA-addressable; each
    matrix picks its own kernel."""
    force(handle)
    run_batch(handle, oracle, False, False, 264, 72, 136, 4, odd_stride=True)


def test_batch_plain_kernel(handle, oracle):
    force(handle, _lib.KERNEL_SIMPLE)
    for (tA, tB) in LAYOUTS:
        run_batch(handle, oracle, tA, tB, 150, 70, 99, 3, ld_pad=3, gap=5, expect_kernel=_lib.KERNEL_SIMPLE)


def test_batch_argument_checks(handle):
    force(handle)
    buf = CuArray(np.zeros(4096, dtype=np.float32))

    def call(**kw):
        args = dict(M=16, N=16, K=16, stride_a=256, stride_b=256, stride_c=256, stride_d=256, batch=2, ab=np.float16,
                    c_type=np.float32, d_type=np.float32)
        args.update(kw)
        handle.gemm_strided_batched(False, False, args["M"], args["N"], args["K"], 1.0, buf, 16, args["stride_a"], buf, 16,
                                    args["stride_b"], args["ab"], 0.0, None, 16, args["stride_c"], args["c_type"], buf, 16,
                                    args["stride_d"], args["d_type"], args["batch"])

    call(batch=0)  # nothing to do
    with pytest.raises(B200Error, match="negative batch"):
        call(batch=-1)
    with pytest.raises(B200Error, match="overlap"):
        call(stride_d=255)
    with pytest.raises(B200Error, match="negative batch stride"):
        call(stride_a=-1)
    with pytest.raises(B200Error, match="Float16 or bfloat16"):
        call(ab=np.float32)
    with pytest.raises(TypeError):
        call(d_type=np.float64)
    L = _lib.lib()
    rc = L.b200_gemm_ex(handle._h, None, 0, 0, 16, 16, 16, 1.0, buf.ptr, 16, buf.ptr, 16, _lib.F32, 0.0, None, 16, _lib.F32,
                        buf.ptr, 16, _lib.F32)
    assert rc == _lib.INVALID_ARG and b"A and B must be Float16 or bfloat16" in L.b200_last_error()
    rc = L.b200_gemm_ex(handle._h, None, 0, 0, 16, 16, 16, 1.0, buf.ptr, 16, buf.ptr, 16, _lib.F16, 0.0, None, 16, 7,
                        buf.ptr, 16, _lib.F32)
    assert rc == _lib.INVALID_ARG
    _lib.check(L.b200_stream_sync(None), "sync")
