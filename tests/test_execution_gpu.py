"""The reference's two WMMA example scripts through the ``cuda(...)`` launch mirror, and the launch keywords
that touch the device (stream, several warps and blocks)."""
import ctypes as C

import numpy as np
import pytest

from cudanative_jl_b200 import _lib, wmma
from cudanative_jl_b200.array import Array, CuArray, pointer, similar
from cudanative_jl_b200.execution import blockIdx, cuda, synchronize, threadIdx

pytestmark = pytest.mark.gpu


def isapprox(x, y, rtol):
    return np.all(np.abs(x - y) <= rtol * np.maximum(np.abs(x), np.abs(y)))


def test_high_level_example(oracle):
    from cudanative_jl_b200.examples import wmma_high_level as example
    a, b, c, d = example.main(seed=3)
    # examples/wmma/high-level.jl:49: @test all(isapprox.(a * b + 0.5 * c, d; rtol=0.01))
    assert isapprox(a.astype(np.float32) @ b.astype(np.float32) + 0.5 * c, d, 0.01)
    assert oracle.unit_close(d, oracle.wmma_unit_ref(a, b, c, beta=0.5))


def test_low_level_example(oracle):
    from cudanative_jl_b200.examples import wmma_low_level as example
    a, b, c, d = example.main(seed=4)
    # examples/wmma/low-level.jl:45
    assert isapprox(a.astype(np.float32) @ b.astype(np.float32) + c, d, 0.01)
    assert oracle.unit_close(d, oracle.wmma_unit_ref(a, b, c))


def test_launch_on_a_stream_is_asynchronous_and_ordered(oracle):
    L = _lib.lib()
    s = C.c_void_p()
    _lib.check(L.b200_stream_create(C.byref(s)), "stream")
    try:
        rand = np.random.default_rng(5)
        a = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
        b = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
        c = np.asfortranarray(rand.random((16, 16)).astype(np.float32))
        a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
        d_dev, e_dev = similar(c_dev), similar(c_dev)
        conf = wmma.Config(16, 16, 16, np.float32)

        def kernel(a_dev, b_dev, c_dev, d_dev):
            d = wmma.mma(wmma.load_a(pointer(a_dev), 16, wmma.ColMajor, conf), wmma.load_b(pointer(b_dev), 16, wmma.ColMajor, conf),
                         wmma.load_c(pointer(c_dev), 16, wmma.ColMajor, conf), conf)
            wmma.store_d(pointer(d_dev), d, 16, wmma.ColMajor, conf)

        # two dependent launches on one stream: E = A * B + (A * B + C)
        cuda(kernel, a_dev, b_dev, c_dev, d_dev, threads=32, stream=s)
        cuda(kernel, a_dev, b_dev, d_dev, e_dev, threads=32, stream=s)
        synchronize(s)
        d = Array(d_dev)
        assert oracle.unit_close(d, oracle.wmma_unit_ref(a, b, c))
        assert oracle.unit_close(Array(e_dev), oracle.wmma_unit_ref(a, b, d))
    finally:
        L.b200_stream_destroy(s)


def test_warps_and_blocks_index_their_own_tiles(oracle):
    """A 32 x 32 result as four 16 x 16 tiles: block x picks the tile row, the warp inside the block the
    tile column -- the way a hand-written WMMA kernel indexes (threadIdx / blockIdx are 1-based as in Julia)."""
    rand = np.random.default_rng(6)
    a = np.asfortranarray(rand.random((32, 16)).astype(np.float16))
    b = np.asfortranarray(rand.random((16, 32)).astype(np.float16))
    c = np.asfortranarray(rand.random((32, 32)).astype(np.float32))
    a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
    d_dev = similar(c_dev)
    conf = wmma.Config(16, 16, 16, np.float32)

    def kernel(a_dev, b_dev, c_dev, d_dev):
        ti = blockIdx().x - 1
        tj = (threadIdx().x - 1) // 32
        a_frag = wmma.load_a(pointer(a_dev) + 16 * ti, 32, wmma.ColMajor, conf)
        b_frag = wmma.load_b(pointer(b_dev) + 16 * 16 * tj, 16, wmma.ColMajor, conf)
        c_frag = wmma.load_c(pointer(c_dev) + (16 * ti + 32 * 16 * tj), 32, wmma.ColMajor, conf)
        wmma.store_d(pointer(d_dev) + (16 * ti + 32 * 16 * tj), wmma.mma(a_frag, b_frag, c_frag, conf), 32, wmma.ColMajor, conf)

    cuda(kernel, a_dev, b_dev, c_dev, d_dev, threads=64, blocks=2)
    synchronize()
    d = Array(d_dev)
    for ti in range(2):
        for tj in range(2):
            ref = oracle.wmma_unit_ref(np.asfortranarray(a[16 * ti:16 * ti + 16]), np.asfortranarray(b[:, 16 * tj:16 * tj + 16]),
                                       np.asfortranarray(c[16 * ti:16 * ti + 16, 16 * tj:16 * tj + 16]))
            assert oracle.unit_close(np.asfortranarray(d[16 * ti:16 * ti + 16, 16 * tj:16 * tj + 16]), ref)


def test_low_level_wrappers_check_their_types():
    a_dev = CuArray(np.zeros((16, 16), dtype=np.float16, order="F"))
    c_dev = CuArray(np.zeros((16, 16), dtype=np.float32, order="F"))

    def wrong_pointer(a_dev):
        wmma.llvm_wmma_load_c_col_m16n16k16_stride_f32(pointer(a_dev), 16)

    with pytest.raises(TypeError, match="expected a pointer to float32"):
        cuda(wrong_pointer, a_dev, threads=32)

    def wrong_layout(a_dev, c_dev):
        a = wmma.llvm_wmma_load_a_row_m16n16k16_stride_f16(pointer(a_dev), 16)
        b = wmma.llvm_wmma_load_b_col_m16n16k16_global_stride_f16(pointer(a_dev), 16)
        c = wmma.llvm_wmma_load_c_col_m16n16k16_stride_f32(pointer(c_dev), 16)
        wmma.llvm_wmma_mma_col_col_m16n16k16_f32_f32(a, b, c)

    with pytest.raises(TypeError, match="fragments were loaded as RowMajor"):
        cuda(wrong_layout, a_dev, c_dev, threads=32)
    synchronize()
