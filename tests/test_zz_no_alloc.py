"""The allocation-free split-K entry point (b200_gemm_f16f32_splitk_static) against the regular
entry point.

It exists for callers that cannot allocate device memory at the moment they need a product -- code
under an allocator lock or inside a pool callback, loops that promised no driver allocations after
start-up, plug-ins that only ever get fixed buffers from their host.  Its scratch (partial products
and status word) is a 16 MiB array inside the library image, shared by every call on a device, so
the test makes two calls in a row with different problems and checks that neither sees the other's
leftovers.  Collected last on purpose (file name): if it fails under ``-x`` every other test has
already run."""
import ctypes as C

import numpy as np
import pytest

from cudanative_jl_b200 import _lib
from cudanative_jl_b200.array import Array, CuArray, CuHostArray
from helpers import operands

pytestmark = pytest.mark.gpu


def static_gemm(lib, tA, tB, M, N, K, alpha, a_dev, lda, b_dev, ldb, beta, c_dev, d_dev, split_k, sync=1):
    return lib.b200_gemm_f16f32_splitk_static(None, int(tA), int(tB), M, N, K, alpha, a_dev.ptr, lda, b_dev.ptr, ldb, beta,
                                              c_dev.ptr if c_dev is not None else None, M, d_dev.ptr, M, split_k, sync)


def test_two_calls_in_a_row_match_the_regular_entry_point(lib, handle, oracle):
    cases = [
        # (tA, tB, M, N, K, alpha, beta, split_k, seed): a skinny product first, whose partials fill
        # most of the static array, then a smaller, differently shaped one that reuses it
        (False, False, 4096, 128, 4096, 1.0, 0.0, 4, 201),
        (True, False, 640, 200, 1000, 2.0, 0.5, 3, 202),
    ]
    for (tA, tB, M, N, K, alpha, beta, split_k, seed) in cases:
        a, b, c = operands(M, N, K, tA, tB, seed=seed)
        a_dev, b_dev = CuArray(a), CuArray(b)
        c_dev = CuArray(c) if beta != 0.0 else None
        d_static = CuArray(np.full((M, N), np.float32(-1.0), dtype=np.float32, order="F"))
        rc = static_gemm(lib, tA, tB, M, N, K, alpha, a_dev, a.shape[0], b_dev, b.shape[0], beta, c_dev, d_static, split_k)
        assert rc == _lib.OK, lib.b200_last_error().decode()
        # the regular entry point with the same split
        handle.set_option(_lib.OPT_FORCE_KERNEL, _lib.KERNEL_TCGEN05)
        handle.set_option(_lib.OPT_CTA_PAIR, 1)
        handle.set_option(_lib.OPT_SPLIT_K, split_k)
        d_regular = CuHostArray(np.float32, shape=(M, N))
        handle.gemm(tA, tB, M, N, K, alpha, a_dev, a.shape[0], b_dev, b.shape[0], beta, c_dev, M, d_regular, M)
        got, want = Array(d_static), Array(d_regular)
        assert handle.device_status()[0] == 0
        oracle.assert_close(got, want, "static vs regular entry point")
        oracle.assert_close(got, oracle.gemm_ref(tA, tB, alpha, a, b, beta, c if beta != 0.0 else None), "static vs oracle")


def test_asynchronous_form_and_limits(lib, oracle):
    M, N, K = 256, 256, 512
    a, b, c = operands(M, N, K, False, False, seed=203)
    a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
    d_dev = CuHostArray(np.float32, shape=(M, N))
    assert static_gemm(lib, False, False, M, N, K, 1.0, a_dev, M, b_dev, K, 1.0, c_dev, d_dev, 2, sync=0) == _lib.OK
    _lib.check(lib.b200_stream_sync(None), "sync")
    oracle.assert_close(Array(d_dev), oracle.gemm_ref(False, False, 1.0, a, b, 1.0, c), "asynchronous call")
    # partials beyond the 16 MiB array are refused, with a message that names the limit
    big_m, big_n = 16384, 512
    assert lib.b200_gemm_f16f32_splitk_static(None, 0, 0, big_m, big_n, 256, 1.0, a_dev.ptr, big_m, b_dev.ptr, 256, 0.0, None,
                                              big_m, d_dev.ptr, big_m, 2, 1) == _lib.INVALID_ARG
    assert b"static scratch holds 16777216" in lib.b200_last_error()
    # argument checks
    assert static_gemm(lib, False, False, M, N, K, 1.0, a_dev, M, b_dev, K, 1.0, c_dev, d_dev, 1) == _lib.INVALID_ARG
    assert static_gemm(lib, False, False, M, N, K, 1.0, a_dev, M, b_dev, K, 1.0, None, d_dev, 2) == _lib.INVALID_ARG


def test_status_accessor_reports_a_wait_that_ran_out(lib):
    """The asynchronous form cannot return a time-out itself; b200_static_status is how such a caller
    learns of one.  A warp that waits 1 ms on a barrier nothing signals makes the case (no fault, no
    endless loop), the accessor reports it once and the word is clear afterwards."""
    code, block, detail = C.c_int(-1), C.c_int(-1), C.c_int(-1)
    _lib.check(lib.b200_static_status(C.byref(code), C.byref(block), C.byref(detail)), "static_status")
    assert code.value == 0
    _lib.check(lib.b200_static_selftest_bounded_wait(None, 1_000_000), "selftest")
    _lib.check(lib.b200_stream_sync(None), "sync")
    _lib.check(lib.b200_static_status(C.byref(code), C.byref(block), C.byref(detail)), "static_status")
    assert (code.value, block.value) == (107, 0)
    _lib.check(lib.b200_static_status(C.byref(code), C.byref(block), C.byref(detail)), "static_status")
    assert code.value == 0
    assert lib.b200_static_selftest_bounded_wait(None, 10) == _lib.INVALID_ARG
    # a product through the same array right afterwards is unaffected
    M, N, K = 256, 128, 512
    a, b, c = operands(M, N, K, False, False, seed=204)
    d_dev = CuHostArray(np.float32, shape=(M, N))
    assert static_gemm(lib, False, False, M, N, K, 1.0, CuArray(a), M, CuArray(b), K, 0.0, None, d_dev, 2) == _lib.OK


def test_no_device_memory_is_taken_after_the_warm_up(lib, oracle):
    """What the entry point exists for: after b200_static_warmup (address lookup, kernel loading) calls of
    any shape class leave the device's free memory exactly where it was -- no cudaMalloc, no growth of
    a driver pool.  Two different problems, two calls each."""
    import torch

    torch.cuda.init()
    _lib.check(lib.b200_static_warmup(), "static_warmup")
    cases = [(False, False, 2048, 128, 2048, 4, 211), (True, False, 512, 512, 1024, 2, 212)]
    staged = []
    for (tA, tB, M, N, K, split_k, seed) in cases:
        a, b, c = operands(M, N, K, tA, tB, seed=seed)
        staged.append((tA, tB, M, N, K, split_k, a, b, c, CuArray(a), CuArray(b), CuArray(c), CuHostArray(np.float32, shape=(M, N))))
    _lib.check(lib.b200_stream_sync(None), "sync")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(2):
        for (tA, tB, M, N, K, split_k, a, b, c, a_dev, b_dev, c_dev, d_dev) in staged:
            assert static_gemm(lib, tA, tB, M, N, K, 1.0, a_dev, a.shape[0], b_dev, b.shape[0], 1.0, c_dev, d_dev, split_k, sync=0) == _lib.OK
    _lib.check(lib.b200_stream_sync(None), "sync")
    code = C.c_int(-1)
    _lib.check(lib.b200_static_status(C.byref(code), None, None), "static_status")
    assert code.value == 0
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before, f"device free memory moved by {free_before - free_after} bytes across four calls"
    for (tA, tB, M, N, K, split_k, a, b, c, a_dev, b_dev, c_dev, d_dev) in staged:
        oracle.assert_close(Array(d_dev), oracle.gemm_ref(tA, tB, 1.0, a, b, 1.0, c), "after the memory check")
