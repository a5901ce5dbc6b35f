"""The CUDA path on the committed fixtures of tests/golden/ (inputs AND expected outputs stored; made by
tests/golden/make_golden.py from the CPU oracle): the 16x16x16 unit of benchmark config 1, the cut-down
config 3, and a small bfloat16 batch."""
from pathlib import Path

import numpy as np
import pytest

from cudanative_jl_b200 import _lib, wmma
from cudanative_jl_b200.array import Array, CuArray, CuHostArray
from cudanative_jl_b200.bfloat16 import BFloat16
from cudanative_jl_b200.wmma import RowMajor
from helpers import run_gemm

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("lowering", [wmma.LOWER_WARP, wmma.LOWER_TCGEN05])
def test_unit_fixture(oracle, lowering):
    g = np.load(GOLDEN / "config1_unit.npz")
    a, b, c = (np.asfortranarray(g[k]) for k in "abc")
    d_dev = CuHostArray(np.float32, shape=(16, 16))
    wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(c), d_dev, lowering=lowering)
    wmma.synchronize()
    assert oracle.unit_close(Array(d_dev), g["d"])
    wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(c), d_dev, beta=0.5, lowering=lowering)
    wmma.synchronize()
    assert oracle.unit_close(Array(d_dev), g["d_half_c"])
    d16_dev = CuHostArray(np.float16, shape=(16, 16))
    wmma.wmma_16x16x16(CuArray(a), CuArray(b), CuArray(np.asfortranarray(c.astype(np.float16))), d16_dev, a_layout=RowMajor,
                       b_layout=RowMajor, c_layout=RowMajor, d_layout=RowMajor, alpha=np.float16(0.75), beta=np.float16(0.25),
                       lowering=lowering)
    wmma.synchronize()
    d16 = Array(d16_dev)
    assert d16.dtype == np.float16 and oracle.unit_close(d16, g["d_rowmajor_f16"])


@pytest.mark.parametrize("kernel", [_lib.KERNEL_AUTO, _lib.KERNEL_TCGEN05, _lib.KERNEL_SIMPLE])
def test_config3_small_fixture(handle, oracle, kernel):
    g = np.load(GOLDEN / "config3_small.npz")
    a, b, c = (np.asfortranarray(g[k]) for k in "abc")
    K, M = a.shape
    N = b.shape[1]
    handle.set_option(_lib.OPT_FORCE_KERNEL, kernel)
    d = run_gemm(handle, True, False, M, N, K, 2.0, a, b, 0.5, c)
    assert handle.last_launch()["kernel"] == (_lib.KERNEL_SIMPLE if kernel == _lib.KERNEL_SIMPLE else _lib.KERNEL_TCGEN05)
    oracle.assert_close(d, g["d"], "vs stored sgemm result")
    oracle.assert_close(d, g["d64"], "vs stored double-accumulation result")


@pytest.mark.parametrize("d_type", [np.float32, BFloat16])
def test_bfloat16_batch_fixture(handle, oracle, d_type):
    g = np.load(GOLDEN / "bf16_batch_small.npz")
    M, K = g["a0"].shape
    N = g["b0"].shape[1]
    flat = lambda name: np.concatenate([np.asfortranarray(g[f"{name}{i}"]).ravel(order="F") for i in range(2)])  # noqa: E731
    d_dev = CuArray(np.zeros(2 * M * N, dtype=np.uint16 if d_type is BFloat16 else np.float32))
    handle.gemm_strided_batched(False, False, M, N, K, 1.25, CuArray(flat("a")), M, M * K, CuArray(flat("b")), K, K * N, BFloat16,
                                0.5, CuArray(flat("c")), M, M * N, np.float32, d_dev, M, M * N, d_type, 2)
    _lib.check(_lib.lib().b200_stream_sync(None), "sync")
    assert handle.device_status()[0] == 0
    assert handle.last_launch()["kernel"] == _lib.KERNEL_TCGEN05
    out = Array(d_dev)
    for i in range(2):
        d = out[i * M * N:(i + 1) * M * N].reshape((M, N), order="F")
        if d_type is BFloat16:
            # equal to the stored, once-rounded result except where the binary32 values straddle a rounding boundary
            want = oracle.bf16_widen(g[f"d{i}_bf16"])
            got = oracle.bf16_widen(d)
            assert np.max(np.abs(got - want) / (np.abs(want) + 1)) <= 2.0 ** -7
            oracle.assert_close(got, want, f"matrix {i}, bfloat16 D")
        else:
            oracle.assert_close(d, g[f"d{i}"], f"matrix {i}")
