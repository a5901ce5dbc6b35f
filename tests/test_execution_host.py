"""Launch conventions of ``cuda(...)`` (the mirror of ``@cuda``, src/execution.jl of CUDAnative.jl) that
need no GPU: keywords and their errors, the ``config`` callback, kernel caching, thread / block indices."""
import numpy as np
import pytest

from cudanative_jl_b200 import B200Error, execution as ex, wmma
from cudanative_jl_b200.execution import Dim3, blockDim, blockIdx, cuda, cufunction, gridDim, threadIdx


def test_defaults_are_one_thread_one_block_default_stream():
    seen = []

    def kernel(x):
        seen.append((x, threadIdx(), blockIdx(), blockDim(), gridDim(), ex.current_stream()))

    cuda(kernel, 7)
    assert seen == [(7, Dim3(1, 1, 1), Dim3(1, 1, 1), Dim3(1, 1, 1), Dim3(1, 1, 1), None)]
    with pytest.raises(RuntimeError):
        threadIdx()  # only defined inside a launch


def test_body_runs_once_per_warp_with_julia_indices():
    seen = []

    def kernel():
        seen.append((blockIdx().x, blockIdx().y, threadIdx().x, threadIdx().y))

    cuda(kernel, threads=(32, 3), blocks=(2, 2))
    # 3 warps per block (x = 32 lanes, y = 1..3), 4 blocks; indices are 1-based
    assert len(seen) == 12
    assert sorted(set(s[:2] for s in seen)) == [(1, 1), (1, 2), (2, 1), (2, 2)]
    assert sorted(set(s[2:] for s in seen)) == [(1, 1), (1, 2), (1, 3)]
    seen.clear()
    cuda(kernel, threads=96)
    assert [s[2] for s in seen] == [1, 33, 65]  # first thread of each warp


def test_unknown_keyword_is_refused_like_the_macro_does():
    # src/execution.jl:64-67: throw(ArgumentError("Unsupported keyword argument '$key'"))
    with pytest.raises(TypeError, match="Unsupported keyword argument 'thread'"):
        cuda(lambda: None, thread=32)
    cuda(lambda: None, threads=32, blocks=1, shmem=0, stream=None, cooperative=False, maxregs=64, name="k")
    with pytest.raises(B200Error, match="dynamic parallelism"):
        cuda(lambda: None, dynamic=True)
    with pytest.raises(ValueError):
        cuda(lambda: None, threads=2048)
    with pytest.raises(ValueError):
        cuda(lambda: None, blocks=0)


def test_config_callback_sees_the_kernel_and_overrides_the_launch():
    # src/execution.jl:209-215: config(kernel) returns some of threads / blocks / shmem
    seen = []

    def kernel(n):
        seen.append((blockDim().x, gridDim().x))

    def config(k):
        assert isinstance(k, ex.HostKernel) and k.f is kernel
        return dict(threads=64, blocks=3)

    cuda(kernel, 5, threads=32, config=config)
    assert seen == [(64, 3)] * 6  # 2 warps x 3 blocks
    with pytest.raises(TypeError, match="returned by config"):
        cuda(kernel, 5, config=lambda k: dict(warps=2))


def test_kernels_are_cached_per_function_and_argument_types():
    def kernel(x):
        pass

    k1 = cufunction(kernel, (int,))
    assert cufunction(kernel, (int,)) is k1
    assert cufunction(kernel, (float,)) is not k1
    cuda(kernel, 3)
    cuda(kernel, 4)
    assert k1.launches == 2
    with pytest.raises(TypeError, match="do not match"):
        k1(2.5)
    with pytest.raises(TypeError, match="Unsupported keyword"):
        cufunction(kernel, (int,), fastmath=True)


def test_stream_is_visible_inside_the_body_only():
    seen = []
    cuda(lambda: seen.append(ex.current_stream()), threads=32, stream=1234)
    assert seen == [1234] and ex.current_stream() is None


def test_wmma_operation_without_a_full_warp_is_refused():
    conf = wmma.Config(16, 16, 16, np.float32)

    def kernel():
        wmma.fill_c(np.float32(0), conf)

    with pytest.raises(B200Error, match="whole warps"):
        cuda(kernel)  # threads defaults to 1


def test_low_level_wrapper_names_exist():
    # the 24 + 12 + 16 wrappers of src/device/cuda/wmma.jl:104-257
    names = wmma.LLVM_WRAPPERS
    assert len(names) == 52 and len(set(names)) == 52
    assert sum(n.startswith("llvm_wmma_load_") for n in names) == 24
    assert sum(n.startswith("llvm_wmma_store_d_") for n in names) == 12
    assert sum(n.startswith("llvm_wmma_mma_") for n in names) == 16
    for n in ("llvm_wmma_load_a_col_m16n16k16_stride_f16", "llvm_wmma_load_c_row_m16n16k16_global_stride_f32",
              "llvm_wmma_store_d_col_m16n16k16_shared_stride_f16", "llvm_wmma_mma_row_col_m16n16k16_f16_f32"):
        assert callable(getattr(wmma, n))
    with pytest.raises(B200Error, match="shared-memory address"):
        wmma.llvm_wmma_load_a_col_m16n16k16_shared_stride_f16(0, 16)
