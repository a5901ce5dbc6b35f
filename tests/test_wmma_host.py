"""Host-side WMMA API: the exact equalities of the reference's host-only tests
(test/device/wmma.jl:156-184 of CUDAnative.jl), plus the argument errors of wmma.jl:434-477."""
import numpy as np
import pytest

from cudanative_jl_b200 import wmma
from cudanative_jl_b200.wmma import (ColMajor, Config, Fragment, MatrixA, RowMajor, Unspecified, VecElement, flatten,
                                     unflatten)

f16 = np.float16


def ntuple(f, n):
    return tuple(f(i) for i in range(1, n + 1))


def test_flattening():
    # test/device/wmma.jl:158-164
    assert flatten(5) == (5,)
    assert flatten(5.0) == (5.0,)
    assert flatten(VecElement(f16(5))) == (f16(5),)
    assert flatten(ntuple(lambda i: i, 8)) == ntuple(lambda i: i, 8)
    assert flatten(ntuple(lambda i: VecElement(f16(i)), 8)) == ntuple(lambda i: f16(i), 8)
    assert flatten(ntuple(lambda i: ntuple(lambda j: (i - 1) * 2 + j, 2), 8)) == ntuple(lambda i: i, 16)
    assert flatten(ntuple(lambda i: ntuple(lambda j: VecElement(f16((i - 1) * 2 + j)), 2), 8)) == ntuple(lambda i: f16(i), 16)


def test_unflattening():
    # test/device/wmma.jl:168-174
    assert unflatten(int, (5,)) == 5
    assert unflatten(float, (5.0,)) == 5.0
    assert unflatten((VecElement, f16), (f16(5),)) == VecElement(f16(5))
    assert unflatten((8, int), ntuple(lambda i: i, 8)) == ntuple(lambda i: i, 8)
    assert unflatten((8, (VecElement, f16)), ntuple(lambda i: f16(i), 8)) == ntuple(lambda i: VecElement(f16(i)), 8)
    assert unflatten((8, (2, int)), ntuple(lambda i: i, 16)) == ntuple(lambda i: ntuple(lambda j: (i - 1) * 2 + j, 2), 8)
    assert unflatten((8, (2, (VecElement, f16))), ntuple(lambda i: f16(i), 16)) == \
        ntuple(lambda i: ntuple(lambda j: VecElement(f16((i - 1) * 2 + j)), 2), 8)


@pytest.mark.parametrize("sz", [1, 2, 5])
@pytest.mark.parametrize("ty", [np.float16, np.float32])
def test_broadcasting_over_fragments(sz, ty):
    # test/device/wmma.jl:180-183: ty(5) .* frag and ty(5) .+ frag return fragments of the same type
    frag = Fragment(16, 16, 16, sz, ty, RowMajor, MatrixA, ntuple(lambda i: ty(i), sz))
    assert ty(5) * frag == Fragment(16, 16, 16, sz, ty, RowMajor, MatrixA, ntuple(lambda i: ty(5 * i), sz))
    assert ty(5) + frag == Fragment(16, 16, 16, sz, ty, RowMajor, MatrixA, ntuple(lambda i: ty(5 + i), sz))
    assert (ty(5) * frag).T == np.dtype(ty) and (ty(5) * frag).L is RowMajor


def test_fragment_indexing_and_types():
    frag = Fragment(16, 16, 16, 3, np.float32, ColMajor, MatrixA, (1.0, 2.0, 3.0))
    assert frag[0] == 1.0 and frag[-1] == 3.0 and len(frag) == 3 and frag.x == (1.0, 2.0, 3.0)
    assert frag != Fragment(16, 16, 16, 3, np.float32, RowMajor, MatrixA, (1.0, 2.0, 3.0))


def test_config_repr_and_shape_check():
    conf = Config[16, 16, 16, np.float32]
    assert repr(conf) == "Config{16,16,16,float32}"
    assert conf == Config(16, 16, 16, np.float32)
    with pytest.raises(ValueError, match=r"Invalid shape for WMMA: \(M, N, K\) = \(8, 16, 16\)"):
        wmma._check_shape(Config(8, 16, 16, np.float32))  # wmma.jl:450-456


def test_invalid_layout_and_type_messages():
    with pytest.raises(ValueError, match="Invalid layout for WMMA"):
        wmma._layout_code(Unspecified)  # wmma.jl:442-448: only row / col load and store
    with pytest.raises(ValueError, match="Invalid element type for WMMA"):
        wmma._frag_elems("a", np.float64)
    with pytest.raises(ValueError, match="Invalid type float32 for matrix a"):
        wmma._frag_elems("a", np.float32)  # wmma.jl:469-476
    assert wmma._frag_elems("a", np.float16) == 16 and wmma._frag_elems("c", np.float32) == 8  # wmma.jl:413-420


def test_cuhostarray_retries_allocation_after_gc(monkeypatch, pkg):
    """src/array.jl:23-29: an allocation that fails for lack of memory is retried once after a
    garbage collection.  Exercised against a stand-in for the library (no GPU needed)."""
    import ctypes as C
    from cudanative_jl_b200 import _lib, array

    calls = {"malloc": 0, "gc": 0}

    class FakeLib:
        def b200_malloc(self, out, nbytes):
            calls["malloc"] += 1
            if calls["malloc"] == 1:
                return _lib.CUDA_ERROR
            C.cast(out, C.POINTER(C.c_void_p))[0] = 4096
            return _lib.OK

        def b200_last_error(self):
            return b"cudaMalloc(dptr, bytes ? bytes : 1): cudaErrorMemoryAllocation (out of memory)"

        def b200_status_string(self, s):
            return b"B200_CUDA_ERROR"

        def b200_free(self, p):
            return _lib.OK

    import gc
    monkeypatch.setattr(_lib, "lib", lambda: FakeLib())
    monkeypatch.setattr(gc, "collect", lambda *a: calls.__setitem__("gc", calls["gc"] + 1) or 0)
    arr = array.CuHostArray(np.float32, shape=(16, 16))
    assert arr.ptr == 4096 and calls == {"malloc": 2, "gc": 1}
    arr.ptr = None  # nothing real to free
