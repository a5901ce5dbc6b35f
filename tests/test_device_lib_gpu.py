"""The linkable device-side fragment library (csrc/wmma_device_lib.cu): all 52 `extern "C" __device__`
functions exercised from a foreign kernel (tests/device_lib_harness.cu) that links against the
relocatable object, checked against the CPU oracle.  Mirrors test/device/wmma.jl:13-151 of
CUDAnative.jl (llvm_wmma_load / store with all-42 tiles, llvm_wmma_mma over layouts and types)."""
import ctypes as C
import itertools
import re
from pathlib import Path

import numpy as np
import pytest

from cudanative_jl_b200 import rng
from cudanative_jl_b200.array import Array, CuArray

ROOT = Path(__file__).resolve().parent.parent
HARNESS = ROOT / "tests" / "libdevice_harness.so"
PTX = ROOT / "cudanative.jl_b200" / "b200wmma_device.ptx"


def reference_names():
    """The 52 wrapper names src/device/cuda/wmma.jl:104-257 generates, with the b200_ prefix."""
    names = []
    for mat, types in (("a", ["f16"]), ("b", ["f16"]), ("c", ["f16", "f32"])):
        for lay, as_, ty in itertools.product(["col", "row"], ["", "_global", "_shared"], types):
            names.append(f"b200_wmma_load_{mat}_{lay}_m16n16k16{as_}_stride_{ty}")
    for lay, as_, ty in itertools.product(["col", "row"], ["", "_global", "_shared"], ["f16", "f32"]):
        names.append(f"b200_wmma_store_d_{lay}_m16n16k16{as_}_stride_{ty}")
    for al, bl, d, c in itertools.product(["col", "row"], ["col", "row"], ["f16", "f32"], ["f16", "f32"]):
        names.append(f"b200_wmma_mma_{al}_{bl}_m16n16k16_{d}_{c}")
    return names


def test_ptx_exports_the_52_reference_names(pkg):
    pkg.build.build_device_lib()
    text = PTX.read_text()
    exported = set(re.findall(r"\.visible \.func[^\n]*?\b(b200_wmma_[a-z0-9_]+)\(", text)) | \
        set(re.findall(r"\.visible \.func\s+(b200_wmma_[a-z0-9_]+)\(", text))
    names = reference_names()
    assert len(names) == 52
    assert set(names) <= exported, sorted(set(names) - exported)
    assert ".target sm_100a" in text


def _ptx_body(text, name):
    i = text.index(name + "(")
    return text[i:text.index("\n}\n", i)]


@pytest.mark.parametrize("ty", ["f16", "f32"])
@pytest.mark.parametrize("lay", ["col", "row"])
def test_ptx_uses_the_address_space_of_the_variant(pkg, lay, ty):
    """test/device/wmma.jl:254-291 checks that stores through a global / shared pointer compile to the
    state-space forms of the instruction, not the generic one.  Same property here: the _global and
    _shared variants load and store with ld/st.global and ld/st.shared, the unsuffixed ones generically."""
    pkg.build.build_device_lib()
    text = PTX.read_text()
    mem = lambda body: set(re.findall(r"\b(?:st|ld)\.(global|shared)\.", body))
    generic = lambda body: re.search(r"\b(?:st|ld)\.(?:b16|u16|f32|b32|u32)\b", body) is not None
    for op, mat in (("store_d", ""), ("load_c", "")):
        base = f"b200_wmma_{op}_{lay}_m16n16k16"
        assert mem(_ptx_body(text, f"{base}_global_stride_{ty}")) == {"global"}
        assert mem(_ptx_body(text, f"{base}_shared_stride_{ty}")) == {"shared"}
        body = _ptx_body(text, f"{base}_stride_{ty}")
        assert mem(body) == set() and generic(body)


@pytest.fixture(scope="module")
def harness(pkg):
    pkg.build.build_device_lib()
    lib = C.CDLL(str(HARNESS))
    lib.harness_run.restype = C.c_int
    lib.harness_run.argtypes = [C.c_int] * 7 + [C.c_void_p] * 4
    lib.harness_run_block16x2.restype = C.c_int
    lib.harness_run_block16x2.argtypes = [C.c_int] * 7 + [C.c_void_p] * 4
    return lib


@pytest.mark.gpu
@pytest.mark.parametrize("as_", [0, 1, 3], ids=["generic", "global", "shared"])
def test_all_layouts_and_types_through_the_linked_functions(harness, oracle, as_):
    """16 layout combinations x (C, D) types, per address space: every load, mma and store variant."""
    for i, (ar, br, cr, dr, ct, dt) in enumerate(itertools.product([0, 1], [0, 1], [0, 1], [0, 1],
                                                                    [np.float16, np.float32], [np.float16, np.float32])):
        a = rng.matrix(500 + i, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
        b = rng.matrix(500 + i, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
        c = rng.matrix(500 + i, 2, 16, 16, rng.UNIFORM, 1.0, ct)
        a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
        d_dev = CuArray(np.zeros((16, 16), dtype=dt, order="F"))
        rc = harness.harness_run(ar, br, cr, dr, int(ct == np.float16), int(dt == np.float16), as_, a_dev.ptr, b_dev.ptr,
                                 c_dev.ptr, d_dev.ptr)
        assert rc == 0, f"cudaError {rc}"
        ref = oracle.wmma_unit_ref(a, b, c, a_layout=ar, b_layout=br, c_layout=cr, d_layout=dr, d_type=dt)
        assert oracle.unit_close(Array(d_dev), ref), f"case {i}: layouts {ar}{br}{cr}{dr} C {ct.__name__} D {dt.__name__}"


@pytest.mark.gpu
@pytest.mark.parametrize("as_", [0, 1], ids=["generic", "global"])
def test_any_block_shape_like_the_reference_intrinsics(harness, oracle, as_):
    """The reference's fragment operations are warp-level instructions and work in a block of any shape;
    a kernel launched with threads = (16, 2) has lanes that are not threadIdx.x & 31.  All 16 layout
    combinations through the linked functions in such a block."""
    for i, (ar, br, cr, dr) in enumerate(itertools.product([0, 1], [0, 1], [0, 1], [0, 1])):
        a = rng.matrix(600 + i, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
        b = rng.matrix(600 + i, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
        c = rng.matrix(600 + i, 2, 16, 16, rng.UNIFORM, 1.0, np.float32)
        a_dev, b_dev, c_dev = CuArray(a), CuArray(b), CuArray(c)
        d_dev = CuArray(np.zeros((16, 16), dtype=np.float32, order="F"))
        rc = harness.harness_run_block16x2(ar, br, cr, dr, 0, 0, as_, a_dev.ptr, b_dev.ptr, c_dev.ptr, d_dev.ptr)
        assert rc == 0, f"cudaError {rc}"
        ref = oracle.wmma_unit_ref(a, b, c, a_layout=ar, b_layout=br, c_layout=cr, d_layout=dr, d_type=np.float32)
        assert oracle.unit_close(Array(d_dev), ref), f"case {i}: layouts {ar}{br}{cr}{dr} in a 16 x 2 block"


@pytest.mark.gpu
def test_load_store_identity_with_42(harness):
    """test/device/wmma.jl:13-100: tiles of 42 go through load and store unchanged (A = 0 so D = C)."""
    for as_, dr, cr in itertools.product([0, 1, 3], [0, 1], [0, 1]):
        for ty in (np.float16, np.float32):
            z = CuArray(np.zeros((16, 16), np.float16, order="F"))
            c_dev = CuArray(np.full((16, 16), 42, dtype=ty, order="F"))
            d_dev = CuArray(np.zeros((16, 16), dtype=ty, order="F"))
            assert harness.harness_run(0, 0, cr, dr, int(ty == np.float16), int(ty == np.float16), as_, z.ptr, z.ptr,
                                       c_dev.ptr, d_dev.ptr) == 0
            assert np.all(Array(d_dev) == ty(42))
