"""The C-ABI shared library loads and exports every symbol include/b200wmma.h declares."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200wmma.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("b200_gemm_f16f32", "b200_gemm_f16f32_host", "b200_wmma_16x16x16", "b200_wmma_load",
                 "b200_wmma_mma", "b200_wmma_store_d", "b200_wmma_fill_c", "b200_wmma_bcast", "b200_create"):
        assert must in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in b200wmma.h but not exported"


def test_binding_covers_the_header(pkg):
    assert sorted(pkg._lib.SIGNATURES) == declared_symbols()


def test_status_strings(lib, pkg):
    assert lib.b200_status_string(pkg._lib.OK) == b"B200_OK"
    assert lib.b200_status_string(pkg._lib.DEVICE_TIMEOUT) == b"B200_DEVICE_TIMEOUT"
    assert lib.b200_status_string(99) == b"B200_UNKNOWN_STATUS"
    assert lib.b200_version() >= 100


def test_argument_errors_need_no_gpu(lib, pkg):
    # null handle / null out pointer are rejected before any CUDA call
    assert lib.b200_create(None, 0) == pkg._lib.INVALID_ARG
    assert b"out is null" in lib.b200_last_error()
    assert lib.b200_gemm_f16f32(None, None, 0, 0, 1, 1, 1, 1.0, None, 1, None, 1, 0.0, None, 1, None, 1) == pkg._lib.INVALID_ARG
    assert lib.b200_wmma_16x16x16(None, 0, 7, 0, 0, 0, 1, 1, 1, 0, 0.0, 0, 0.0, None, 16, None, 16, None, 16, None, 16) == pkg._lib.INVALID_ARG
    assert b"Invalid layout for WMMA".lower() in lib.b200_last_error().lower()
    assert lib.b200_wmma_load(None, 0, 0, 1, None, 16, None) == pkg._lib.INVALID_ARG  # Float32 A fragment
    assert lib.b200_set_option(None, 0, 0) == pkg._lib.INVALID_ARG


def test_no_device_is_reported_not_hidden(lib, pkg):
    # On a machine without a usable GPU the library must say so; it has no CPU path to fall to.
    n = lib.b200_device_count()
    if n > 0:
        return
    h = C.c_void_p()
    rc = lib.b200_create(C.byref(h), 0)
    assert rc in (pkg._lib.NO_DEVICE, pkg._lib.CUDA_ERROR)
    assert h.value is None


def test_header_is_plain_c(tmp_path):
    """The ABI header must compile as C (it is what a Julia / Go / Rust FFI generator would read)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        import pytest
        pytest.skip("no C compiler")
    src = tmp_path / "use.c"
    src.write_text('#include "b200wmma.h"\nint main(void) { b200_handle* h = 0; return b200_destroy(h) == B200_OK ? 0 : 1; }\n')
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", str(HEADER.parent), "-c", str(src),
                        "-o", str(tmp_path / "use.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
